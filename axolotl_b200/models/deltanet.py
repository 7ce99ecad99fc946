"""Gated DeltaNet mixer (Qwen3-Next linear-attention layers): q / k / v pass a short causal depthwise convolution,
q and k are L2-normalised, and a matrix state S [d_k, d_v] per head follows the gated delta rule

    S_t = a_t S_{t-1} + b_t k_t (v_t - a_t S_{t-1}^T k_t)^T        o_t = S_t^T q_t / sqrt(d_k)

with a_t = exp(g_t) a learned decay and b_t = sigmoid(.) the write strength; the output goes through an RMSNorm
gated by silu(z) (the norm-then-gate kernel, ``rmsnorm_gated_*_kernel``) and the output projection. On packed token
streams neither the convolution nor the state crosses a document boundary.

Chunked evaluation (fp32 tensor contractions, differentiable by autograd): inside a chunk with cumulative log decay G
the corrected values U solve the unit lower-triangular system (I + L) U = b (V - exp(G) K S0), where
L_ij = b_i exp(G_i - G_j) <k_i, k_j> for j < i. With T = (I + L)^-1 (one batched triangular solve for all chunks),
U = T(bV) - T(b exp(G) K) S0, the outputs are exp(G_i) S0^T q_i + sum_{j<=i} exp(G_i - G_j) <q_i, k_j> u_j and the
state leaves the chunk as exp(G_C) S0 + sum_j exp(G_C - G_j) k_j u_j^T; only that last recurrence is sequential.

The reference trains these layers through HF's modelling code and the flash-linear-attention kernels, with its fused
gated RMSNorm (src/axolotl/kernels/rms_norm_gated.py:36-381).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fn
from .config import ModelConfig
from .layers import FusedLinear


def gated_delta_rule(q, k, v, g, beta, chunk=64):
    """One document. q, k [L, h, dk] (already normalised, q scaled), v [L, h, dv], g [L, h] (log decay <= 0),
    beta [L, h]. Returns o [L, h, dv]."""
    L, h, dk = k.shape
    dv = v.shape[-1]
    C = min(chunk, max(L, 1))
    pad = (-L) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, 0, 0, pad)), F.pad(beta, (0, 0, 0, pad))
    n = (L + pad) // C
    q, k, v = (t.view(n, C, h, -1).permute(0, 2, 1, 3) for t in (q, k, v))            # [n, h, C, d]
    g, beta = g.view(n, C, h).permute(0, 2, 1), beta.view(n, C, h).permute(0, 2, 1)    # [n, h, C]
    G = g.cumsum(-1)
    diff = G[..., :, None] - G[..., None, :]                                           # G_i - G_j
    low = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    decay = torch.exp(diff.masked_fill(~low, float("-inf")))                           # j <= i, else 0
    kk = k @ k.transpose(-1, -2)
    Lmat = (beta[..., :, None] * kk * decay).tril(-1)
    eye = torch.eye(C, dtype=q.dtype, device=q.device)
    T = torch.linalg.solve_triangular(eye + Lmat, eye.expand(n, h, C, C), upper=False)
    W1 = T @ (beta[..., None] * v)                                                     # [n, h, C, dv]
    W2 = T @ (beta[..., None] * torch.exp(G)[..., None] * k)                           # [n, h, C, dk]
    qk = (q @ k.transpose(-1, -2)) * decay                                             # [n, h, C, C]
    eG = torch.exp(G)
    tail = torch.exp(G[..., -1:] - G)                                                  # exp(G_C - G_j)
    S = torch.zeros(h, dk, dv, dtype=q.dtype, device=q.device)
    outs = []
    for c in range(n):
        U = W1[c] - W2[c] @ S                                                          # [h, C, dv]
        outs.append((eG[c][..., None] * q[c]) @ S + qk[c] @ U)
        S = eG[c][:, -1, None, None] * S + (tail[c][..., None] * k[c]).transpose(-1, -2) @ U
    o = torch.stack(outs)                                                              # [n, h, C, dv]
    return o.permute(0, 2, 1, 3).reshape(n * C, h, dv)[:L]


def _unit_lower_inverse(Lm):
    """(I + L)^-1 for strictly lower-triangular L [..., C, C]. L is nilpotent (L^C = 0), so the Neumann series is the
    finite product (I - L)(I + L^2)(I + L^4)...: log2(C) batched matrix products instead of C steps of substitution."""
    C = Lm.shape[-1]
    eye = torch.eye(C, dtype=Lm.dtype, device=Lm.device)
    inv = eye - Lm
    P = Lm @ Lm                                      # (-L)^2 = L^2
    k = 2
    while k < C:
        inv = inv + inv @ P
        k *= 2
        if k < C:
            P = P @ P
    return inv


def _delta_layout(cu, C, device):
    """Documents padded to multiples of C and laid end to end: gather index into the token stream (one extra zero row at
    index T), position of every token in the padded layout, and the [documents, max chunks] grid of chunk numbers (the
    number of chunks = an all-zero chunk that leaves the state alone)."""
    import numpy as np

    T = int(cu[-1])
    idx, back, per_doc = [], [], []
    off = nchunks = 0
    for s, e in zip(cu[:-1], cu[1:]):
        L = int(e) - int(s)
        if L <= 0:
            continue
        n = (L + C - 1) // C
        row = np.full(n * C, T, dtype=np.int64)
        row[:L] = np.arange(int(s), int(e))
        idx.append(row)
        back.append(off + np.arange(L))
        per_doc.append(np.arange(nchunks, nchunks + n))
        off += n * C
        nchunks += n
    grid = np.full((len(per_doc), max(len(p) for p in per_doc)), nchunks, dtype=np.int64)
    for d, pch in enumerate(per_doc):
        grid[d, : len(pch)] = pch
    to = lambda a: torch.from_numpy(a).to(device)
    return to(np.concatenate(idx)), to(np.concatenate(back)), to(grid)


def _delta_packed_core(q, k, v, g, beta, idx, back, grid, C, lowp):
    T, h, dk = k.shape
    dv = v.shape[-1]

    def pad(t):
        return torch.cat([t, t.new_zeros(1, *t.shape[1:])], 0).index_select(0, idx)
    n = idx.numel() // C
    q, k, v = (pad(t).view(n, C, h, -1).permute(0, 2, 1, 3) for t in (q, k, v))          # [n, h, C, d]
    g, beta = pad(g).view(n, C, h).permute(0, 2, 1).float(), pad(beta).view(n, C, h).permute(0, 2, 1).float()
    ct = lowp if lowp is not None else q.dtype
    mm = lambda a, b: (a.to(ct) @ b.to(ct)).float()                                        # tensor-core contraction, fp32 result
    G = g.cumsum(-1)
    low = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    decay = torch.exp((G[..., :, None] - G[..., None, :]).masked_fill(~low, float("-inf")))
    Lmat = (beta[..., :, None] * mm(k, k.transpose(-1, -2)) * decay).tril(-1)
    Tm = _unit_lower_inverse(Lmat)
    W1 = mm(Tm, beta[..., None] * v.float())                                               # [n, h, C, dv]
    W2 = mm(Tm, beta[..., None] * torch.exp(G)[..., None] * k.float())                     # [n, h, C, dk]
    qk = mm(q, k.transpose(-1, -2)) * decay
    eG = torch.exp(G)
    qe = eG[..., None] * q.float()                                                         # queries with the decay since the chunk start
    kt = (torch.exp(G[..., -1:] - G)[..., None] * k.float()).transpose(-1, -2)             # keys with the decay to the chunk end
    last = eG[..., -1]                                                                     # [n, h]

    def grid_of(t, fill=0.0, dtype=None):
        """[chunks, ...] -> [chunk positions, documents, ...] (one gather up front; documents shorter than the longest read an
        all-zero chunk with decay 1 that leaves their state alone)."""
        t = torch.cat([t, torch.full((1, *t.shape[1:]), fill, dtype=t.dtype, device=t.device)], 0)
        t = t.index_select(0, grid.t().reshape(-1)).view(grid.shape[1], grid.shape[0], *t.shape[1:])
        return t.to(dtype) if dtype is not None else t
    W1g, W2g, qkg, qeg, ktg, lastg = grid_of(W1), grid_of(W2, dtype=ct), grid_of(qk, dtype=ct), grid_of(qe, dtype=ct), \
        grid_of(kt, dtype=ct), grid_of(last, 1.0)
    D = grid.shape[0]
    S = torch.zeros(D, h, dk, dv, dtype=torch.float32, device=q.device)
    outs = []
    for c in range(grid.shape[1]):                                                         # chunk by chunk, all documents at once
        Sl = S.to(ct)
        U = W1g[c] - (W2g[c] @ Sl).float()
        Ul = U.to(ct)
        outs.append((qeg[c] @ Sl).float() + (qkg[c] @ Ul).float())
        S = lastg[c][..., None, None] * S + (ktg[c] @ Ul).float()
    out = torch.stack(outs)                                                                # [positions, documents, h, C, dv]
    # back to chunk order: chunk number grid[d, c] holds out[c, d]
    flat = torch.zeros(n + 1, h, C, dv, dtype=torch.float32, device=q.device)
    flat = flat.index_copy(0, grid.t().reshape(-1), out.view(-1, h, C, dv))
    return flat[:n].permute(0, 2, 1, 3).reshape(n * C, h, dv).index_select(0, back)


def gated_delta_rule_packed(q, k, v, g, beta, cu, chunk=64, lowp=None):
    """The chunked gated delta rule for EVERY document of a packed row: the per-chunk work (Gram matrices, triangular
    solves) runs once over all chunks, the state recurrence advances all documents together, one step per chunk
    position. ``lowp``: operand dtype of the matrix products (fp32 accumulation and state)."""
    C = min(chunk, max(int(max(e - s for s, e in zip(cu[:-1], cu[1:]))), 1))
    idx, back, grid = _delta_layout(cu, C, q.device)
    return _delta_packed_core(q, k, v, g, beta, idx, back, grid, C, lowp)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ex = cfg.extra or {}
        H = cfg.hidden_size
        self.nv, self.nk = int(ex["linear_num_value_heads"]), int(ex["linear_num_key_heads"])
        self.dk, self.dv = int(ex["linear_key_head_dim"]), int(ex["linear_value_head_dim"])
        self.key_dim, self.value_dim = self.dk * self.nk, self.dv * self.nv
        self.k = int(ex.get("linear_conv_kernel_dim", 4))
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.eps = cfg.rms_norm_eps
        # Qwen3-Next lays its two input projections out per key head ([q | k | v | z] and [b | a]); Qwen3.5 has four flat
        # projections (q|k|v, z, b, a), fused into one GEMM here under their checkpoint names
        self.flat = cfg.model_type != "qwen3_next"
        if self.flat:
            self.in_proj = FusedLinear(H, [self.conv_dim, self.value_dim, self.nv, self.nv],
                                       ["in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a"], dtype=dtype, device=device)
        else:
            self.in_proj_qkvz = FusedLinear(H, [2 * self.key_dim + 2 * self.value_dim], ["in_proj_qkvz"], dtype=dtype, device=device)
            self.in_proj_ba = FusedLinear(H, [2 * self.nv], ["in_proj_ba"], dtype=dtype, device=device)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, self.k, dtype=dtype, device=device))
        self.dt_bias = nn.Parameter(torch.ones(self.nv, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=dtype, device=device))
        self.norm_weight = nn.Parameter(torch.ones(self.dv, dtype=dtype, device=device))
        self.out_proj = FusedLinear(self.value_dim, [H], ["out_proj"], dtype=dtype, device=device)
        self.window, self.use_rope = 0, False

    def _conv(self, x, positions):
        w = self.conv_weight.float()
        out = x.float() * w[:, self.k - 1]
        pos = positions.to(x.device)
        for j in range(1, self.k):
            out = out + F.pad(x.float(), (0, 0, j, 0))[: x.shape[0]] * w[:, self.k - 1 - j] * (pos >= j)[:, None]
        return F.silu(out)

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        if getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("cached decoding is not available for linear-attention layers; generate(use_cache=False)")
        if getattr(meta, "cp", False):
            raise NotImplementedError("context parallelism is not available for Gated DeltaNet layers (a chunk's transition is a full "
                                      "d_k x d_k matrix per head rather than a scalar decay; that hand-over is not built)")
        T = x.shape[0]
        r = self.nv // self.nk
        if self.flat:
            mixed, z, b, a = torch.split(self.in_proj(x), [self.conv_dim, self.value_dim, self.nv, self.nv], dim=-1)
        else:
            # the projection is laid out per key head: [q | k | v (r value heads) | z (r value heads)]
            qkvz = self.in_proj_qkvz(x).view(T, self.nk, 2 * self.dk + 2 * r * self.dv)
            q, k, v, z = torch.split(qkvz, [self.dk, self.dk, r * self.dv, r * self.dv], dim=-1)
            ba = self.in_proj_ba(x).view(T, self.nk, 2 * r)
            b, a = ba[..., :r].reshape(T, self.nv), ba[..., r:].reshape(T, self.nv)
            mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1)
        mixed = self._conv(mixed, positions)
        q, k, v = torch.split(mixed, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k, v = q.view(T, self.nk, self.dk), k.view(T, self.nk, self.dk), v.view(T, self.nv, self.dv)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * (self.dk ** -0.5)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        if r > 1:
            q, k = q.repeat_interleave(r, dim=1), k.repeat_interleave(r, dim=1)
        beta = torch.sigmoid(b.float())
        g = -torch.exp(self.A_log.float()) * F.softplus(a.float() + self.dt_bias.float())
        cu = [int(c) for c in meta.cu_seqlens_host]
        o = gated_delta_rule_packed(q, k, v, g, beta, cu, 64, torch.bfloat16 if (x.is_cuda and x.dtype == torch.bfloat16) else None)
        o = Fn.rmsnorm_gated(o.reshape(T * self.nv, self.dv).to(x.dtype), z.reshape(T * self.nv, self.dv).contiguous(),
                             self.norm_weight, self.eps)
        return self.out_proj(o.reshape(T, self.value_dim))
