"""Mamba-2 (state-space duality) mixer for the hybrid families (Granite 4.0-H `granitemoehybrid`, Bamba, Nemotron-H, Falcon-H1): in_proj ->
causal depthwise convolution -> selective state-space scan -> gated RMSNorm -> out_proj, on PACKED token streams:
neither the convolution nor the recurrent state crosses a document boundary.

The scan is the chunked SSD algorithm written with dense tensor contractions (fp32): inside a chunk of Q tokens the
output is a masked, decay-weighted (C B^T) product; between chunks one [heads, P, N] state per chunk is carried by a
short recurrence. Autograd differentiates the contractions. On a GPU these run as library batched GEMMs; a fused
tcgen05 scan kernel is not part of this package yet.

Context parallelism: every rank scans its contiguous chunk of the row from a zero state; the scan is linear in its
initial state, so the state that arrives from the earlier chunks of the same document is added afterwards
(``exp(cumulative decay) * C . H_in``). Every rank all-gathers (final state of its last document segment, total decay
of its chunk) once per layer and folds the chain of earlier ranks locally, so a document that spans ANY number of
chunks is exact; the convolution reads the last ``k - 1`` pre-convolution rows of the previous rank. Both exchanges
are differentiable (all-reduce of the gathered gradient).

The reference trains these models through HF's modelling code and the mamba-ssm / causal-conv1d kernels and passes
the state one hop along the ring (src/axolotl/monkeypatch/models/mamba_utils.py:53-187).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .config import ModelConfig
from .layers import FusedLinear


def ssd_chunked(xd, a, B, C, chunk=128):
    """One document. xd [L, h, P] (inputs already multiplied by dt), a [L, h] (log decay per step, <= 0),
    B, C [L, h, N]. Returns y [L, h, P] with y_t = sum_{s<=t} exp(a_{s+1} + .. + a_t) (C_t . B_s) xd_s."""
    L, h, P = xd.shape
    N = B.shape[-1]
    Q = min(chunk, max(L, 1))
    pad = (-L) % Q
    if pad:
        xd, a, B, C = (F.pad(t, (0, 0) * (t.dim() - 1) + (0, pad)) for t in (xd, a, B, C))
    nc = (L + pad) // Q
    xd, B, C = xd.view(nc, Q, h, P), B.view(nc, Q, h, N), C.view(nc, Q, h, N)
    cum = a.view(nc, Q, h).cumsum(1)                                            # [nc, Q, h]
    seg = cum[:, :, None, :] - cum[:, None, :, :]                                # [nc, i, j, h]
    causal = torch.ones(Q, Q, dtype=torch.bool, device=xd.device).tril()
    decay = torch.exp(seg.masked_fill(~causal[None, :, :, None], float("-inf")))
    G = torch.einsum("cihn,cjhn->cijh", C, B)
    y = torch.einsum("cijh,cjhp->cihp", G * decay, xd)
    if nc > 1:
        to_end = torch.exp(cum[:, -1:, :] - cum)                                 # [nc, Q, h]
        S = torch.einsum("cjhn,cjh,cjhp->chpn", B, to_end, xd)                  # state contributed by each chunk
        chunk_decay = torch.exp(cum[:, -1, :])                                   # [nc, h]
        carried, R = [], torch.zeros(h, P, N, dtype=xd.dtype, device=xd.device)
        for c in range(nc):
            carried.append(R)
            R = chunk_decay[c][:, None, None] * R + S[c]
        y = y + torch.einsum("cihn,chpn,cih->cihp", C, torch.stack(carried), torch.exp(cum))
    return y.reshape(nc * Q, h, P)[:L]


def _packed_layout(cu, Q, device):
    """Every document padded to a multiple of Q positions and laid end to end: (gather index into the token stream with
    one extra zero row at index T, index of every token in the padded layout, same-document matrix of the chunks)."""
    import numpy as np

    T = int(cu[-1])
    idx, back, doc_of_chunk = [], [], []
    off = 0
    for d, (s, e) in enumerate(zip(cu[:-1], cu[1:])):
        L = int(e) - int(s)
        if L <= 0:
            continue
        n = (L + Q - 1) // Q
        row = np.full(n * Q, T, dtype=np.int64)
        row[:L] = np.arange(int(s), int(e))
        idx.append(row)
        back.append(off + np.arange(L))
        doc_of_chunk += [d] * n
        off += n * Q
    idx, back = np.concatenate(idx), np.concatenate(back)
    doc = np.asarray(doc_of_chunk)
    same = doc[:, None] == doc[None, :]
    lower = np.tril(np.ones((len(doc), len(doc)), dtype=bool), -1)
    return (torch.from_numpy(idx).to(device), torch.from_numpy(back).to(device), torch.from_numpy(same & lower).to(device))


def _ssd_packed_core(xd, a, B, C, idx, back, pair_ok, Q, lowp):
    """xd [T, h, P], a [T, h], B / C [T, G, N] (one per GROUP of h / G heads; [T, h, N] works too). Everything is laid out
    [chunks, groups, heads-of-group, positions, ...] so that every contraction is a plain batched matrix product and the
    group-level tensors broadcast over their heads without copies; operands are converted to ``lowp`` once, up front."""
    T, h, P = xd.shape
    Gn, N = B.shape[1], B.shape[2]
    rep = h // Gn
    ct = lowp if lowp is not None else xd.dtype                                      # operand dtype of the contractions

    def pad(t):
        return torch.cat([t, t.new_zeros(1, *t.shape[1:])], 0).index_select(0, idx)
    nc = idx.numel() // Q
    x_p = pad(xd.to(ct)).view(nc, Q, Gn, rep, P).permute(0, 2, 3, 1, 4)              # [nc, G, r, Q, P]
    B_p = pad(B.to(ct)).view(nc, Q, Gn, N).permute(0, 2, 1, 3)                       # [nc, G, Q, N]
    C_p = pad(C.to(ct)).view(nc, Q, Gn, N).permute(0, 2, 1, 3)
    cum = pad(a.float()).view(nc, Q, Gn, rep).permute(0, 2, 3, 1).cumsum(-1)         # [nc, G, r, Q] fp32
    causal = torch.ones(Q, Q, dtype=torch.bool, device=xd.device).tril()
    decay = torch.exp((cum[..., :, None] - cum[..., None, :]).masked_fill(~causal, float("-inf"))).to(ct)   # [nc, G, r, i, j]
    Gm = C_p @ B_p.transpose(-1, -2)                                                 # [nc, G, i, j]: once per group
    y = ((Gm[:, :, None] * decay) @ x_p).float()                                     # [nc, G, r, Q, P]
    if nc > 1:
        to_end = torch.exp(cum[..., -1:] - cum).to(ct)                               # [nc, G, r, Q]
        S = ((x_p * to_end[..., None]).transpose(-1, -2) @ B_p[:, :, None]).float()  # [nc, G, r, P, N] state each chunk adds
        tot = cum[..., -1].reshape(nc, h)                                            # [nc, h] log decay over a chunk
        E = tot.cumsum(0) - tot                                                      # log decay from the row start to a chunk start
        # state that enters chunk c: sum over earlier chunks j of the same document of exp(E_c - E_j - tot_j) S_j
        M = torch.exp((E[:, None, :] - E[None, :, :] - tot[None, :, :]).masked_fill(~pair_ok[:, :, None], float("-inf")))
        R = (M.permute(2, 0, 1) @ S.reshape(nc, h, P * N).permute(1, 0, 2)).view(h, nc, P, N).permute(1, 0, 2, 3)
        R = R.reshape(nc, Gn, rep, P, N).to(ct)
        y = y + ((C_p[:, :, None] * torch.exp(cum).to(ct)[..., None]) @ R.transpose(-1, -2)).float()
    return y.permute(0, 3, 1, 2, 4).reshape(nc * Q, h, P).index_select(0, back)


def ssd_packed(xd, a, B, C, cu, chunk=128, lowp=None):
    """The chunked scan of EVERY document of a packed row in one batched pass (no loop over documents or chunks): chunks
    of all documents form the batch axis of the contractions, and the state a chunk receives is one masked matrix
    product over the earlier chunks of its document. ``lowp`` (e.g. bf16 on the device): operand dtype of the
    contractions (fp32 accumulation; decays and cumulative sums stay fp32). The big [chunks, Q, Q, heads] intermediates
    are recomputed in the backward pass instead of being kept."""
    Q = min(chunk, max(int(max(e - s for s, e in zip(cu[:-1], cu[1:]))), 1))
    idx, back, pair_ok = _packed_layout(cu, Q, xd.device)
    args = (xd, a, B, C, idx, back, pair_ok, Q, lowp)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (xd, a, B, C)):
        from torch.utils.checkpoint import checkpoint

        return checkpoint(_ssd_packed_core, *args, use_reentrant=False)
    return _ssd_packed_core(*args)


class _AllGatherStack(torch.autograd.Function):
    """[...] on every rank -> [world, ...]; the gradient of a rank's slice is the sum of what all ranks send back."""

    @staticmethod
    def forward(ctx, t, group, world, rank):
        ctx.group, ctx.rank = group, rank
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.stack(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g[ctx.rank], None, None, None


def cp_segments(cu, c0, c1):
    """Document pieces inside the chunk [c0, c1) as chunk-relative (lo, hi), and whether the first piece continues a
    document that started on an earlier rank."""
    segs = []
    for s, e in zip(cu[:-1], cu[1:]):
        lo, hi = max(int(s), c0), min(int(e), c1)
        if lo < hi:
            segs.append((lo - c0, hi - c0))
    starts = {int(v) for v in cu}
    return segs, (c0 > 0 and c0 not in starts)


class Mamba2Mixer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ex = cfg.extra or {}
        H = cfg.hidden_size
        if cfg.model_type == "nemotron_h":      # its own key names; the inner width is heads x head width; grouped gated norm
            self.nh, self.P = int(ex["mamba_num_heads"]), int(ex["mamba_head_dim"])
            self.G, self.N = int(ex.get("n_groups", 8)), int(ex["ssm_state_size"])
            self.k = int(ex.get("conv_kernel", 4))
            self.d_inner = self.nh * self.P
            self.chunk = int(ex.get("chunk_size", 128))
            self.norm_groups = self.G
            bias, conv_bias = bool(ex.get("use_bias", False)), bool(ex.get("use_conv_bias", True))
        else:
            self.nh, self.P = int(ex["mamba_n_heads"]), int(ex["mamba_d_head"])
            self.G, self.N = int(ex.get("mamba_n_groups", 1)), int(ex["mamba_d_state"])
            self.k = int(ex.get("mamba_d_conv", 4))
            self.d_inner = int(ex["mamba_d_ssm"]) if ex.get("mamba_d_ssm") else int(ex.get("mamba_expand", 2) * H)
            if self.d_inner != self.nh * self.P:
                raise ValueError(f"mamba_expand * hidden ({self.d_inner}) must equal mamba_n_heads * mamba_d_head ({self.nh * self.P})")
            self.chunk = int(ex.get("mamba_chunk_size", 256))
            self.norm_groups = 1
            bias, conv_bias = bool(ex.get("mamba_proj_bias", False)), bool(ex.get("mamba_conv_bias", True))
        # Falcon-H1: scalar on the mixer input, one multiplier per section of the in_proj output (z | x | B | C | dt),
        # the gated norm is optional, grouped, and may run before the gate; out_proj has its own bias switch
        self.in_multiplier, self.has_norm, self.norm_before_gate, out_bias = 1.0, True, False, bias
        mup = None
        if cfg.model_type == "falcon_h1":
            self.in_multiplier = float(ex.get("ssm_in_multiplier") or 1.0)
            self.has_norm = bool(ex.get("mamba_rms_norm", False))
            self.norm_before_gate = bool(ex.get("mamba_norm_before_gate", True))
            self.norm_groups = self.G
            out_bias = bool(ex.get("projectors_bias", False))
            zm = [float(v) for v in (ex.get("ssm_multipliers") or [1.0] * 5)]
            gn = self.G * self.N
            mup = torch.cat([torch.full((n,), v) for n, v in zip((self.d_inner, self.d_inner, gn, gn, self.nh), zm)])
        self.register_buffer("mup_vector", mup.to(device) if (mup is not None and device is not None) else mup, persistent=False)
        self.conv_dim = self.d_inner + 2 * self.G * self.N
        lim = ex.get("time_step_limit") or (0.0, float("inf"))
        self.dt_limit = (float(lim[0]), float(lim[1]))
        self.eps = cfg.rms_norm_eps
        self.in_proj = FusedLinear(H, [self.d_inner + self.conv_dim + self.nh], ["in_proj"], bias=bias, dtype=dtype, device=device)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_dim, self.k, dtype=dtype, device=device))
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_dim, dtype=dtype, device=device)) if conv_bias else None
        self.dt_bias = nn.Parameter(torch.ones(self.nh, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, self.nh + 1, dtype=torch.float32, device=device)).to(dtype))
        self.D = nn.Parameter(torch.ones(self.nh, dtype=dtype, device=device))
        self.norm_weight = nn.Parameter(torch.ones(self.d_inner, dtype=dtype, device=device)) if self.has_norm else None
        self.out_proj = FusedLinear(self.d_inner, [H], ["out_proj"], bias=out_bias, dtype=dtype, device=device)
        self.window, self.use_rope = 0, False

    def _conv(self, x, positions, halo=None):
        """Causal depthwise convolution over the token axis that reads zeros before the start of a document; ``halo``
        holds the k - 1 rows that precede x (context parallelism: the previous rank's last rows)."""
        w = self.conv_weight.float()
        out = x.float() * w[:, self.k - 1]
        pos = positions.to(x.device)
        T = x.shape[0]
        xp = F.pad(x.float(), (0, 0, self.k - 1, 0)) if halo is None else torch.cat([halo.float(), x.float()], 0)
        for j in range(1, self.k):
            shifted = xp[self.k - 1 - j: self.k - 1 - j + T]
            out = out + shifted * w[:, self.k - 1 - j] * (pos >= j)[:, None]
        if self.conv_bias is not None:
            out = out + self.conv_bias.float()
        return F.silu(out)

    def _scan_cp(self, xd, a, B, C, cu, meta):
        """The scan of this rank's chunk with the state that earlier chunks of the same document hand over."""
        segs, continues = cp_segments(cu, meta.c0, meta.c1)
        ys = [ssd_chunked(xd[lo:hi], a[lo:hi], B[lo:hi], C[lo:hi], self.chunk) for lo, hi in segs]
        lo, hi = segs[-1]
        cum_last = a[lo:hi].cumsum(0)                                            # [L, h]
        S = torch.einsum("lhn,lh,lhp->hpn", B[lo:hi], torch.exp(cum_last[-1:] - cum_last), xd[lo:hi])
        # the incoming state passes THROUGH this chunk only when the chunk is one piece of one document
        through = torch.exp(cum_last[-1]) if (len(segs) == 1 and continues) else torch.zeros_like(cum_last[-1])
        packed = torch.cat([S.reshape(-1), through])
        allr = _AllGatherStack.apply(packed, meta.ctx.group, meta.world, meta.rank)     # [world, h*P*N + h]
        if not continues:        # (zero-weight use: the backward pass of every rank must reach the collective)
            ys[0] = ys[0] + allr.sum() * 0.0
            return torch.cat(ys, 0)
        n_state = S.numel()
        H_in = torch.zeros_like(S)
        for j in range(meta.rank):                                              # fold the chain of earlier ranks
            H_in = allr[j, :n_state].view_as(S) + allr[j, n_state:][:, None, None] * H_in
        lo, hi = segs[0]
        cum = a[lo:hi].cumsum(0)
        ys[0] = ys[0] + torch.exp(cum)[..., None] * torch.einsum("lhn,hpn->lhp", C[lo:hi], H_in)
        return torch.cat(ys, 0)

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        if getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("cached decoding is not available for state-space layers; generate(use_cache=False)")
        T = x.shape[0]
        zxbcdt = self.in_proj(x * self.in_multiplier if self.in_multiplier != 1.0 else x)
        if self.mup_vector is not None:
            zxbcdt = zxbcdt * self.mup_vector.to(zxbcdt.dtype)
        z, xBC, dt = torch.split(zxbcdt, [self.d_inner, self.conv_dim, self.nh], dim=-1)
        cp = getattr(meta, "cp", False)
        halo = None
        if cp:      # the convolution's look-back across the chunk border
            tails = _AllGatherStack.apply(xBC[T - (self.k - 1):], meta.ctx.group, meta.world, meta.rank)
            # (rank 0 keeps a zero-weight use of the gathered rows: every rank's backward pass must reach the collective)
            halo = tails[meta.rank - 1] if meta.rank > 0 else tails[0] * 0.0
        xBC = self._conv(xBC, positions, halo)
        xs, B, C = torch.split(xBC, [self.d_inner, self.G * self.N, self.G * self.N], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias.float()).clamp(self.dt_limit[0], self.dt_limit[1])
        A = -torch.exp(self.A_log.float())
        xs = xs.view(T, self.nh, self.P)
        rep = self.nh // self.G
        B, C = B.view(T, self.G, self.N), C.view(T, self.G, self.N)
        xd, a = xs * dt[..., None], A[None] * dt
        cu = [int(v) for v in meta.cu_seqlens_host]
        if cp:
            y = self._scan_cp(xd, a, B.repeat_interleave(rep, dim=1), C.repeat_interleave(rep, dim=1), cu, meta)
        else:
            y = ssd_packed(xd, a, B, C, cu, min(self.chunk, 128), torch.bfloat16 if (x.is_cuda and x.dtype == torch.bfloat16) else None)
        y = y + self.D.float()[None, :, None] * xs
        y = y.reshape(T, self.d_inner)
        if not (self.has_norm and self.norm_before_gate):
            y = y * F.silu(z.float())                                            # gate first, then the norm
        if self.has_norm:
            if self.norm_groups > 1:                                             # one RMS per group of channels
                yg = y.view(T, self.norm_groups, -1)
                y = (yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + self.eps)).reshape(T, self.d_inner)
            else:
                y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + self.eps)
            y = self.norm_weight.float() * y
            if self.norm_before_gate:
                y = y * F.silu(z.float())
        return self.out_proj(y.to(x.dtype))
