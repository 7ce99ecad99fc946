"""Dynamic sparse attention (GLM-5 `glm_moe_dsa`, the DeepSeek-V3.2 design): latent attention whose every query
attends only the ``index_topk`` keys that a light "lightning indexer" scores highest.

* The indexer has its own small projections (``wq_b`` from the query bottleneck, one shared 128-wide key per
  position with a LayerNorm, per-head mixing weights). Its scores are
  ``sum_h w[s, h] * relu(q[s, h] . k[t])``; on a GPU one tcgen05 kernel produces the [positions, keys] matrix
  without ever holding the per-head scores (``csrc/indexer.cu``). It is not differentiated (the selection is a
  constant of the graph, as in HF's modelling code).
* A document no longer than ``index_topk`` selects every causal key, so it runs through the ordinary wide-head
  varlen attention kernels. Longer documents take the dense-mask form: blocks of queries against all their causal
  keys with the unselected ones masked out, recomputed in the backward pass. (The reference's gather kernel is
  enabled on sm_90 / sm_120 only; on this architecture it runs the dense-mask form too:
  src/axolotl/integrations/kernels/libs/glm_dsa/dispatch.py:26-46, 97-160.)

Reference: src/axolotl/integrations/kernels/libs/glm_dsa/indexer.py:38-176 (fused scorer + top-k),
attention_mla_absorb.py:91-565 (sparse gather attention), patch.py:1-284.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import _lib
from ..ops import functional as Fn
from .config import ModelConfig
from .layers import FusedLinear
from .mla import MLAttention

QUERY_CHUNK = 8192     # rows of the score matrix held at once (fp32 [chunk, keys])
MASK_BLOCK = 512       # query rows per block of the dense-mask attention


def indexer_scores_ref(q, k, w, causal_off=0):
    """q [Lq, H, D], k [Lk, D], w [Lq, H] -> [Lq, Lk] fp32, -inf where key t > s + causal_off."""
    s = torch.einsum("shd,td->sht", q.float(), k.float())
    out = torch.einsum("sht,sh->st", F.relu(s), w.float())
    Lq, Lk = out.shape
    vis = torch.arange(Lk, device=out.device)[None, :] <= (torch.arange(Lq, device=out.device)[:, None] + causal_off)
    return out.masked_fill(~vis, float("-inf"))


def indexer_scores(q, k, w, causal_off=0):
    """Scores of one document (or of a block of its queries against keys [0, Lk))."""
    Lq, H, D = q.shape
    Lk = k.shape[0]
    if not (q.is_cuda and q.dtype == torch.bfloat16 and D == 128 and H in (32, 64, 128)):
        return indexer_scores_ref(q, k, w, causal_off)
    q = q.contiguous()
    k = k.contiguous()
    w = w.float().contiguous()
    out = torch.full((Lq, Lk), float("-inf"), dtype=torch.float32, device=q.device)
    _lib.check_rc(_lib.cuda_lib().axb_indexer_scores(q.data_ptr(), D, k.data_ptr(), D, w.data_ptr(), out.data_ptr(), Lk,
                                                     Lq, Lk, H, D, causal_off, _lib.status_word(q.device).data_ptr(),
                                                     _lib.stream_ptr()), "indexer_scores")
    return out


def _masked_block(qb, kk, vv, sel, q0, scale):
    """qb [B, H, D], kk [n, H, D], vv [n, H, Dv], sel [B, topk] selected key indices (may hold future keys: masked here)."""
    B, n = qb.shape[0], kk.shape[0]
    keep = torch.zeros(B, n, dtype=torch.bool, device=qb.device)
    keep.scatter_(1, sel.clamp(max=n - 1), True)
    keep &= torch.arange(n, device=qb.device)[None, :] <= (q0 + torch.arange(B, device=qb.device))[:, None]
    sc = torch.einsum("bhd,nhd->hbn", qb, kk).float() * scale
    sc = sc.masked_fill(~keep[None], float("-inf"))
    pr = sc.softmax(-1).to(vv.dtype)
    return torch.einsum("hbn,nhd->bhd", pr, vv)


def topk_masked_attention(q, k, v, topk_idx, scale, block=MASK_BLOCK):
    """One document. q, k [L, H, D], v [L, H, Dv], topk_idx [L, topk] (int64). Causal attention restricted to the
    selected keys, block of queries by block; every block is recomputed in the backward pass."""
    L = q.shape[0]
    outs = []
    for b0 in range(0, L, block):
        b1 = min(b0 + block, L)
        args = (q[b0:b1], k[:b1], v[:b1], topk_idx[b0:b1], b0, scale)
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            outs.append(checkpoint(_masked_block, *args, use_reentrant=False))
        else:
            outs.append(_masked_block(*args))
    return torch.cat(outs, 0)


class LightningIndexer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ex = cfg.extra or {}
        self.H, self.D = int(ex.get("index_n_heads") or 32), int(ex.get("index_head_dim") or 128)
        self.d_rope = int(ex.get("qk_rope_head_dim") or 64)
        self.topk = int(ex.get("index_topk") or 2048)
        q_rank = int(ex["q_lora_rank"])
        self.wq_b = FusedLinear(q_rank, [self.H * self.D], ["wq_b"], dtype=dtype, device=device)
        self.wk = FusedLinear(cfg.hidden_size, [self.D], ["wk"], dtype=dtype, device=device)
        self.k_norm_weight = nn.Parameter(torch.ones(self.D, dtype=dtype, device=device))
        self.k_norm_bias = nn.Parameter(torch.zeros(self.D, dtype=dtype, device=device))
        self.weights_proj = FusedLinear(cfg.hidden_size, [self.H], ["weights_proj"], dtype=dtype, device=device)
        self.softmax_scale = self.D ** -0.5
        for prm in self.parameters():            # the selection is not differentiated: nothing here is trained
            prm.requires_grad_(False)

    def _rope(self, t, positions, inv_freq, attn_scale):
        """Split-half rotation of the first d_rope dimensions of [T, n, D]."""
        d = self.d_rope
        ang = positions.float()[:, None] * inv_freq.float()[None, :]          # [T, d/2]
        cos = (torch.cat([ang, ang], -1).cos() * attn_scale)[:, None, :]
        sin = (torch.cat([ang, ang], -1).sin() * attn_scale)[:, None, :]
        x = t[..., :d].float()
        rot = torch.cat([-x[..., d // 2:], x[..., : d // 2]], -1)
        return torch.cat([(x * cos + rot * sin).to(t.dtype), t[..., d:]], -1)

    @torch.no_grad()
    def select(self, x, q_resid, positions, inv_freq, attn_scale, cu):
        """Per document longer than ``topk``: the selected key indices [L, topk] (document-relative); None for the
        documents where every causal key is selected."""
        T = x.shape[0]
        if all(e - s <= self.topk for s, e in zip(cu[:-1], cu[1:])):
            return [None] * (len(cu) - 1)
        q = self._rope(self.wq_b(q_resid).view(T, self.H, self.D), positions, inv_freq, attn_scale)
        k = F.layer_norm(self.wk(x).float(), (self.D,), self.k_norm_weight.float(), self.k_norm_bias.float(), 1e-6).to(x.dtype)
        k = self._rope(k[:, None, :], positions, inv_freq, attn_scale)[:, 0]
        w = self.weights_proj(x).float() * (self.H ** -0.5) * self.softmax_scale
        out = []
        for s, e in zip(cu[:-1], cu[1:]):
            if e - s <= self.topk:
                out.append(None)
                continue
            sel = []
            for c0 in range(s, e, QUERY_CHUNK):
                c1 = min(c0 + QUERY_CHUNK, e)
                sc = indexer_scores(q[c0:c1], k[s:c1], w[c0:c1], causal_off=c0 - s)
                kk = min(self.topk, sc.shape[1])
                idx = sc.topk(kk, dim=-1).indices
                if kk < self.topk:                      # (a chunk that ends before topk keys exist)
                    idx = F.pad(idx, (0, self.topk - kk), value=0)
                sel.append(idx)
            out.append(torch.cat(sel, 0))
        return out


class SparseMLAttention(MLAttention):
    """Latent attention with the top-k key selection of the lightning indexer."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__(cfg, dtype, device)
        if not self.q_lora_rank:
            raise ValueError("glm_moe_dsa: the indexer reads the query bottleneck, q_lora_rank must be set")
        self.indexer = LightningIndexer(cfg, dtype, device)

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        if getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("KV-cache decoding is not available for latent attention; generate(use_cache=False)")
        if getattr(meta, "cp", False):
            raise NotImplementedError("context parallelism is not available for dynamic sparse attention")
        cu = [int(v) for v in meta.cu_seqlens_host]
        q_resid = self.q_a_layernorm.plain(self.q_a_proj(x))
        sel = self.indexer.select(x, q_resid, positions, inv_freq, attn_scale, cu)
        qkv = self.pre(x, positions, inv_freq, attn_scale, q_resid=q_resid)
        dense = self.core(qkv, meta).view(x.shape[0], self.Hq, self.Dv)     # exact for every document within topk keys
        if all(s is None for s in sel):
            return self.o_proj(dense.reshape(x.shape[0], self.Hq * self.Dv))
        T = x.shape[0]
        nq = self.Hq * self.D
        q, k = qkv[:, :nq].view(T, self.Hq, self.D), qkv[:, nq:2 * nq].view(T, self.Hq, self.D)
        v = qkv[:, 2 * nq:].view(T, self.Hq, self.Dv)
        outs = []
        for (s, e), idx in zip(zip(cu[:-1], cu[1:]), sel):
            if e <= s:
                continue
            # (the rows the varlen kernel produced for a longer document are dropped: its queries see selected keys only)
            outs.append(dense[s:e] if idx is None else topk_masked_attention(q[s:e], k[s:e], v[s:e], idx, self.scale))
        return self.o_proj(torch.cat(outs, 0).reshape(T, self.Hq * self.Dv))
