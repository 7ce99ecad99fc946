"""Gated short convolution (LFM2's non-attention operator): ``y = out_proj(C * conv(B * x))`` where B, C and x are
three slices of one input projection and ``conv`` is a causal depthwise convolution over a handful of positions.
On packed token streams the convolution reads zeros before the start of a document; under context parallelism the
previous rank's last rows arrive as a halo, exactly like the convolution of the Mamba-2 mixer.

The reference trains LFM2 through HF's modelling code with sample packing (src/axolotl/monkeypatch/multipack.py:12-70
lists `lfm2` / `lfm2_moe`); HF's fast path calls the causal-conv1d package.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .config import ModelConfig
from .layers import FusedLinear


class ShortConv(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        ex = cfg.extra or {}
        H = cfg.hidden_size
        self.H, self.k = H, int(ex.get("conv_L_cache") or 3)
        bias = bool(ex.get("conv_bias", False))
        self.in_proj = FusedLinear(H, [3 * H], ["in_proj"], bias=bias, dtype=dtype, device=device)
        self.out_proj = FusedLinear(H, [H], ["out_proj"], bias=bias, dtype=dtype, device=device)
        self.conv_weight = nn.Parameter(torch.empty(H, self.k, dtype=dtype, device=device))
        self.conv_bias = nn.Parameter(torch.zeros(H, dtype=dtype, device=device)) if bias else None
        self.window, self.use_rope = 0, False

    def forward(self, x, positions, inv_freq, attn_scale, meta):
        if getattr(meta, "kv_cache", None) is not None:
            raise NotImplementedError("cached decoding is not available for short-convolution layers; generate(use_cache=False)")
        T = x.shape[0]
        B, C, u = self.in_proj(x).split(self.H, dim=-1)
        bx = (B * u).float()
        halo = None
        if getattr(meta, "cp", False):
            from .mamba import _AllGatherStack

            tails = _AllGatherStack.apply(bx[T - (self.k - 1):], meta.ctx.group, meta.world, meta.rank)
            halo = tails[meta.rank - 1] if meta.rank > 0 else tails[0] * 0.0
        xp = torch.nn.functional.pad(bx, (0, 0, self.k - 1, 0)) if halo is None else torch.cat([halo.float(), bx], 0)
        w = self.conv_weight.float()
        pos = positions.to(x.device)
        out = bx * w[:, self.k - 1]
        for j in range(1, self.k):
            out = out + xp[self.k - 1 - j: self.k - 1 - j + T] * w[:, self.k - 1 - j] * (pos >= j)[:, None]
        if self.conv_bias is not None:
            out = out + self.conv_bias.float()
        return self.out_proj((C.float() * out).to(x.dtype))
