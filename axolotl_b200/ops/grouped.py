"""Grouped expert computation on CUDA: tokens sorted by expert, one pass per projection.

Each expert's rows go through the tcgen05 GEMM (bf16 weights, or NVFP4 weights dequantised by the
nvfp4 kernel right before use) with its LoRA update folded in as a K-extension. Gradients flow
through the same autograd functions as the dense layers.
"""
from __future__ import annotations

import torch

from . import functional as Fn
from .lora import _LinearFn, _LoRALinearFn


def adapters_enabled():
    from ..models.layers import adapters_enabled as f

    return f()


def _proj(x, W, A, B, scaling, r):
    if A is None:
        return _LinearFn.apply(x, W, None)
    A16 = A.detach().to(torch.bfloat16).contiguous()
    B16 = B.detach().to(torch.bfloat16).contiguous()
    return _LoRALinearFn.apply(x, W, A, B, A16, B16, float(scaling), ((0, W.shape[0], 0, r),), None)


def grouped_experts_forward(experts, x_sorted, counts):
    outs = []
    start = 0
    r = experts.lora_r
    for e, n in enumerate(counts):
        if n == 0:
            continue
        xe = x_sorted[start:start + n].contiguous()
        start += n
        Ag = Bg = Ad = Bd = None
        if experts.lora is not None and adapters_enabled():
            Ag, Bg = experts.expert_lora("gate_up", e)
            Ad, Bd = experts.expert_lora("down", e)
        gu = _proj(xe, experts.expert_weight("gate_up", e), Ag, Bg, experts.scaling, r)
        h = Fn.glu(gu, experts.act)
        outs.append(_proj(h, experts.expert_weight("down", e), Ad, Bd, experts.scaling, r))
    if not outs:
        return x_sorted.new_zeros((0, experts.H))
    return torch.cat(outs, 0)


@torch.no_grad()
def quantize_experts_nvfp4_(model):
    """Replaces the bf16 expert stacks of every MoE block by frozen NVFP4 tensors (packed nibbles,
    E4M3 block scales, fp32 per-expert scale)."""
    from ..models.moe import Experts
    from .nvfp4 import quantize_nvfp4

    for m in model.modules():
        if isinstance(m, Experts) and m.nvfp4 is None:
            q = {}
            for which, W in (("gate_up", m.gate_up_proj), ("down", m.down_proj)):
                qd, sc, pts = quantize_nvfp4(W.detach())
                q[which] = {"qdata": qd, "scale": sc, "pts": pts.reshape(-1)}
            m.nvfp4 = q
            m.gate_up_proj = None
            m.down_proj = None
    return model
