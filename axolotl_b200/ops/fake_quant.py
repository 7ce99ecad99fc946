"""Fake quantisation for quantisation-aware training (QAT): weights are rounded to the target
grid in the forward pass while gradients pass straight through to the full-precision masters.
Grids: symmetric int8 / int4 per group along the input dimension, NVFP4 (16-element blocks, E4M3
scales) and per-row FP8 E4M3. Reference: torchao-based prepare/convert in
src/axolotl/utils/quantization.py:293-422 (``qat: {weight_dtype, group_size, activation_dtype}``).
"""
from __future__ import annotations

import torch


def fake_quantize(w: torch.Tensor, weight_dtype: str = "int8", group_size: int | None = 32) -> torch.Tensor:
    """Returns the dequantised value of quantising ``w`` [N, K] (same dtype, no gradient)."""
    wd = (weight_dtype or "int8").lower()
    x = w.detach().float()
    N, K = x.shape
    if wd in ("int8", "int4"):
        qmax = 127.0 if wd == "int8" else 7.0
        g = group_size if group_size and K % group_size == 0 else K
        xg = x.view(N, K // g, g)
        scale = xg.abs().amax(-1, keepdim=True).clamp(min=1e-12) / qmax
        q = torch.clamp(torch.round(xg / scale), -qmax - 1, qmax)
        return (q * scale).view(N, K).to(w.dtype)
    if wd in ("nvfp4", "fp4"):
        from .nvfp4 import dequantize_nvfp4, quantize_nvfp4

        q, s, pts = quantize_nvfp4(x)
        return dequantize_nvfp4(q, s, pts, dtype=torch.float32).to(w.dtype) if not q.is_cuda else \
            dequantize_nvfp4(q, s, pts).to(w.dtype)
    if wd in ("fp8", "float8", "float8_e4m3fn", "fp8_e4m3"):
        scale = x.abs().amax(1, keepdim=True).clamp(min=1e-12) / 448.0
        return ((x / scale).to(torch.float8_e4m3fn).float() * scale).to(w.dtype)
    if wd in ("mxfp4",):
        g = 32
        xg = x.view(N, K // g, g)
        e = torch.floor(torch.log2(xg.abs().amax(-1, keepdim=True).clamp(min=2 ** -126))) - 2   # E8M0 shared exponent
        scale = torch.exp2(e)
        grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=x.device)
        mag = (xg / scale).abs().clamp(max=6.0)
        idx = (mag[..., None] - grid).abs().argmin(-1)
        return (grid[idx] * torch.sign(xg) * scale).view(N, K).to(w.dtype)
    if wd in ("mxfp8",):
        g = 32
        xg = x.view(N, K // g, g)
        e = torch.floor(torch.log2(xg.abs().amax(-1, keepdim=True).clamp(min=2 ** -126))) - 8   # E8M0 scale, E4M3 payload
        scale = torch.exp2(e)
        return ((xg / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * scale).view(N, K).to(w.dtype)
    raise ValueError(f"unknown QAT weight dtype '{weight_dtype}'")


class _FakeQuantAct(torch.autograd.Function):
    """Dynamic per-token activation fake-quantisation with a straight-through gradient."""

    @staticmethod
    def forward(ctx, x, kind):
        xf = x.float()
        amax = xf.abs().amax(-1, keepdim=True).clamp(min=1e-12)
        if kind == "int8":
            scale = amax / 127.0
            return (torch.clamp(torch.round(xf / scale), -128, 127) * scale).to(x.dtype)
        scale = amax / 448.0
        return ((xf / scale).to(torch.float8_e4m3fn).float() * scale).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None


def fake_quantize_activation(x: torch.Tensor, activation_dtype: str | None) -> torch.Tensor:
    """``qat.activation_dtype``: int8 or fp8 (E4M3), one scale per token row; None leaves ``x`` alone."""
    if not activation_dtype:
        return x
    ad = str(activation_dtype).lower()
    if ad in ("int8",):
        return _FakeQuantAct.apply(x, "int8")
    if ad in ("fp8", "float8", "float8_e4m3fn"):
        return _FakeQuantAct.apply(x, "fp8")
    raise ValueError(f"unknown QAT activation dtype '{activation_dtype}'")


def ste_weight(param: torch.Tensor, weight_dtype: str, group_size: int | None):
    """Tensor to feed the GEMM in place of ``param``: quantised values, gradient routed to ``param``.
    On CUDA the custom GEMM functions accumulate weight gradients into ``param._axb_grad`` (the
    optimizer's flat fp32 view); the quantised copy is handed the same view so the straight-through
    gradient lands there directly. Elsewhere the usual ``w + (q - w).detach()`` form is used."""
    wq = fake_quantize(param, weight_dtype, group_size)
    buf = getattr(param, "_axb_grad", None)
    if param.is_cuda and buf is not None:
        wq.requires_grad_(True)
        wq._axb_grad = buf
        return wq
    return param + (wq - param.detach())
