"""Fused flat-buffer AdamW with device-side global-norm clipping.

All trainable parameters of a model are views into one fp32 master buffer (plus an optional bf16
shadow used by the GEMM kernels); gradients likewise. One kernel computes the squared gradient
norm, one kernel applies clip + AdamW + the bf16 re-cast: no host synchronisation per step.
Replaces ``adamw_torch_fused`` + ``clip_grad_norm_`` of the reference's HF Trainer path.
"""
from __future__ import annotations

import math

import torch

from . import _lib


def grad_sumsq(flat_grad: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Sum of squares of an fp32 buffer as a 1-element device tensor (accumulates into ``out``)."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=flat_grad.device)
    if not flat_grad.is_cuda:
        out += flat_grad.float().pow(2).sum()
        return out
    lib = _lib.cuda_lib()
    _lib.check_rc(lib.axb_sumsq(flat_grad.data_ptr(), flat_grad.numel(), out.data_ptr(),
                                _lib.stream_ptr()), "sumsq")
    return out


def adamw_step_(param, grad, exp_avg, exp_avg_sq, *, step, lr, beta1=0.9, beta2=0.999, eps=1e-8,
                weight_decay=0.0, bf16_copy=None, gnorm_sq=None, max_norm=0.0, grad_scale=1.0):
    """In-place decoupled-weight-decay Adam on flat fp32 buffers.

    ``gnorm_sq`` (device scalar: squared norm of the *unscaled* gradient) with ``max_norm > 0``
    enables clipping inside the kernel. ``grad_scale`` multiplies the gradient first (e.g.
    1 / world_size after a sum-reduce).
    """
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not param.is_cuda:
        g = grad.float() * grad_scale
        if gnorm_sq is not None and max_norm > 0:
            nrm = math.sqrt(float(gnorm_sq)) * grad_scale
            g = g * min(1.0, max_norm / (nrm + 1e-6))
        exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        param.mul_(1 - lr * weight_decay)
        param.addcdiv_(exp_avg / bc1, (exp_avg_sq / bc2).sqrt() + eps, value=-lr)
        if bf16_copy is not None:
            bf16_copy.copy_(param)
        return
    lib = _lib.cuda_lib()
    _lib.check_rc(
        lib.axb_adamw(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
                      _lib.ptr(bf16_copy), param.numel(), lr, beta1, beta2, eps, weight_decay, bc1,
                      bc2, _lib.ptr(gnorm_sq), max_norm, grad_scale, _lib.stream_ptr()),
        "adamw")
