"""Fused LoRA linear: ``y = x W^T + s * (x A^T) B^T`` with the low-rank product folded into the
base GEMM as a K-extension (one extra accumulation block in TMEM), and a backward pass that
never materialises ``W + s B A``.

Several projections that share the same input (q/k/v, gate/up) are handled as ONE GEMM over the
row-concatenated weight: ``A_cat`` stacks the A matrices, ``B_cat`` is block diagonal.

Covers what the reference implements as LoRA_MLP / LoRA_QKV / LoRA_O autograd functions on top
of cuBLAS (src/axolotl/kernels/lora.py:283-1209, 1623-1769).
"""
from __future__ import annotations

import torch

from .gemm import gemm, glu_fusable, pick_splits


SKINNY_SPLITS = int(__import__("os").environ.get("AXB_LORA_SKINNY_SPLITS", "0"))


def skinny_gemm(a, b, *, trans_b=False, alpha=1.0):
    """``alpha * a @ op(b)^T`` for an output only a few columns wide ([T, R], R = adapter rank): with one
    128-row tile per CTA such a GEMM has T/128 CTAs, too few to pull the wide operand at memory speed, so
    the K range can be split over several CTAs (fp32 atomics into a zeroed [T, R] buffer, cast once).
    Off by default (AXB_LORA_SKINNY_SPLITS=2|4 enables it): the Llama-3-8B LoRA step measured 306.6 /
    307.3 / 307.6 ms with 2 / 4 / no splits on one B200, i.e. no difference beyond run-to-run noise."""
    T = a.shape[0]
    R = b.shape[1] if trans_b else b.shape[0]
    K = a.shape[1]
    tiles = (T + 127) // 128
    sp = SKINNY_SPLITS
    if not a.is_cuda or sp <= 1 or tiles * sp > 1024 or K < 2048:
        return gemm(a, b, trans_b=trans_b, alpha=alpha)
    acc = torch.zeros((T, R), dtype=torch.float32, device=a.device)
    gemm(a, b, trans_b=trans_b, alpha=alpha, out=acc, accumulate=True, splits=sp)
    return acc.to(torch.bfloat16)


USE_FUSED_DY = __import__("os").environ.get("AXB_LORA_FUSED_DY", "1") != "0"


def fused_dy_ok(dy, B16, xa) -> bool:
    """Whether the one-pass kernel (t = dy B and dB = dy^T xa from a single read of dy) applies."""
    return (USE_FUSED_DY and dy.is_cuda and dy.dtype == torch.bfloat16 and B16 is not None and xa is not None
            and B16.shape[1] <= 64 and dy.shape[0] >= 512 and dy.stride(1) == 1 and dy.stride(0) % 8 == 0
            and B16.stride(1) == 1 and B16.stride(0) % 8 == 0 and xa.stride(1) == 1 and xa.stride(0) % 8 == 0)


def lora_bwd_dy(dy, B16, xa, blocks, scaling, dB_acc):
    """``t = scaling * dy @ B16`` (bf16 [T, R]) and ``dB_acc[blocks] += dy^T @ xa`` (fp32 [N, R], only the
    diagonal blocks) from ONE pass over ``dy`` (csrc/lora_fused.cu)."""
    import ctypes

    from . import _lib

    lib = _lib.cuda_lib()
    T, N = dy.shape
    R = B16.shape[1]
    t32 = torch.zeros((T, R), dtype=torch.float32, device=dy.device)
    flat = (ctypes.c_int * (4 * len(blocks)))(*[int(v) for blk in blocks for v in blk])
    rc = lib.axb_lora_bwd_dy(dy.data_ptr(), dy.stride(0), B16.data_ptr(), B16.stride(0), xa.data_ptr(), xa.stride(0),
                             t32.data_ptr(), dB_acc.data_ptr(), dB_acc.stride(0), T, N, R, flat, len(blocks),
                             _lib.status_word(dy.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "axb_lora_bwd_dy")
    t = torch.empty((T, R), dtype=torch.bfloat16, device=dy.device)
    _lib.check_rc(lib.axb_cast_f32_to_bf16(t32.data_ptr(), t.data_ptr(), t32.numel(), float(scaling), _lib.stream_ptr()),
                  "cast_f32_to_bf16")
    return t


def _t_and_dB(dy, B, B16, xa, blocks, scaling, need_dB):
    """(t, dB) of one projection: the fused one-pass kernel when it applies, two GEMM passes otherwise."""
    if need_dB and fused_dy_ok(dy, B16, xa):
        tgt = getattr(B, "_axb_grad", None)
        buf = tgt if tgt is not None else torch.zeros(B.shape, dtype=torch.float32, device=dy.device)
        t = lora_bwd_dy(dy, B16, xa, blocks, scaling, buf)
        return t, (None if tgt is not None else buf.to(B.dtype)), True
    return skinny_gemm(dy, B16, trans_b=True, alpha=scaling), None, False


class _LoRALinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, W, A, B, A16, B16, scaling, blocks, bias):
        """x [T,K] bf16; W [N,K] bf16 (frozen or trainable); A [R,K] / B [N,R] fp32 masters with
        bf16 shadows A16 / B16; blocks = ((row0, rows, r0, r), ...) diagonal blocks of B."""
        xa = skinny_gemm(x, A16, alpha=scaling)  # [T, R], already scaled
        y = gemm(x, W, a2=xa, b2=B16)
        if bias is not None:
            y = y + bias
        ctx.save_for_backward(x, W, A, B, A16, B16, xa)
        ctx.scaling, ctx.blocks, ctx.has_bias = scaling, blocks, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, W, A, B, A16, B16, xa = ctx.saved_tensors
        s = ctx.scaling
        dy = dy.contiguous()
        T, K = x.shape
        N, R = B16.shape
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        # t = s * dy @ B  -> [T, R]  (and, in the same pass over dy, dB = dy^T xa)
        t, dB_fused, dB_done = _t_and_dB(dy, B, B16, xa, ctx.blocks, s, ctx.needs_input_grad[3])
        dx = gemm(dy, W, trans_b=True, a2=t, b2=A16) if need_dx else None
        dA = dB = None
        if ctx.needs_input_grad[2]:
            tgt = getattr(A, "_axb_grad", None)
            buf = tgt if tgt is not None else torch.zeros(A.shape, dtype=torch.float32, device=x.device)
            sp = pick_splits((K + 255) // 256, (T + 63) // 64)
            gemm(t, x, trans_a=True, trans_b=True, out=buf, accumulate=True, splits=sp)
            dA = None if tgt is not None else buf.to(A.dtype)
        if dB_done:
            dB = dB_fused
        elif ctx.needs_input_grad[3]:
            tgt = getattr(B, "_axb_grad", None)
            buf = tgt if tgt is not None else torch.zeros(B.shape, dtype=torch.float32, device=x.device)
            for (row0, rows, r0, r) in ctx.blocks:
                sp = pick_splits((rows + 127) // 128, (T + 63) // 64)
                # dB_blk [rows, r] = dy[:, row0:row0+rows]^T @ xa[:, r0:r0+r]   (xa carries s)
                gemm(dy[:, row0:row0 + rows], xa[:, r0:r0 + r], trans_a=True, trans_b=True,
                     out=buf[row0:row0 + rows, r0:r0 + r], accumulate=True, splits=sp, bn=64)
            dB = None if tgt is not None else buf.to(B.dtype)
        dW = None
        if need_dw:
            dWf = torch.zeros(W.shape, dtype=torch.float32, device=x.device)
            sp = pick_splits(((N + 127) // 128) * ((K + 255) // 256), (T + 63) // 64)
            gemm(dy, x, trans_a=True, trans_b=True, out=dWf, accumulate=True, splits=sp)
            dW = dWf.to(W.dtype)
        dbias = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[8] else None
        return dx, dW, dA, dB, None, None, None, None, dbias


class _LinearFn(torch.autograd.Function):
    """Plain ``x W^T`` on the tcgen05 GEMM (frozen or trainable weight, optional bias)."""

    @staticmethod
    def forward(ctx, x, W, bias):
        ctx.save_for_backward(x, W)
        ctx.has_bias = bias is not None
        y = gemm(x, W)
        if bias is not None:
            y = y + bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x, W = ctx.saved_tensors
        dy = dy.contiguous()
        T, K = x.shape
        N = W.shape[0]
        dx = gemm(dy, W, trans_b=True) if ctx.needs_input_grad[0] else None
        dW = None
        if ctx.needs_input_grad[1]:
            tgt = getattr(W, "_axb_grad", None)
            buf = tgt if tgt is not None else torch.zeros(W.shape, dtype=torch.float32, device=x.device)
            sp = pick_splits(((N + 127) // 128) * ((K + 255) // 256), (T + 63) // 64)
            gemm(dy, x, trans_a=True, trans_b=True, out=buf, accumulate=True, splits=sp)
            dW = None if tgt is not None else buf.to(W.dtype)
        dbias = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dW, dbias


def _adapter_grads(A, B, t, x, dy, xa, blocks, dB_done=False, dB_fused=None):
    """Gradients of the fp32 LoRA masters: dA [R, K] = t^T x and the diagonal blocks of dB [N, R] =
    dy^T xa (``t`` = s dy B and ``xa`` = s x A^T carry the scaling). Accumulated straight into the
    optimizer's flat gradient buffer (``_axb_grad``) when the parameter has one."""
    T, K = x.shape
    dA = dB = None
    if A is not None and A.requires_grad:
        tgt = getattr(A, "_axb_grad", None)
        buf = tgt if tgt is not None else torch.zeros(A.shape, dtype=torch.float32, device=x.device)
        sp = pick_splits((K + 255) // 256, (T + 63) // 64)
        gemm(t, x, trans_a=True, trans_b=True, out=buf, accumulate=True, splits=sp)
        dA = None if tgt is not None else buf.to(A.dtype)
    if dB_done:
        dB = dB_fused
    elif B is not None and B.requires_grad:
        tgt = getattr(B, "_axb_grad", None)
        buf = tgt if tgt is not None else torch.zeros(B.shape, dtype=torch.float32, device=x.device)
        for (row0, rows, r0, r) in blocks:
            sp = pick_splits((rows + 127) // 128, (T + 63) // 64)
            gemm(dy[:, row0:row0 + rows], xa[:, r0:r0 + r], trans_a=True, trans_b=True,
                 out=buf[row0:row0 + rows, r0:r0 + r], accumulate=True, splits=sp, bn=64)
        dB = None if tgt is not None else buf.to(B.dtype)
    return dA, dB


def _weight_grad(W, dy, x):
    """dW [N, K] = dy^T x for a trainable dense weight (fp32 accumulation, see ``_adapter_grads``)."""
    T, K = x.shape
    N = dy.shape[1]
    tgt = getattr(W, "_axb_grad", None)
    buf = tgt if tgt is not None else torch.zeros((N, K), dtype=torch.float32, device=x.device)
    sp = pick_splits(((N + 127) // 128) * ((K + 255) // 256), (T + 63) // 64)
    gemm(dy, x, trans_a=True, trans_b=True, out=buf, accumulate=True, splits=sp)
    return None if tgt is not None else buf.to(W.dtype)


class _GLUMLPFn(torch.autograd.Function):
    """Whole gated MLP ``down(act(gate(x)) * up(x))`` with optional LoRA on both projections.

    The GLU never runs as a kernel of its own: the gate|up GEMM's epilogue writes gate|up (kept for the
    backward pass) and h = act(gate) * up, and the input-gradient GEMM of the down projection turns its
    accumulator dh into d_gate | d_up before it is stored. Saved: x, gate|up, h and the two skinny
    products x A^T, h A^T; the reference's LoRA_MLP keeps gate, up and recomputes h
    (src/axolotl/kernels/lora.py:283-705)."""

    @staticmethod
    def forward(ctx, x, Wgu, Wd, Agu, Bgu, Agu16, Bgu16, Ad, Bd, Ad16, Bd16, cfg):
        T, I = x.shape[0], cfg["I"]
        xa = skinny_gemm(x, Agu16, alpha=cfg["s_gu"]) if Agu16 is not None else None
        gu = torch.empty((T, 2 * I), dtype=torch.bfloat16, device=x.device)
        h = torch.empty((T, I), dtype=torch.bfloat16, device=x.device)
        gemm(x, Wgu, a2=xa, b2=Bgu16, out=gu, glu=("fwd", cfg["kind"], cfg["limit"], h))
        ha = skinny_gemm(h, Ad16, alpha=cfg["s_d"]) if Ad16 is not None else None
        y = gemm(h, Wd, a2=ha, b2=Bd16)
        ctx.save_for_backward(x, Wgu, Wd, Agu, Bgu, Agu16, Bgu16, Ad, Bd, Ad16, Bd16, gu, h, xa, ha)
        ctx.cfg = cfg
        return y

    @staticmethod
    def backward(ctx, dy):
        x, Wgu, Wd, Agu, Bgu, Agu16, Bgu16, Ad, Bd, Ad16, Bd16, gu, h, xa, ha = ctx.saved_tensors
        cfg = ctx.cfg
        dy = dy.contiguous()
        need = ctx.needs_input_grad
        # ---- down projection: dh = dy W_d + t_d A_d never reaches memory, d_gate | d_up does
        t_d, dBd_f, dBd_done = (_t_and_dB(dy, Bd, Bd16, ha, cfg["blocks_d"], cfg["s_d"], need[8]) if Ad16 is not None
                                else (None, None, False))
        dgu = torch.empty_like(gu)
        gemm(dy, Wd, trans_b=True, a2=t_d, b2=Ad16, out=dgu, glu=("bwd", cfg["kind"], cfg["limit"], gu))
        dAd, dBd = _adapter_grads(Ad if need[7] else None, Bd if need[8] else None, t_d, h, dy, ha, cfg["blocks_d"],
                                  dBd_done, dBd_f)
        dWd = _weight_grad(Wd, dy, h) if need[2] else None
        # ---- gate|up projection
        t_gu, dBgu_f, dBgu_done = (_t_and_dB(dgu, Bgu, Bgu16, xa, cfg["blocks_gu"], cfg["s_gu"], need[4])
                                   if Agu16 is not None else (None, None, False))
        dx = gemm(dgu, Wgu, trans_b=True, a2=t_gu, b2=Agu16) if need[0] else None
        dAgu, dBgu = _adapter_grads(Agu if need[3] else None, Bgu if need[4] else None, t_gu, x, dgu, xa,
                                    cfg["blocks_gu"], dBgu_done, dBgu_f)
        dWgu = _weight_grad(Wgu, dgu, x) if need[1] else None
        return dx, dWgu, dWd, dAgu, dBgu, None, None, dAd, dBd, None, None, None


def _plain_fused(m) -> bool:
    """A FusedLinear the fused MLP can drive directly: dense or LoRA, nothing else attached."""
    return (m.bias is None and m.dora_magnitude is None and m.mora_M is None and m.qat is None
            and not (m.lora_A is not None and m.lora_dropout > 0.0 and m.training))


def glu_mlp(x, gate_up, down, kind, limit, adapters_on=True):
    """``down(act(gate(x)) * up(x))`` through ``_GLUMLPFn`` when both projections qualify and the problem
    is large enough for the CTA-pair kernel's GLU epilogues; returns None otherwise (the caller then
    runs the projections and the GLU kernel one by one)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or kind not in (0, 1):   # the epilogues know silu and tanh-gelu
        return None
    from ..models.layers import FusedLinear

    if type(gate_up) is not FusedLinear or type(down) is not FusedLinear:
        return None
    if not (_plain_fused(gate_up) and _plain_fused(down)):
        return None
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    I = down.in_features
    if sum(gate_up.out_features) != 2 * I or not glu_fusable(x2.shape[0], I, x.device):
        return None

    def lora_of(m):
        if m.lora_A is None or m.merged or not adapters_on:
            return None, None, None, None, 1.0, ()
        if m.lora_A16 is None:
            m.refresh_shadows()
        return m.lora_A, m.lora_B, m.lora_A16, m.lora_B16, float(m.scaling), m.lora_blocks

    Agu, Bgu, Agu16, Bgu16, s_gu, blocks_gu = lora_of(gate_up)
    Ad, Bd, Ad16, Bd16, s_d, blocks_d = lora_of(down)
    cfg = {"I": I, "kind": kind, "limit": float(limit or 0.0), "s_gu": s_gu, "s_d": s_d,
           "blocks_gu": blocks_gu, "blocks_d": blocks_d}
    y = _GLUMLPFn.apply(x2.contiguous(), gate_up.weight, down.weight, Agu, Bgu, Agu16, Bgu16, Ad, Bd, Ad16, Bd16, cfg)
    return y.view(*shp[:-1], y.shape[-1])


def _cpu_weight(W, dtype):
    """Dense view of a (possibly 4-bit) weight for the CPU reference path."""
    st = getattr(W, "_axb_quant", None)
    if st is not None:
        from .nf4 import dequantize_nf4

        return dequantize_nf4(W.data, st, dtype=dtype)
    return W.to(dtype)


def linear(x, W, bias=None):
    """``x @ W^T (+ bias)``; 2-D or N-D ``x``. CPU tensors use torch ops directly."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, _cpu_weight(W, x.dtype), None if bias is None else bias.to(x.dtype))
    shp = x.shape
    y = _LinearFn.apply(x.reshape(-1, shp[-1]).contiguous(), W, bias)
    return y.view(*shp[:-1], y.shape[-1])


def lora_linear(x, W, A, B, A16, B16, scaling, blocks, bias=None, dropout_p=0.0, training=False):
    """Fused LoRA projection (see module docstring). ``A16`` / ``B16`` are the bf16 shadows of the
    fp32 masters on CUDA and may be None on CPU."""
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if not x.is_cuda or (dropout_p > 0.0 and training):
        xd = torch.nn.functional.dropout(x2, dropout_p, training) if dropout_p > 0.0 else x2
        if x.is_cuda:
            base = _LinearFn.apply(x2.contiguous(), W, bias)
            lo = _LinearFn.apply(_LinearFn.apply(xd.contiguous(), A.to(x.dtype), None),
                                 B.to(x.dtype), None)
            y = base + scaling * lo
        else:
            y = torch.nn.functional.linear(x2, _cpu_weight(W, x2.dtype), None if bias is None else bias.to(x2.dtype))
            y = y + scaling * ((xd @ A.to(x2.dtype).t()) @ B.to(x2.dtype).t())
        return y.view(*shp[:-1], y.shape[-1])
    y = _LoRALinearFn.apply(x2.contiguous(), W, A, B, A16, B16, float(scaling), blocks, bias)
    return y.view(*shp[:-1], y.shape[-1])
