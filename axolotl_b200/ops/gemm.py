"""bf16 GEMM on the tcgen05 kernel (CUDA) with a plain PyTorch path for CPU tensors.

``gemm(a, b)`` computes ``alpha * (op(a) @ op(b)^T + a2 @ b2^T) + beta * c_in`` where
``op(a)`` is ``a`` ([M, K]) or, with ``trans_a``, a matrix stored as [K, M]; likewise
``op(b)`` is ``b`` ([N, K]) or, with ``trans_b``, stored as [K, N]. The optional ``a2``/``b2``
pair is the K-extension that fuses a LoRA update into the same accumulator tile.
"""
from __future__ import annotations

import os

import torch

from . import _lib

_SM = 148
# CTA-pair (cta_group::2, 256x256 tile per SM pair) kernel: the default for large GEMMs;
# AXB_GEMM_PAIR=0 keeps every launch on the single-CTA kernel.
USE_PAIR = os.environ.get("AXB_GEMM_PAIR", "1") != "0"
# GLU folded into the gate|up GEMM epilogue (forward) and the down-projection input-gradient GEMM
# (backward); AXB_GLU_EPILOGUE=0 runs the stand-alone GLU kernels instead.
USE_GLU_EPILOGUE = os.environ.get("AXB_GLU_EPILOGUE", "1") != "0"


def _pick_bn(M: int, N: int) -> int:
    m_tiles = (M + 127) // 128
    for bn in (256, 128, 64):
        if bn > 64 and N <= bn // 2:
            continue
        if m_tiles * ((N + bn - 1) // bn) >= _SM or bn == 64:
            return bn
    return 64


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("gemm operands must be 2-D")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
        if t.stride(0) % 8 != 0:
            raise ValueError("gemm operand rows must be a multiple of 8 elements")
    return t


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    trans_a: bool = False,
    trans_b: bool = False,
    a2: torch.Tensor | None = None,
    b2: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    c_in: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    splits: int = 1,
    bn: int | None = None,
    glu: tuple | None = None,
) -> torch.Tensor:
    """``glu`` selects a GLU epilogue of the CTA-pair kernel (callers check ``glu_fusable`` first):
    ``("fwd", kind, limit, h_out)``: ``b`` is the [2I, K] gate|up weight, ``out`` [M, 2I] receives
    gate|up and ``h_out`` [M, I] ``act(gate) * up``; ``("bwd", kind, limit, gate_up)``: the product is
    dh [M, I] and ``out`` [M, 2I] receives d_gate | d_up (``out`` may be ``gate_up`` itself)."""
    quant = getattr(b, "_axb_quant", None)
    if quant is not None:
        # frozen 4-bit weight: expand into the shared bf16 scratch right before the GEMM reads it
        from .nf4 import dequantize_nf4, scratch_weight

        b = dequantize_nf4(b, quant, out=scratch_weight(quant.shape, b.device) if b.is_cuda else None,
                           dtype=torch.bfloat16 if b.is_cuda else a.dtype)
    shard = getattr(b, "_axb_shard", None)
    if shard is not None:
        return _gemm_allgather(a, b, shard, trans_a=trans_a, trans_b=trans_b, a2=a2, b2=b2, alpha=alpha,
                               beta=beta, c_in=c_in, out=out, out_dtype=out_dtype, bn=bn, glu=glu)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[1] if trans_b else b.shape[0]
    Kb = b.shape[0] if trans_b else b.shape[1]
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    K2 = 0
    if a2 is not None:
        K2 = a2.shape[0] if trans_a else a2.shape[1]

    if not a.is_cuda:
        # reference path (CPU): same contraction in the operand dtype with fp32 accumulation
        fa = (a.t() if trans_a else a).float()
        fb = (b if trans_b else b.t()).float()
        acc = fa @ fb
        if a2 is not None:
            acc = acc + (a2.t() if trans_a else a2).float() @ (b2 if trans_b else b2.t()).float()
        acc = acc * alpha
        if c_in is not None and beta != 0.0:
            acc = acc + beta * c_in.float()
        if accumulate:
            out.add_(acc.to(out.dtype))
            return out
        res = acc.to(out_dtype if a.dtype == torch.bfloat16 or out_dtype == torch.float32 else a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    lib = _lib.cuda_lib()
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("the tcgen05 GEMM takes bf16 operands")
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    if a2 is not None:
        a2 = _row_major_2d(a2)
        b2 = _row_major_2d(b2)
    if accumulate and splits <= 1 and out is not None and out.dtype == torch.float32 and c_in is None and a.is_cuda:
        # a single K pass owns every output tile: plain read-add-write (beta = 1) instead of fp32
        # atomics, which also makes the launch eligible for the 2-CTA kernel
        return gemm(a, b, trans_a=trans_a, trans_b=trans_b, a2=a2, b2=b2, alpha=alpha, beta=1.0, c_in=out, out=out,
                    out_dtype=torch.float32, accumulate=False, splits=1, bn=bn)
    if accumulate:
        if out is None or out.dtype != torch.float32:
            raise ValueError("accumulate=True needs an fp32 `out`")
        out_mode = 2
    else:
        if splits > 1:
            raise ValueError("split-K needs accumulate=True (fp32 atomics)")
        out_mode = 0 if out_dtype == torch.bfloat16 else 1
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.stride(1) != 1:
        raise ValueError("gemm output must be row-major")
    if c_in is not None:
        if c_in.stride(1) != 1 or c_in.dtype != out.dtype:
            raise ValueError("c_in must be row-major with the output dtype")
    if glu is not None:
        _glu_launch(lib, glu, a, int(trans_a), b.data_ptr(), b.stride(0), int(trans_b), out, M, N, K, a2, b2, K2,
                    alpha, (None, 0, 0, 0, None, 0))
        return out
    if bn is None:
        bn = _pick_bn(M, N)
    if not accumulate and _use_pair(M, N, bn):
        rc = lib.axb_gemm_bf16_pair(
            a.data_ptr(), a.stride(0), int(trans_a), b.data_ptr(), b.stride(0), int(trans_b),
            out.data_ptr(), out.stride(0), _lib.ptr(c_in), c_in.stride(0) if c_in is not None else 0, M, N, K,
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
            K2, float(alpha), float(beta if c_in is not None else 0.0), out_mode, None, 0, 0, 0, None, 0,
            _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "axb_gemm_bf16_pair")
        return out
    rc = lib.axb_gemm_bf16(
        a.data_ptr(), a.stride(0), int(trans_a),
        b.data_ptr(), b.stride(0), int(trans_b),
        out.data_ptr(), out.stride(0),
        _lib.ptr(c_in), c_in.stride(0) if c_in is not None else 0,
        M, N, K,
        _lib.ptr(a2), a2.stride(0) if a2 is not None else 0,
        _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
        K2, float(alpha), float(beta if c_in is not None else 0.0), out_mode, int(splits), int(bn),
        _lib.status_word(a.device).data_ptr(), _lib.stream_ptr(),
    )
    _lib.check_rc(rc, "axb_gemm_bf16")
    return out


def glu_fusable(M: int, I: int, device) -> bool:
    """Whether the GLU epilogues of the CTA-pair kernel serve an MLP with ``M`` token rows and ``I``
    intermediate columns (enough 256-row tiles for the 74 SM pairs, whole 32-column chunks)."""
    return (USE_PAIR and USE_GLU_EPILOGUE and device.type == "cuda" and M >= 512 and I % 32 == 0
            and ((M + 255) // 256) * ((I + 255) // 256) >= 74)


def _glu_launch(lib, glu, a, trans_a, b_ptr, ldb, trans_b, out, M, N, K, a2, b2, K2, alpha, pf):
    mode, kind, limit, other = glu
    if out is None or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("the GLU epilogue writes a row-major bf16 [M, 2I] `out`")
    if mode == "fwd":
        # b: [2I, K]; N passed by the caller is 2I
        I = N // 2
        h = other
        rc = lib.axb_gemm_bf16_pair_glu(
            a.data_ptr(), a.stride(0), trans_a, b_ptr, ldb, trans_b, out.data_ptr(), out.stride(0), None, 0,
            M, I, K, _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2),
            b2.stride(0) if b2 is not None else 0, K2, float(alpha), 1, int(kind), float(limit or 0.0),
            h.data_ptr(), h.stride(0), *pf, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
    else:
        gu = other
        rc = lib.axb_gemm_bf16_pair_glu(
            a.data_ptr(), a.stride(0), trans_a, b_ptr, ldb, trans_b, out.data_ptr(), out.stride(0),
            gu.data_ptr(), gu.stride(0), M, N, K, _lib.ptr(a2), a2.stride(0) if a2 is not None else 0,
            _lib.ptr(b2), b2.stride(0) if b2 is not None else 0, K2, float(alpha), 2, int(kind),
            float(limit or 0.0), None, 0, *pf, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "axb_gemm_bf16_pair_glu")


def _use_pair(M, N, bn) -> bool:
    """The 2-CTA kernel (256x256 tile per SM pair, each CTA stages half of B) wins once there are
    enough 256x256 tiles for the 74 SM pairs; small or skinny problems keep the 1-CTA kernel."""
    return USE_PAIR and bn == 256 and M >= 512 and N >= 512 and ((M + 255) // 256) * ((N + 255) // 256) >= 74


def pick_splits(out_tiles: int, k_blocks: int) -> int:
    """Split-K factor for skinny weight-gradient GEMMs so that all SMs get work."""
    if out_tiles >= _SM:
        return 1
    return max(1, min(k_blocks, _SM // max(out_tiles, 1)))


def _gemm_allgather(a, b_shard, info, *, trans_a, trans_b, a2, b2, alpha, beta, c_in, out, out_dtype, bn, glu=None):
    """GEMM against a row-sharded B. The full B is read from a staging buffer that an earlier
    launch filled; this launch's extra CTAs all-gather the next weight of the schedule (see
    parallel/fsdp.py)."""
    if trans_a:
        raise ValueError("the sharded-weight GEMM takes a row-major A")
    from ..parallel import symm as _symm  # noqa: F401  (registers the kernel signatures)

    lib = _lib.cuda_lib()
    a = _row_major_2d(a)
    M, Ka = a.shape
    rows, cols = info.rows, info.cols            # stored (full) B matrix
    N, K = (cols, rows) if trans_b else (rows, cols)
    if Ka != K:
        raise ValueError(f"gemm: inner dimensions differ ({Ka} vs {K})")
    K2 = 0
    if a2 is not None:
        a2, b2 = _row_major_2d(a2), _row_major_2d(b2)
        K2 = a2.shape[1]
    out_mode = 0 if out_dtype == torch.bfloat16 else 1
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if bn is None:
        bn = _pick_bn(M, N)
    ctx = info.ctx
    staging, plans = ctx.acquire(info, backward=trans_b)
    plan = None
    if plans and ctx.copy_engine:
        for pl in plans:          # copy engines: distance-1 and distance-2 weights, beside this GEMM
            ctx.prefetch_by_copy(pl)
            ctx.committed(pl)
        pf = (None, 0, 0, 0, None, 0)
    elif plans and plans[0][0].index in (info.index + 1, info.index - 1):
        plan = plans[0]           # gather CTAs of this launch: the next weight only
        nxt, slot = plan
        pf = (nxt.peer_bases_dev.data_ptr(), nxt.shard_offset, nxt.shard_bytes, nxt.world,
              ctx.staging[slot].data_ptr(), ctx.prefetch_ctas(nxt, 2.0 * M * N * K))
    else:
        pf = (None, 0, 0, 0, None, 0)
    if glu is not None:
        _glu_launch(lib, glu, a, 0, staging.data_ptr(), cols, int(trans_b), out, M, N, K, a2, b2, K2, alpha, pf)
    elif _use_pair(M, N, bn):
        rc = lib.axb_gemm_bf16_pair(
            a.data_ptr(), a.stride(0), 0, staging.data_ptr(), cols, int(trans_b), out.data_ptr(), out.stride(0),
            _lib.ptr(c_in), c_in.stride(0) if c_in is not None else 0, M, N, K,
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
            K2, float(alpha), float(beta if c_in is not None else 0.0), out_mode,
            *pf, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "axb_gemm_bf16_pair")
    else:
        rc = lib.axb_gemm_bf16_prefetch(
            a.data_ptr(), a.stride(0), 0, staging.data_ptr(), cols, int(trans_b), out.data_ptr(), out.stride(0),
            _lib.ptr(c_in), c_in.stride(0) if c_in is not None else 0, M, N, K,
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
            K2, float(alpha), float(beta if c_in is not None else 0.0), out_mode, 1, int(bn),
            *pf, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "axb_gemm_bf16_prefetch")
    if plan is not None:
        ctx.committed(plan)
    return out
