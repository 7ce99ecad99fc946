"""ctypes bindings for the in-tree native libraries.

``libaxb200.so`` holds every sm_100a kernel (C ABI, raw device pointers + stream);
``libaxb200_host.so`` holds host-only helpers (multipack packer, attention tile tables).
On a machine with a CUDA device the kernel library is mandatory: ops raise instead of silently
falling back to eager PyTorch when it cannot be loaded.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_cuda_lib = None
_host_lib = None

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_CUDA_SIGS = {
    "axb_gemm_bf16": [vp, i64, i32, vp, i64, i32, vp, i64, vp, i64, i32, i32, i32, vp, i64, vp, i64,
                      i32, f32, f32, i32, i32, i32, vp, vp],
    "axb_gemm_bf16_pair": [vp, i64, i32, vp, i64, i32, vp, i64, vp, i64, i32, i32, i32, vp, i64, vp, i64,
                           i32, f32, f32, i32, vp, C.c_ulonglong, C.c_ulonglong, i32, vp, i32, vp, vp],
    "axb_gemm_bf16_pair_glu": [vp, i64, i32, vp, i64, i32, vp, i64, vp, i64, i32, i32, i32, vp, i64, vp, i64,
                               i32, f32, i32, i32, f32, vp, i64, vp, C.c_ulonglong, C.c_ulonglong, i32, vp, i32,
                               vp, vp],
    "axb_lora_bwd_dy": [vp, i64, vp, i64, vp, i64, vp, vp, i64, i32, i32, i32, vp, i32, vp, vp],
    "axb_gemm_set_backoff": [i32, i32],
    "axb_gemm_set_pair_tuning": [i32, i32, i32],
    "axb_nvfp4_dequant": [vp, vp, vp, vp, i64, i64, vp],
    "axb_moe_dispatch_rows": [vp, vp, vp, vp, i64, i32, vp],
    "axb_moe_combine_rows": [vp, vp, vp, vp, i64, i32, i32, vp],
    "axb_moe_combine_dw": [vp, vp, vp, vp, i64, i32, i32, vp],
    "axb_nf4_dequant": [vp, vp, vp, i64, i32, vp],
    "axb_fp8_block_dequant": [vp, vp, vp, i64, i64, i32, vp],
    "axb_nvfp4_dequant_batched": [vp, vp, vp, vp, i64, i64, i64, vp, vp],
    # A, lda, W, A2, lda2, W2, C, ldc, E, N, K, K2, trans_w, alpha, out_mode, bn, blk_expert, n_blocks, max_blocks, status, stream
    "axb_grouped_gemm": [vp, i64, vp, vp, i64, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, i32, vp, vp, i32, vp, vp],
    # A, lda, B, ldb, C, ldc, c_batch, E, Mg, Ng, rows, alpha, out_mode, bn, seg_start, seg_rows, status, stream
    # A, lda, qdata, scale, pts, A2, lda2, W2, C, ldc, E, Wn, Wk, K2, trans_w, alpha, out_mode, blk_expert, n_blocks, max_blocks, status, stream
    "axb_grouped_gemm_w4a16": [vp, i64, vp, vp, vp, vp, i64, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, vp, vp, i32, vp, vp],
    "axb_flash_wide_fwd": [vp, i64, i64, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp, i64, vp, f32, f32, vp, vp],
    "axb_flash_wide_bwd": [vp, i64, vp, vp, i64, vp, i64, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp, i64, vp, vp,
                           f32, f32, vp, vp],
    "axb_glu_fwd_rows": [vp, vp, i64, i32, i32, f32, vp, vp],
    "axb_glu_bwd_rows": [vp, vp, vp, i64, i32, i32, f32, vp, vp],
    "axb_ep_gather_rows_n": [vp, i32, vp, vp, vp, vp, vp, vp, i64, i32, i64, vp, vp],
    "axb_moe_gemv": [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "axb_rope_partial": [vp, vp, vp, i32, i32, i32, i32, i64, f32, f32, vp],
    "axb_ebft_rewards": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "axb_indexer_scores": [vp, i64, vp, i64, vp, vp, i64, i32, i32, i32, i32, i32, vp, vp],
    "axb_layernorm_fwd": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, f32, vp],
    "axb_layernorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp],
    "axb_xielu_fwd": [vp, vp, i64, f32, f32, f32, f32, vp],
    "axb_xielu_bwd": [vp, vp, vp, vp, i64, f32, f32, f32, f32, vp],
    "axb_gated_pool_fwd": [vp, vp, vp, i64, i32, i32, vp],
    "axb_gated_pool_bwd": [vp, vp, vp, vp, vp, vp, i64, i32, i32, vp],
    "axb_mhc_mix_fwd": [vp, vp, vp, vp, vp, vp, i64, i32, i32, f32, f32, vp],
    "axb_mhc_mix_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, f32, f32, vp],
    "axb_bounds_check_enabled": [],
    "axb_bounds_fetch": [vp],
    "axb_bounds_reset": [],
    "axb_grouped_gram": [vp, i64, vp, i64, vp, i64, i64, i32, i32, i32, i64, f32, i32, i32, vp, vp, vp, vp],
    "axb_ep_gather_rows": [vp, i32, vp, vp, vp, vp, vp, vp, i64, i32, i64, vp],
    "axb_ep_scatter_add": [vp, i32, vp, vp, vp, vp, i64, i32, i64, vp],
    "axb_ep_stage_rows": [vp, i32, i32, vp, vp, i64, i32, vp],
    "axb_ep_reduce_rows": [vp, i32, i32, vp, vp, i64, i32, vp],
    "axb_peer_put_i32": [vp, vp, i64, vp],
    "axb_ep_gather_tables": [vp, i32, i64, vp, vp],
    "axb_ep_put_scalars": [vp, i32, vp, vp, vp, i64, i64, vp],
    "axb_rmsnorm_fwd": [vp, vp, vp, vp, vp, vp, i64, i32, f32, f32, vp],
    "axb_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp],
    "axb_rope_qk": [vp, vp, vp, i32, i32, i32, i32, i64, f32, f32, vp, vp, vp, f32, vp],
    "axb_rope_qk_bwd": [vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, f32, vp, vp, vp, vp, vp, vp],
    "axb_dora_norm": [vp, vp, vp, vp, vp, i64, i32, f32, vp],
    "axb_glu_fwd": [vp, vp, i64, i32, i32, f32, vp],
    "axb_glu_bwd": [vp, vp, vp, i64, i32, i32, f32, vp],
    "axb_rmsnorm_gated_fwd": [vp, vp, vp, vp, vp, i64, i32, f32, f32, vp],
    "axb_rmsnorm_gated_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp],
    "axb_entropy": [vp, vp, vp, i64, i32, i64, f32, vp],
    "axb_decode_attn": [vp, i64, i32, vp, vp, vp, vp, i64, i32, i32, i32, i32, i64, f32, i32, vp],
    "axb_sinkgd_step": [vp, i32, vp, vp, vp, i32, i32, i32, f32, f32, f32, vp],
    "axb_embedding_fwd": [vp, vp, vp, i64, i32, i64, vp],
    "axb_embedding_bwd": [vp, vp, vp, i64, i32, i64, vp],
    "axb_ce_fwd_bwd": [vp, vp, vp, vp, i64, i32, i64, f32, i64, i32, vp],
    "axb_ce_fwd_bwd_softcap": [vp, vp, vp, vp, i64, i32, i64, f32, i64, i32, f32, vp],
    "axb_sumsq": [vp, i64, vp, vp],
    "axb_adamw": [vp, vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, f32, vp, f32, f32, vp],
    "axb_cast_bf16_to_f32": [vp, vp, i64, f32, i32, vp],
    "axb_cast_f32_to_bf16": [vp, vp, i64, f32, vp],
    "axb_add_bf16": [vp, vp, i64, vp],
    "axb_flash_varlen_fwd": [vp, i64, i64, i32, i32, i32, i32, i32, i32, vp, i32, vp, i64, vp, f32,
                             vp, vp],
    "axb_flash_varlen_bwd": [vp, i64, vp, vp, i64, vp, i64, i32, i32, i32, i32, i32, i32, vp, i32,
                             vp, i64, vp, vp, f32, vp, vp],
}

_HOST_SIGS = {
    "axb_pack_first_fit": [vp, i64, i32, i32, i64, vp],
    "axb_pack_sequential": [vp, i64, i32, i32, vp],
    "axb_build_attn_tiles": [vp, i32, i32, i32, vp, i32],
}


def _bind(lib, sigs, optional=()):
    for name, argtypes in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if name in optional:
                continue
            raise
        fn.argtypes = argtypes
        fn.restype = C.c_int
    return lib


def register_cuda_sigs(sigs: dict) -> None:
    """Lets other modules (parallel/, moe) declare the kernels they call."""
    _CUDA_SIGS.update(sigs)
    global _cuda_lib
    if _cuda_lib is not None:
        _bind(_cuda_lib, sigs)


def cuda_lib():
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                # AXB_BOUNDS_CHECK=1: the variant built with -DAXB_BOUNDS_CHECK (index checks in the kernels)
                checked = os.environ.get("AXB_BOUNDS_CHECK", "0") not in ("", "0")
                path = _LIB_DIR / ("libaxb200_checked.so" if checked else "libaxb200.so")
                if not path.exists():
                    raise RuntimeError(
                        f"{path} is missing: run `python -m axolotl_b200.build` (needs nvcc). "
                        "axolotl_b200 does not fall back to eager PyTorch on a CUDA device."
                    )
                _cuda_lib = _bind(C.CDLL(str(path)), _CUDA_SIGS)
    return _cuda_lib


def host_lib():
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                path = _LIB_DIR / "libaxb200_host.so"
                if not path.exists():
                    from .. import build as _build

                    _build.build()
                _host_lib = _bind(C.CDLL(str(path)), _HOST_SIGS)
    return _host_lib


def ptr(t):
    """Raw data pointer of a tensor (or NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    return t


_STATUS_NAMES = {
    1: "TMA stage never arrived (full barrier timeout)",
    2: "smem stage never released (empty barrier timeout)",
    3: "TMEM accumulator never became ready",
    4: "TMEM accumulator never released",
    5: "peer flag never arrived",
    6: "bad argument",
    7: "generic wait timeout",
}


class KernelTimeoutError(RuntimeError):
    pass


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises when a kernel recorded a timeout."""
    t = status_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelTimeoutError(f"axolotl_b200 kernel reported status {code}: {_STATUS_NAMES.get(code, '?')}")


class KernelBoundsError(RuntimeError):
    pass


_BOUNDS_SITES = {1: "embedding token id", 2: "embedding-gradient token id", 3: "cross-entropy label",
                 4: "grouped GEMM expert id", 5: "W4A16 grouped GEMM expert id", 6: "attention document tile",
                 7: "MoE dispatch token index"}


def bounds_violation():
    """(site name, index, limit, count) of the first out-of-range index the bounds-check library recorded since
    the last reset, or None. Always None with the regular library."""
    lib = cuda_lib()
    if not lib.axb_bounds_check_enabled():
        return None
    out = (C.c_longlong * 4)()
    check_rc(lib.axb_bounds_fetch(out), "bounds_fetch")
    if out[0] == 0:
        return None
    return _BOUNDS_SITES.get(int(out[0]), f"site {int(out[0])}"), int(out[1]), int(out[2]), int(out[3])


def check_bounds(reset=True) -> None:
    v = bounds_violation()
    if v is not None:
        if reset:
            cuda_lib().axb_bounds_reset()
        raise KernelBoundsError(f"out-of-range {v[0]}: index {v[1]}, limit {v[2]} ({v[3]} violations; the accesses were skipped)")


launch_count = 0  # native kernel entry points called so far (each launches >= 1 kernel)


def check_rc(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
