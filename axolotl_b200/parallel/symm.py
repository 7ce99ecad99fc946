"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

Allocation and handle exchange ride on ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged over the process group's store, optional NVSwitch multicast binding); the
kernels only need the resulting raw addresses: one pointer per rank, the multicast address where
available, and the signal pads used for device-side flag barriers.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..ops import _lib

_lib.register_cuda_sigs({
    "axb_peer_barrier": [_lib.vp, _lib.i32, _lib.i32, _lib.i32, C.c_uint, _lib.vp, _lib.i64, _lib.vp],
    "axb_rs_adamw_ag": [_lib.vp] * 5 + [_lib.vp] * 3 + [_lib.vp, _lib.vp, _lib.i64, _lib.i32, _lib.i32, C.c_uint]
                       + [_lib.f32] * 9 + [_lib.vp, _lib.vp, _lib.i64, _lib.vp],
    "axb_rs_adamw_ag_sharded": [_lib.vp] * 5 + [_lib.vp] * 3 + [_lib.vp, _lib.vp, _lib.i64, _lib.i32, _lib.i32, C.c_uint]
                               + [_lib.f32] * 9 + [_lib.vp, _lib.vp, _lib.i64, _lib.vp],
    "axb_rs_adamw_ag_pass": [_lib.vp] * 5 + [_lib.vp] * 3 + [_lib.vp, _lib.vp, _lib.i64, _lib.i32, _lib.i32, C.c_uint]
                            + [_lib.f32] * 9 + [_lib.vp, _lib.vp, _lib.i64, _lib.vp, _lib.i32, _lib.i32],
    "axb_peer_allreduce_f32": [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, C.c_uint,
                               _lib.vp, _lib.i64, _lib.vp],
    "axb_gemm_bf16_prefetch": [_lib.vp, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.vp,
                               _lib.i64, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.i64, _lib.vp, _lib.i64,
                               _lib.i32, _lib.f32, _lib.f32, _lib.i32, _lib.i32, _lib.i32,
                               _lib.vp, C.c_ulonglong, C.c_ulonglong, _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.vp],
    "axb_allgather_rows": [_lib.vp, C.c_ulonglong, C.c_ulonglong, _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.vp],
})

WAIT_BUDGET_NS = int(float(os.environ.get("AXB_PEER_WAIT_S", "20")) * 1e9)


def _u64_array(vals):
    return (C.c_ulonglong * len(vals))(*[int(v) for v in vals])


_ALLOCATED_BYTES = 0


def allocated_bytes() -> int:
    """Bytes of symmetric (peer-mapped) memory this process has allocated so far. These arenas are outside
    torch's caching allocator, so ``torch.cuda.max_memory_allocated`` does not see them."""
    return _ALLOCATED_BYTES


class SymmBuffer:
    """A tensor every rank of ``group`` allocated with the same size, plus its peer addresses."""

    def __init__(self, numel, dtype, device, group, use_multicast=True):
        import torch.distributed._symmetric_memory as symm_mem

        global _ALLOCATED_BYTES
        _ALLOCATED_BYTES += int(numel) * torch.empty((), dtype=dtype).element_size()
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.pad_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        mc = int(self.handle.multicast_ptr) if (use_multicast and self.handle.has_multicast_support) else 0
        self.multicast_ptr = mc
        self.ptrs_c = _u64_array(self.ptrs)
        self.pad_ptrs_c = _u64_array(self.pad_ptrs)
        self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64, device=device)  # bit pattern of u64


class PeerSync:
    """Device-side barrier / tiny all-reduce over the signal pads of one symmetric buffer."""

    def __init__(self, device, group):
        self.buf = SymmBuffer(16 * 1024, torch.float32, device, group, use_multicast=False)
        self.rank, self.world = self.buf.rank, self.buf.world
        self.epochs = {}
        self.device = device

    def next_epoch(self, channel, n=1):
        e = self.epochs.get(channel, 0) + 1
        self.epochs[channel] = e + n - 1
        return e

    def barrier(self, channel=1):
        lib = _lib.cuda_lib()
        _lib.check_rc(lib.axb_peer_barrier(self.buf.pad_ptrs_c, self.rank, self.world, channel,
                                           self.next_epoch(channel), _lib.status_word(self.device).data_ptr(),
                                           WAIT_BUDGET_NS, _lib.stream_ptr()), "peer_barrier")

    def all_reduce_(self, t: torch.Tensor, channel=2):
        """In-place sum of a small fp32 vector (<= 1024 elements) across the group."""
        assert t.dtype == torch.float32 and t.numel() <= 1024
        lib = _lib.cuda_lib()
        _lib.check_rc(lib.axb_peer_allreduce_f32(self.buf.ptrs_c, self.buf.pad_ptrs_c, t.data_ptr(), t.numel(),
                                                 self.rank, self.world, channel, self.next_epoch(channel, 2),
                                                 _lib.status_word(self.device).data_ptr(), WAIT_BUDGET_NS,
                                                 _lib.stream_ptr()), "peer_allreduce")
        return t
