"""Context parallelism: every rank owns a contiguous chunk of the packed token stream.

Attention needs the K / V rows of earlier chunks. Instead of a ring of NCCL send/recv steps or an
NCCL all-gather, each rank *stores* its rotated K / V rows straight into a symmetric KV buffer of
every rank (``multimem.st`` through the NVSwitch, or plain peer stores), one flag barrier later
the varlen attention kernel runs on the local q rows against the global K / V with the document
tile table of the whole stream. In the backward pass every rank computes the dK / dV tiles its q
rows contribute to and reduce-adds them over NVLink into the gradient buffer of the rank that
owns those kv rows, inside the attention-backward epilogue; dQ stays local.

Replaces ring-flash-attn's ``llama3_flash_attn_varlen_func`` (all-gather of K/V per head stride +
FA2 varlen) used by the reference (src/axolotl/monkeypatch/ring_attn/patch.py:50-132) and keeps
its conventions: contiguous chunks, global ``cu_seqlens`` from position ids, labels shifted before
the split, loss normalised by the global number of trainable tokens.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import functional as Fn
from .symm import PeerSync, SymmBuffer

_lib.register_cuda_sigs({
    "axb_allgather_store": [_lib.vp, _lib.i64, _lib.i64, _lib.i32, _lib.i64, _lib.vp, _lib.vp, _lib.i32, _lib.vp],
    "axb_flash_varlen_fwd_cp": [_lib.vp, _lib.i64, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i64, _lib.i32, _lib.i32,
                                _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.i64, _lib.vp, _lib.f32, _lib.vp, _lib.vp],
    "axb_flash_varlen_bwd_cp": [_lib.vp, _lib.i64, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i64, _lib.vp, _lib.vp,
                                _lib.i64, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.i64,
                                _lib.vp, _lib.vp, _lib.f32, _lib.i32, _lib.i64, _lib.vp, _lib.vp, _lib.vp],
})


def cp_tiles(cu_seqlens, c0, c1):
    """Tile tables (global rows) for the q rows [c0, c1): forward = 128-row q tiles intersecting
    the window (largest tile_start first); backward = 128-row kv tiles that some q row of the
    window can see (most work first)."""
    fwd, bwd = [], []
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    for d in range(len(cu) - 1):
        s, e = int(cu[d]), int(cu[d + 1])
        if e <= c0 or s >= c1:
            continue
        L = e - s
        for t in range(0, L, 128):
            if s + t < c1 and s + min(t + 128, L) > c0:
                fwd.append((s, L, t, 0))
            if s + t < c1:  # kv tile starts before the end of the window: later q rows of the window see it
                bwd.append((s, L, t, 0))
    fwd.sort(key=lambda x: -x[2])
    bwd.sort(key=lambda x: -(min(x[0] + x[1], c1) - max(x[0] + x[2], c0)))
    return np.asarray(fwd, dtype=np.int32).reshape(-1, 4), np.asarray(bwd, dtype=np.int32).reshape(-1, 4)


class CPMeta:
    """Varlen metadata of one context-parallel rank."""

    def __init__(self, cu_seqlens, total, rank, world, device, ctx):
        self.cu_seqlens_host = np.asarray(cu_seqlens, dtype=np.int32)
        self.total = int(total)
        self.chunk = self.total // world
        self.c0, self.c1 = rank * self.chunk, (rank + 1) * self.chunk
        self.rank, self.world, self.ctx = rank, world, ctx
        self.device = torch.device(device)
        self.cp = True
        if self.device.type == "cuda":
            f, b = cp_tiles(cu_seqlens, self.c0, self.c1)
            self.n_fwd, self.n_bwd = len(f), len(b)
            both = torch.from_numpy(np.concatenate([f, b], 0)).pin_memory().to(self.device, non_blocking=True)
            self.tiles_fwd, self.tiles_bwd = both[: self.n_fwd], both[self.n_fwd:]


class CPContext:
    def __init__(self, device, group, size, rank):
        self.device, self.group, self.size, self.rank = torch.device(device), group, size, rank
        self.fused = self.device.type == "cuda"
        self.kv_bufs = None
        self.dkv_bufs = None
        self.k = 0
        self.kb = 0
        if self.fused:
            self.sync = PeerSync(self.device, group)

    def _ensure(self, total, chunk, kv_width, qkv_width):
        if self.kv_bufs is None or self.kv_bufs[0].tensor.numel() < total * kv_width:
            self.kv_bufs = [SymmBuffer(total * kv_width, torch.bfloat16, self.device, self.group) for _ in range(2)]
            self.dkv_bufs = [SymmBuffer(chunk * qkv_width, torch.bfloat16, self.device, self.group, use_multicast=False)
                             for _ in range(2)]
            dist.barrier(self.group)

    # ------------------------------------------------------------------ batch handling
    def slice_batch(self, batch: dict) -> dict:
        """Global collated batch ([1, S]) -> this rank's chunk, labels shifted before the split."""
        ids, lab, pos = batch["input_ids"], batch["labels"], batch["position_ids"]
        if ids.shape[0] != 1:
            raise ValueError("context parallelism expects one packed row per micro batch")
        S = ids.shape[1]
        if S % (self.size * 128):
            raise ValueError(f"sequence length {S} must be a multiple of {self.size * 128} for context parallelism")
        shifted = torch.cat([lab[:, 1:], torch.full((1, 1), -100, dtype=lab.dtype)], 1)
        c = S // self.size
        sl = slice(self.rank * c, (self.rank + 1) * c)
        cu = batch.get("cu_seqlens")
        if cu is None:
            p = pos.reshape(-1).numpy()
            st = np.flatnonzero(p == 0)
            cu = np.concatenate([st if len(st) and st[0] == 0 else np.concatenate([[0], st]), [S]]).astype(np.int32)
        out = {"input_ids": ids[:, sl].contiguous(), "labels": shifted[:, sl].contiguous(),
               "position_ids": pos[:, sl].contiguous(), "labels_preshifted": True,
               "n_trainable": int((shifted != -100).sum().item()), "n_tokens": int(S),
               "cp_meta_args": (cu, S)}
        return out

    def make_meta(self, cu, total):
        return CPMeta(cu, total, self.rank, self.size, self.device, self)


class _FlashVarlenCP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, meta: CPMeta, Hq, Hk, D, scale):
        cp = meta.ctx
        lib = _lib.cuda_lib()
        T = qkv.shape[0]
        kvw, qw = 2 * Hk * D, (Hq + 2 * Hk) * D
        cp._ensure(meta.total, meta.chunk, kvw, qw)
        buf = cp.kv_bufs[cp.k & 1]
        cp.k += 1
        kv_local = qkv[:, Hq * D:]
        _lib.check_rc(lib.axb_allgather_store(kv_local.data_ptr(), qkv.stride(0), T, kvw, meta.c0,
                                              buf.multicast_ptr or None, buf.ptrs_c, cp.size, _lib.stream_ptr()),
                      "allgather_store")
        cp.sync.barrier(channel=4)
        kv_full = buf.tensor[: meta.total * kvw].view(meta.total, kvw)
        out = torch.empty((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
        lse2 = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(lib.axb_flash_varlen_fwd_cp(qkv.data_ptr(), qkv.stride(0), T, meta.c0, kv_full.data_ptr(), kvw,
                                                  meta.total, Hq, Hk, D, meta.tiles_fwd.data_ptr(), meta.n_fwd,
                                                  out.data_ptr(), out.stride(0), lse2.data_ptr(), scale,
                                                  _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()),
                      "flash_varlen_fwd_cp")
        kv_saved = kv_full.clone()  # the symmetric buffer is reused two layers later
        ctx.save_for_backward(qkv, kv_saved, out, lse2)
        ctx.meta, ctx.dims = meta, (Hq, Hk, D, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, kv_full, out, lse2 = ctx.saved_tensors
        Hq, Hk, D, scale = ctx.dims
        meta = ctx.meta
        cp = meta.ctx
        lib = _lib.cuda_lib()
        T = qkv.shape[0]
        qw = (Hq + 2 * Hk) * D
        dout = dout.contiguous()
        buf = cp.dkv_bufs[cp.kb & 1]   # zero on every rank since its last use
        cp.kb += 1
        dq_acc = torch.empty((T, Hq * D), dtype=torch.float32, device=qkv.device)
        delta = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
        _lib.check_rc(lib.axb_flash_varlen_bwd_cp(
            qkv.data_ptr(), qkv.stride(0), T, meta.c0, kv_full.data_ptr(), kv_full.stride(0), meta.total,
            dout.data_ptr(), out.data_ptr(), out.stride(0), lse2.data_ptr(), Hq, Hk, D, meta.tiles_bwd.data_ptr(),
            meta.n_bwd, buf.tensor.data_ptr(), qw, dq_acc.data_ptr(), delta.data_ptr(), scale, cp.size, meta.chunk,
            buf.ptrs_c, _lib.status_word(qkv.device).data_ptr(), _lib.stream_ptr()), "flash_varlen_bwd_cp")
        cp.sync.barrier(channel=5)       # every rank's dK / dV contributions have landed
        dqkv = buf.tensor[: T * qw].view(T, qw).clone()
        buf.tensor[: T * qw].zero_()
        return dqkv, None, None, None, None, None


def flash_varlen_cp(qkv, meta: CPMeta, Hq, Hk, D, scale):
    if qkv.is_cuda:
        return _FlashVarlenCP.apply(qkv, meta, Hq, Hk, D, scale)
    return _cpu_cp_attention(qkv, meta, Hq, Hk, D, scale)


class _GatherKV(torch.autograd.Function):
    """gloo path: all-gather of K/V with a reduce-scatter-like backward."""

    @staticmethod
    def forward(ctx, kv, group, world, rank):
        ctx.group, ctx.world, ctx.rank = group, world, rank
        parts = [torch.empty_like(kv) for _ in range(world)]
        dist.all_gather(parts, kv.contiguous(), group=group)
        return torch.cat(parts, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        c = g.shape[0] // ctx.world
        return g[ctx.rank * c:(ctx.rank + 1) * c], None, None, None


def _cpu_cp_attention(qkv, meta, Hq, Hk, D, scale):
    T = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(T, Hq, D)
    kv = _GatherKV.apply(qkv[:, Hq * D:], meta.ctx.group, meta.world, meta.rank)
    k = kv[:, : Hk * D].reshape(-1, Hk, D)
    v = kv[:, Hk * D:].reshape(-1, Hk, D)
    rep = Hq // Hk
    out = torch.zeros_like(q)
    cu = meta.cu_seqlens_host
    for d in range(len(cu) - 1):
        s, e = int(cu[d]), int(cu[d + 1])
        lo, hi = max(s, meta.c0), min(e, meta.c1)
        if lo >= hi:
            continue
        qq = q[lo - meta.c0: hi - meta.c0].float().transpose(0, 1)
        kk = k[s:hi].float().repeat_interleave(rep, 1).transpose(0, 1)
        vv = v[s:hi].float().repeat_interleave(rep, 1).transpose(0, 1)
        sc = (qq @ kk.transpose(1, 2)) * scale
        qi = torch.arange(lo, hi)[:, None]
        ki = torch.arange(s, hi)[None, :]
        sc = sc.masked_fill(ki > qi, float("-inf"))
        out[lo - meta.c0: hi - meta.c0] = (sc.softmax(-1) @ vv).transpose(0, 1).to(q.dtype)
    return out.reshape(T, Hq * D)
