"""Tensor parallelism with the all-reduce fused into the GEMM epilogue.

Column-parallel projections (q|k|v, gate|up) keep the output rows of their heads / intermediate
slice; row-parallel projections (o, down) keep the matching input columns. The partial products of
a row-parallel forward GEMM (and of a column-parallel input-gradient GEMM) are summed across the
TP group *inside the GEMM epilogue*: every output tile is reduce-added with ``multimem.red``
(NVSwitch multicast; plain peer atomics as fallback) into a symmetric bf16 buffer on every rank,
so no separate collective kernel and no extra pass over the activation exists. Two symmetric
buffers alternate, which leaves one device-side flag barrier per reduced GEMM.

LoRA on a sharded projection is sharded the same way (B rows with a column-parallel weight, A
columns with a row-parallel weight); the other factor is replicated and its gradient is summed
over the TP group. This is what the reference obtains from transformers' ``tp_plan="auto"``
DTensor plans plus NCCL (src/axolotl/loaders/model.py:847-852).
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from ..models.layers import FusedLinear
from ..ops import _lib
from ..utils.logging import get_logger
from .symm import WAIT_BUDGET_NS, PeerSync, SymmBuffer, _u64_array

LOG = get_logger(__name__)

_lib.register_cuda_sigs({
    "axb_gemm_bf16_allreduce": [_lib.vp, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i32, _lib.i64, _lib.i32, _lib.i32,
                                _lib.i32, _lib.vp, _lib.i64, _lib.vp, _lib.i64, _lib.i32, _lib.f32, _lib.i32, _lib.vp,
                                _lib.vp, _lib.i32, _lib.vp, _lib.vp],
    # A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, A2, lda2, B2, ldb2, K2, alpha, bn, red_mc, red_ptrs, cnt_ptrs,
    # red_rank, red_world, r_ctas, status, stream
    "axb_gemm_bf16_allreduce2": [_lib.vp, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i32, _lib.vp, _lib.i64, _lib.i32,
                                 _lib.i32, _lib.i32, _lib.vp, _lib.i64, _lib.vp, _lib.i64, _lib.i32, _lib.f32, _lib.i32,
                                 _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.vp],
})


class TPContext:
    def __init__(self, device, group, size, rank, max_elems):
        self.device, self.group, self.size, self.rank = torch.device(device), group, size, rank
        self.fused = self.device.type == "cuda"
        self.k = 0
        if self.fused:
            self.bufs = [SymmBuffer(max_elems, torch.bfloat16, self.device, group) for _ in range(2)]
            # per-rank completion counters of 128-row blocks (zeroed here, re-armed by the kernel)
            self.cnt = SymmBuffer(65536, torch.int32, self.device, group, use_multicast=False)
            self.cnt.tensor.zero_()
            self.sync = PeerSync(self.device, group)
            self.reducer_ctas = int(os.environ.get("AXB_TP_REDUCER_CTAS", "0"))   # 0 = by GEMM depth
            torch.cuda.synchronize(self.device)
            dist.barrier(group)

    def _reducers(self, K):
        """Reducer CTAs of a launch: the shallower the GEMM (small K), the more of the launch's time the
        reduction of its output needs. Measured on 2 GPUs: 16 for K = 4096, 8 for K = 14336."""
        if self.reducer_ctas > 0:
            return self.reducer_ctas
        return max(8, min(24, round(16 * 4096 / max(K, 1))))

    def reduced_gemm(self, a, b, *, trans_b=False, a2=None, b2=None, alpha=1.0):
        """sum over the TP group of ``alpha * (a @ op(b)^T + a2 @ op(b2)^T)`` -> [M, N] bf16."""
        from ..ops.gemm import _pick_bn, _row_major_2d, gemm

        if not self.fused:
            y = gemm(a, b, trans_b=trans_b, a2=a2, b2=b2, alpha=alpha)
            dist.all_reduce(y, group=self.group)
            return y
        lib = _lib.cuda_lib()
        shard = getattr(b, "_axb_shard", None)
        if shard is not None:  # FSDP-sharded weight below a TP shard: read it from its staging buffer
            staging, plans = shard.ctx.acquire(shard, backward=trans_b)
            if shard.ctx.copy_engine:       # next weights of the schedule arrive by the copy engines meanwhile
                for pl in plans:
                    shard.ctx.prefetch_by_copy(pl)
                    shard.ctx.committed(pl)
            b = staging[: shard.rows * shard.cols].view(shard.rows, shard.cols)
        a, b = _row_major_2d(a), _row_major_2d(b)
        M, K = a.shape
        N = b.shape[1] if trans_b else b.shape[0]
        K2 = 0
        if a2 is not None:
            a2, b2 = _row_major_2d(a2), _row_major_2d(b2)
            K2 = a2.shape[1]
        buf = self.bufs[self.k & 1]
        self.k += 1
        if M * N > buf.tensor.numel():
            raise ValueError("tensor-parallel reduce buffer is too small for this GEMM")
        if (M + 127) // 128 > self.cnt.tensor.numel():
            raise ValueError("tensor-parallel GEMM has more 128-row blocks than completion counters")
        # one launch: tiles are stored into this rank's symmetric buffer while reducer CTAs sum every
        # finished 128-row block over the ranks (in-switch multimem.ld_reduce, or peer loads) and
        # write the sum back into every rank's buffer
        rc = lib.axb_gemm_bf16_allreduce2(
            a.data_ptr(), a.stride(0), 0, b.data_ptr(), b.stride(0), int(trans_b), buf.tensor.data_ptr(), N, M, N, K,
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2), b2.stride(0) if b2 is not None else 0, K2,
            float(alpha), _pick_bn(M, N), buf.multicast_ptr or None, buf.ptrs_c, self.cnt.ptrs_c, self.rank, self.size,
            self._reducers(K), _lib.status_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "axb_gemm_bf16_allreduce2")
        self.sync.barrier(channel=3)            # every owner has written its blocks into every buffer
        return buf.tensor[: M * N].view(M, N).clone()


class _ColumnParallelLoRA(torch.autograd.Function):
    """y_local = x W_r^T + s (x A^T) B_r^T ;  dx = all-reduce(dy_r W_r + t_r A) fused in the GEMM."""

    @staticmethod
    def forward(ctx, x, W, A, B, scaling, tp):
        from ..ops.gemm import gemm

        has_lora = A is not None
        A16 = A.detach().to(torch.bfloat16) if has_lora and A.dtype != torch.bfloat16 else A
        B16 = B.detach().to(torch.bfloat16) if has_lora and B.dtype != torch.bfloat16 else B
        xa = gemm(x, A16, alpha=scaling) if has_lora else None
        y = gemm(x, W, a2=xa, b2=B16) if has_lora else gemm(x, W)
        ctx.save_for_backward(x, W, A, B, xa)
        ctx.scaling, ctx.tp = scaling, tp
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm, pick_splits

        x, W, A, B, xa = ctx.saved_tensors
        tp, s = ctx.tp, ctx.scaling
        dy = dy.contiguous()
        T, K = x.shape
        has_lora = A is not None
        dA = dB = None
        t = None
        if has_lora:
            A16, B16 = A.detach().to(torch.bfloat16), B.detach().to(torch.bfloat16)
            t = gemm(dy, B16, trans_b=True, alpha=s)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = tp.reduced_gemm(dy, W, trans_b=True, a2=t, b2=A16 if has_lora else None)
        if has_lora:
            dAf = torch.zeros(A.shape, dtype=torch.float32, device=x.device)
            gemm(t, x, trans_a=True, trans_b=True, out=dAf, accumulate=True,
                 splits=pick_splits((K + 255) // 256, (T + 63) // 64))
            dBf = torch.zeros(B.shape, dtype=torch.float32, device=x.device)
            gemm(dy, xa, trans_a=True, trans_b=True, out=dBf, accumulate=True,
                 splits=pick_splits((B.shape[0] + 127) // 128, (T + 63) // 64), bn=64)
            dA, dB = dAf.to(A.dtype), dBf.to(B.dtype)
        return dx, None, dA, dB, None, None


class _RowParallelLoRA(torch.autograd.Function):
    """y = all-reduce(x_r W_r^T + s (x_r A_r^T) B^T) fused in the GEMM ;  dx_r = dy W_r + t A_r."""

    @staticmethod
    def forward(ctx, x, W, A, B, scaling, tp):
        from ..ops.gemm import gemm

        has_lora = A is not None
        A16 = A.detach().to(torch.bfloat16) if has_lora else None
        B16 = B.detach().to(torch.bfloat16) if has_lora else None
        xa = gemm(x, A16, alpha=scaling) if has_lora else None
        y = tp.reduced_gemm(x, W, a2=xa, b2=B16)
        ctx.save_for_backward(x, W, A, B, xa)
        ctx.scaling, ctx.tp = scaling, tp
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm, pick_splits

        x, W, A, B, xa = ctx.saved_tensors
        s = ctx.scaling
        dy = dy.contiguous()
        T, K = x.shape
        has_lora = A is not None
        dA = dB = None
        t = A16 = None
        if has_lora:
            A16, B16 = A.detach().to(torch.bfloat16), B.detach().to(torch.bfloat16)
            t = gemm(dy, B16, trans_b=True, alpha=s)
        dx = gemm(dy, W, trans_b=True, a2=t, b2=A16) if ctx.needs_input_grad[0] else None
        if has_lora:
            dAf = torch.zeros(A.shape, dtype=torch.float32, device=x.device)
            gemm(t, x, trans_a=True, trans_b=True, out=dAf, accumulate=True,
                 splits=pick_splits((K + 255) // 256, (T + 63) // 64))
            dBf = torch.zeros(B.shape, dtype=torch.float32, device=x.device)
            gemm(dy, xa, trans_a=True, trans_b=True, out=dBf, accumulate=True,
                 splits=pick_splits((B.shape[0] + 127) // 128, (T + 63) // 64), bn=64)
            dA, dB = dAf.to(A.dtype), dBf.to(B.dtype)
        return dx, None, dA, dB, None, None


class TPLinear(torch.nn.Module):
    """Tensor-parallel shard of a FusedLinear (keeps its sub-projection bookkeeping for adapters)."""

    def __init__(self, src: FusedLinear, mode: str, tp: TPContext, unit: int = 1):
        super().__init__()
        self.mode, self.tp = mode, tp
        self.names = list(src.names)
        r, n = tp.rank, tp.size
        W = src.weight.detach()
        if mode == "column":
            parts, self.out_features = [], []
            off = 0
            for o in src.out_features:
                if o % (n * unit):
                    raise ValueError(f"output size {o} is not divisible by tp={n}")
                loc = o // n
                parts.append(W[off + r * loc: off + (r + 1) * loc])
                self.out_features.append(loc)
                off += o
            w = torch.cat(parts, 0)
            self.in_features = src.in_features
        else:
            K = src.in_features
            if K % n:
                raise ValueError(f"input size {K} is not divisible by tp={n}")
            loc = K // n
            w = W[:, r * loc:(r + 1) * loc]
            self.in_features, self.out_features = loc, list(src.out_features)
        self.weight = torch.nn.Parameter(w.contiguous().clone(), requires_grad=False)
        self.full_in, self.full_out = src.in_features, list(src.out_features)
        self.lora_A = self.lora_B = None
        self.lora_names, self.lora_r, self.scaling = [], 0, 1.0
        self.lora_blocks = ()
        self.bias = None

    def row_range(self, name):
        i = self.names.index(name)
        r0 = sum(self.out_features[:i])
        return r0, r0 + self.out_features[i]

    def add_lora(self, r, alpha, dropout=0.0, targets=None, use_rslora=False, dtype=torch.float32, init_b_zero=True):
        import math

        targets = [n for n in self.names if targets is None or n in targets]
        if not targets:
            return
        if dropout:
            raise NotImplementedError("lora_dropout is not supported together with tensor parallelism")
        dev = self.weight.device
        R = r * len(targets)
        # the replicated factor must be identical on every TP rank: draw it from a generator that
        # does not depend on the rank; the sharded factor (B for column, A columns for row) is local
        gen = torch.Generator(device="cpu").manual_seed(1234 + self.full_in + sum(self.full_out))
        bound = 1.0 / math.sqrt(self.full_in)  # kaiming_uniform(a=sqrt(5)) bound for fan_in
        A_full = (torch.rand(R, self.full_in, generator=gen) * 2 - 1) * bound
        if self.mode == "column":
            A = A_full
        else:
            loc = self.in_features
            A = A_full[:, self.tp.rank * loc:(self.tp.rank + 1) * loc]
        N = self.weight.shape[0]
        B = torch.zeros(N, R, dtype=dtype, device=dev)
        blocks = []
        for i, n in enumerate(targets):
            r0, r1 = self.row_range(n)
            blocks.append((r0, r1 - r0, i * r, r))
        self.lora_A = torch.nn.Parameter(A.to(device=dev, dtype=dtype).contiguous())
        self.lora_B = torch.nn.Parameter(B)
        # replicated factors: gradient must be summed over the TP group
        (self.lora_A if self.mode == "column" else self.lora_B)._tp_replicated = True
        (self.lora_B if self.mode == "column" else self.lora_A)._tp_sharded = True
        self.lora_blocks, self.lora_names, self.lora_r = tuple(blocks), targets, r
        self.scaling = alpha / math.sqrt(r) if use_rslora else alpha / r
        self._mask = None

    def refresh_shadows(self):
        pass

    def peft_tensors(self):
        out = {}
        for (r0, rows, c0, r), n in zip(self.lora_blocks, self.lora_names):
            out[n] = (self.lora_A[c0:c0 + r], self.lora_B[r0:r0 + rows, c0:c0 + r])
        return out

    def gathered_peft_tensors(self):
        """Full (unsharded) PEFT tensors, assembled over the TP group."""
        out = {}
        for n, (A, B) in self.peft_tensors().items():
            A, B = A.detach().contiguous(), B.detach().contiguous()
            if self.mode == "column":
                parts = [torch.empty_like(B) for _ in range(self.tp.size)]
                dist.all_gather(parts, B, group=self.tp.group)
                out[n] = (A, torch.cat(parts, 0))
            else:
                parts = [torch.empty_like(A) for _ in range(self.tp.size)]
                dist.all_gather(parts, A, group=self.tp.group)
                out[n] = (torch.cat(parts, 1), B)
        return out

    def forward(self, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        A, B = self.lora_A, self.lora_B
        if A is not None:
            from ..models.layers import adapters_enabled

            if not adapters_enabled():
                A = B = None
        if B is not None and len(self.lora_blocks) > 1:
            if self._mask is None:
                m = torch.zeros_like(B)
                for (r0, rows, c0, r) in self.lora_blocks:
                    m[r0:r0 + rows, c0:c0 + r] = 1
                self._mask = m
            B = B * self._mask  # keeps the off-diagonal blocks (and their gradients) at zero
        fn = _ColumnParallelLoRA if self.mode == "column" else _RowParallelLoRA
        if not x2.is_cuda:
            y = _cpu_forward(x2, self.weight, A, B, self.scaling, self.mode, self.tp)
        else:
            y = fn.apply(x2, self.weight, A, B, float(self.scaling), self.tp)
        return y.view(*shp[:-1], y.shape[-1])


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToTP(torch.autograd.Function):
    """identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def _cpu_forward(x, W, A, B, s, mode, tp):
    """gloo path: same math with torch ops and explicit collectives (host-side plumbing tests)."""
    if mode == "column":
        x = _CopyToTP.apply(x, tp.group)
    y = x @ W.to(x.dtype).t()
    if A is not None:
        y = y + s * ((x @ A.to(x.dtype).t()) @ B.to(x.dtype).t())
    if mode == "row":
        y = _AllReduceSum.apply(y, tp.group)
    return y


@torch.no_grad()
def apply_tensor_parallel(model, tp: TPContext):
    """Replaces the projections of every decoder layer by their TP shards (before adapters are
    injected) and narrows the attention head counts."""
    cfg = model.config
    n = tp.size
    if cfg.num_attention_heads % n or cfg.num_key_value_heads % n:
        raise ValueError(f"head counts ({cfg.num_attention_heads}/{cfg.num_key_value_heads}) are not divisible by tp={n}")
    for layer in model.layers:
        att = layer.self_attn
        att.qkv_proj = TPLinear(att.qkv_proj, "column", tp, unit=att.D)
        att.o_proj = TPLinear(att.o_proj, "row", tp)
        att.Hq //= n
        att.Hk //= n
        if not layer.is_moe:
            layer.mlp.gate_up_proj = TPLinear(layer.mlp.gate_up_proj, "column", tp)
            layer.mlp.down_proj = TPLinear(layer.mlp.down_proj, "row", tp)
    torch.cuda.empty_cache() if tp.device.type == "cuda" else None
    return model


def sync_tp_replicated_grads(model, tp: TPContext):
    """Sums the gradients of TP-replicated trainable parameters over the TP group."""
    for p in model.parameters():
        if p.requires_grad and getattr(p, "_tp_replicated", False):
            g = getattr(p, "_axb_grad", None)
            g = g if g is not None else p.grad
            if g is not None:
                dist.all_reduce(g, group=tp.group)
