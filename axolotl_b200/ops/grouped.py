"""Grouped expert computation on CUDA: every projection of a mixture-of-experts layer is ONE
launch of the grouped tcgen05 GEMM over expert-sorted, 128-row padded token segments.

Per projection ``y = x W_e^T + s (x A_e^T) B_e^T``:
  forward   t  = s * x A_e^T                         (grouped GEMM, N = r)
            y  = x W_e^T + t B_e^T                   (grouped GEMM with the LoRA update as K-extension)
  backward  dt = dy B_e                              (grouped GEMM, transposed weights)
            dx = dy W_e + s * dt A_e                 (same, K-extension)
            dA_e = s * dt^T x,   dB_e = dy^T t       (grouped Gram kernels, fp32, accumulated)
Frozen NVFP4 experts are decoded INSIDE the grouped GEMM (csrc/grouped_w4a16.cu: packed tile by TMA,
converter warps write the bf16 operand tile in shared memory), so the bf16 stack never exists in global
memory; the dequantise-into-scratch route remains for shapes the kernel does not take.
The segment layout is built on the device: no host synchronisation per layer.
"""
from __future__ import annotations

import os

import torch

from . import _lib
from . import functional as Fn

BLOCK = 128


def adapters_enabled():
    from ..models.layers import adapters_enabled as f

    return f()


class GroupLayout:
    """Device-side description of padded expert segments.

    ``dest[i]``: padded row of the i-th expert-sorted compact row; ``blk_expert`` / ``n_blocks`` /
    ``seg_start`` / ``seg_rows`` as consumed by the grouped kernels; ``max_blocks`` is a static
    upper bound (ceil(rows / 128) + E) so buffer shapes never depend on the routing."""

    def __init__(self, counts: torch.Tensor, n_rows: int):
        E = counts.numel()
        dev = counts.device
        counts = counts.to(torch.int64)
        padded = (counts + (BLOCK - 1)) // BLOCK * BLOCK
        seg_end = padded.cumsum(0)
        seg_start = seg_end - padded
        self.E, self.n_rows = E, n_rows
        self.max_blocks = (n_rows + BLOCK - 1) // BLOCK + E
        self.max_rows = self.max_blocks * BLOCK
        e_sorted = torch.repeat_interleave(torch.arange(E, device=dev), counts, output_size=n_rows)
        rank = torch.arange(n_rows, device=dev) - (counts.cumsum(0) - counts)[e_sorted]
        self.dest = seg_start[e_sorted] + rank
        blk_row = torch.arange(self.max_blocks, device=dev) * BLOCK
        self.blk_expert = torch.searchsorted(seg_end, blk_row, right=True).clamp(max=E - 1).to(torch.int32)
        self.n_blocks = (seg_end[-1:] // BLOCK).to(torch.int32)
        self.seg_start = seg_start.to(torch.int32)
        self.seg_rows = padded.to(torch.int32)

    def pad(self, x_sorted):
        out = x_sorted.new_zeros((self.max_rows, x_sorted.shape[1]))
        return out.index_copy(0, self.dest, x_sorted)

    def unpad(self, y_pad):
        return y_pad.index_select(0, self.dest)


def _bn_for(n):
    return 64 if n <= 64 else (128 if n <= 128 or n % 256 else 256)


def grouped_gemm(a, w, lay: GroupLayout, *, trans_w=False, a2=None, w2=None, alpha=1.0, out_dtype=torch.bfloat16):
    """a [max_rows, K]; w [E, N, K] (or [E, K, N] with trans_w); optional K-extension a2 [max_rows, K2],
    w2 [E, N, K2] (or [E, K2, N]). Returns [max_rows, N]."""
    E = w.shape[0]
    if trans_w:
        K, N = w.shape[1], w.shape[2]
    else:
        N, K = w.shape[1], w.shape[2]
    assert a.shape[1] == K and a.shape[0] == lay.max_rows and a.is_contiguous() and w.is_contiguous()
    K2 = 0
    if a2 is not None:
        K2 = a2.shape[1]
        assert a2.is_contiguous() and w2.is_contiguous()
    out = torch.empty((lay.max_rows, N), dtype=out_dtype, device=a.device)
    lib = _lib.cuda_lib()
    _lib.check_rc(lib.axb_grouped_gemm(
        a.data_ptr(), a.stride(0), w.data_ptr(), a2.data_ptr() if a2 is not None else None,
        a2.stride(0) if a2 is not None else 0, w2.data_ptr() if w2 is not None else None, out.data_ptr(),
        out.stride(0), E, N, K, K2, 1 if trans_w else 0, float(alpha), 0 if out_dtype == torch.bfloat16 else 1,
        _bn_for(N), lay.blk_expert.data_ptr(), lay.n_blocks.data_ptr(), lay.max_blocks,
        _lib.status_word().data_ptr(), _lib.stream_ptr()), "grouped_gemm")
    return out


def grouped_gram(a, b, lay: GroupLayout, out, *, alpha=1.0, accumulate=False):
    """out[e] (+)= alpha * a[seg_e]^T b[seg_e]; a [rows, Mg], b [rows, Ng], out fp32 [E, Mg, Ng]."""
    E, Mg, Ng = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and a.is_contiguous() and b.is_contiguous()
    lib = _lib.cuda_lib()
    _lib.check_rc(lib.axb_grouped_gram(
        a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(1), out.stride(0), E, Mg, Ng,
        a.shape[0], float(alpha), 2 if accumulate else 1, _bn_for(Ng), lay.seg_start.data_ptr(),
        lay.seg_rows.data_ptr(), _lib.status_word().data_ptr(), _lib.stream_ptr()), "grouped_gram")
    return out


# NVFP4 expert stacks are decoded inside the grouped GEMM (no bf16 copy of the weights is ever written);
# AXB_W4A16=0 falls back to dequantise-then-GEMM, which gives bit-identical results.
USE_W4A16 = os.environ.get("AXB_W4A16", "1") != "0"


def w4a16_ok(q):
    E, N, Kh = q["qdata"].shape
    return USE_W4A16 and (Kh * 2) % 64 == 0 and N % 8 == 0 and q["qdata"].is_contiguous() and q["scale"].is_contiguous()


def _pts32(q):
    p = q.get("_pts32")
    if p is None or p.device != q["qdata"].device:
        p = q["_pts32"] = q["pts"].to(torch.float32).contiguous()
    return p


def grouped_gemm_w4a16(a, q, lay: GroupLayout, *, trans_w=False, a2=None, w2=None, alpha=1.0, out_dtype=torch.bfloat16):
    """``grouped_gemm`` over NVFP4 weights ``q`` = {qdata uint8 [E, N, K/2], scale e4m3 [E, N, K/16], pts [E]}
    with the 4-bit decode inside the kernel. ``trans_w``: the input-gradient product a . W (a [rows, N])."""
    E, Wn, Kh = q["qdata"].shape
    Wk = Kh * 2
    assert a.shape[1] == (Wn if trans_w else Wk) and a.shape[0] == lay.max_rows and a.is_contiguous()
    K2 = 0
    if a2 is not None:
        K2 = a2.shape[1]
        assert a2.is_contiguous() and w2.is_contiguous()
    out = torch.empty((lay.max_rows, Wk if trans_w else Wn), dtype=out_dtype, device=a.device)
    _lib.check_rc(_lib.cuda_lib().axb_grouped_gemm_w4a16(
        a.data_ptr(), a.stride(0), q["qdata"].data_ptr(), q["scale"].data_ptr(), _pts32(q).data_ptr(),
        a2.data_ptr() if a2 is not None else None, a2.stride(0) if a2 is not None else 0,
        w2.data_ptr() if w2 is not None else None, out.data_ptr(), out.stride(0), E, Wn, Wk, K2,
        1 if trans_w else 0, float(alpha), 0 if out_dtype == torch.bfloat16 else 1, lay.blk_expert.data_ptr(),
        lay.n_blocks.data_ptr(), lay.max_blocks, _lib.status_word().data_ptr(), _lib.stream_ptr()), "grouped_gemm_w4a16")
    return out


# Dequantised expert stacks may be kept from the forward to the backward pass of the same layer
# while they fit a memory budget (half of the memory that is free when the first one is cached);
# beyond the budget the backward pass dequantises again. 180 GB of HBM usually holds all of them.
_WCACHE = {"bytes": 0, "budget": None}


def _expert_weights(experts, which, keep=False, take=False, active=None):
    """bf16 [E, N, K] stack of one projection (dequantised from NVFP4 when the experts are quantised).
    ``keep``: forward pass of a training step (offer the result to the cache); ``take``: backward
    pass (use and release the cached copy if there is one). ``active`` (int32 [E] on the device,
    e.g. the padded rows per expert): experts whose entry is 0 are not dequantised -- their slice of
    the result is never read by the grouped GEMMs (reference: selective expert dequantisation,
    src/axolotl/integrations/kernels/libs/scattermoe_lora/selective_dequant_kernel.py:45-179)."""
    if experts.nvfp4 is None:
        return experts.gate_up_proj if which == "gate_up" else experts.down_proj
    cache = experts.__dict__.setdefault("_dequant_cache", {})
    if take and which in cache:
        W = cache.pop(which)
        _WCACHE["bytes"] -= W.numel() * 2
        return W
    q = experts.nvfp4[which]
    E, N, K2 = q["qdata"].shape
    out = torch.empty((E, N, K2 * 2), dtype=torch.bfloat16, device=q["qdata"].device)
    pts = q["pts"].to(torch.float32).contiguous()
    _lib.check_rc(_lib.cuda_lib().axb_nvfp4_dequant_batched(
        q["qdata"].data_ptr(), q["scale"].data_ptr(), pts.data_ptr(), out.data_ptr(), E, N, K2 * 2,
        active.data_ptr() if active is not None else None, _lib.stream_ptr()), "nvfp4_dequant_batched")
    if keep and which not in cache:
        if _WCACHE["budget"] is None:
            _WCACHE["budget"] = int(torch.cuda.mem_get_info(out.device)[0] * 0.5)
        if _WCACHE["bytes"] + out.numel() * 2 <= _WCACHE["budget"]:
            cache[which] = out
            _WCACHE["bytes"] += out.numel() * 2
    return out


# bf16 operand copies of the expert adapters are rebuilt once per optimizer step, not once per GEMM:
# the trainer bumps this counter whenever parameters may have changed.
_PARAM_EPOCH = [0]


def bump_param_epoch():
    _PARAM_EPOCH[0] += 1


def _adapter_operands(experts, which, A, B, E):
    """(A16 [E, r, K], Bt16 [E, N, r]) bf16 operand layouts of one expert adapter, cached per epoch."""
    cache = experts.__dict__.setdefault("_operand_cache", {})
    hit = cache.get(which)
    if hit is not None and hit[0] == _PARAM_EPOCH[0] and hit[1] is A and hit[2] is B and torch.is_grad_enabled() == hit[5]:
        return hit[3], hit[4]
    r = A.shape[0] // E
    A16 = A.detach().to(torch.bfloat16).view(E, r, -1).contiguous()
    Bt16 = B.detach().view(-1, r, E).permute(2, 0, 1).to(torch.bfloat16).contiguous()
    cache[which] = (_PARAM_EPOCH[0], A, B, A16, Bt16, torch.is_grad_enabled())
    return A16, Bt16


def _grad_buffer(p):
    g = getattr(p, "_axb_grad", None)
    return g


class _GroupedProj(torch.autograd.Function):
    """One expert projection over padded segments; A [E*r, K] and B [N, r*E] are the PEFT-layout
    adapter parameters (B viewed [N, r, E])."""

    @staticmethod
    def forward(ctx, x, experts, which, lay, A, B, scaling):
        q = experts.nvfp4[which] if experts.nvfp4 is not None else None
        w4 = q is not None and w4a16_ok(q)
        if w4:
            E = q["qdata"].shape[0]
            mm = lambda a, **kw: grouped_gemm_w4a16(a, q, lay, **kw)
        else:
            W = _expert_weights(experts, which, keep=bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[4]),
                                active=lay.seg_rows)
            E = W.shape[0]
            mm = lambda a, **kw: grouped_gemm(a, W, lay, **kw)
        if A is not None:
            A16, Bt16 = _adapter_operands(experts, which, A, B, E)
            t = grouped_gemm(x, A16, lay, alpha=scaling)
            y = mm(x, a2=t, w2=Bt16)
            ctx.save_for_backward(x, t, A, B)
        else:
            y = mm(x)
            ctx.save_for_backward(x)
        ctx.experts, ctx.which, ctx.lay, ctx.scaling, ctx.has_lora = experts, which, lay, scaling, A is not None
        ctx.train_w = experts.nvfp4 is None and W.requires_grad
        ctx.w4 = w4
        return y

    @staticmethod
    def backward(ctx, dy):
        experts, which, lay = ctx.experts, ctx.which, ctx.lay
        dy = dy.contiguous()
        if ctx.w4:
            q = experts.nvfp4[which]
            E, W = q["qdata"].shape[0], None
            mm = lambda a, **kw: grouped_gemm_w4a16(a, q, lay, trans_w=True, **kw)
        else:
            W = _expert_weights(experts, which, take=True, active=lay.seg_rows)
            E = W.shape[0]
            mm = lambda a, **kw: grouped_gemm(a, W, lay, trans_w=True, **kw)
        dA = dB = None
        if ctx.has_lora:
            x, t, A, B = ctx.saved_tensors
            r = A.shape[0] // E
            A16, Bt16 = _adapter_operands(experts, which, A, B, E)
            dt = grouped_gemm(dy, Bt16, lay, trans_w=True, alpha=ctx.scaling)    # s * dy B_e   [rows, r]
            dx = mm(dy, a2=dt, w2=A16)
            gA = _grad_buffer(A)
            if gA is not None:      # accumulate straight into the optimizer's flat gradient view
                grouped_gram(dt, x, lay, gA.view(E, r, -1), accumulate=True)
            else:
                dA = grouped_gram(dt, x, lay, torch.empty((E, r, x.shape[1]), dtype=torch.float32,
                                                          device=x.device)).view(E * r, -1).to(A.dtype)
            dBt = grouped_gram(dy, t, lay, torch.empty((E, dy.shape[1], r), dtype=torch.float32, device=x.device))
            dB_full = dBt.permute(1, 2, 0).reshape(B.shape)                      # [N, r, E] -> [N, r*E]
            gB = _grad_buffer(B)
            if gB is not None:
                gB.add_(dB_full)
            else:
                dB = dB_full.to(B.dtype)
        else:
            (x,) = ctx.saved_tensors
            dx = mm(dy)
        if ctx.train_w:
            gW = grouped_gram(dy, x, lay, torch.empty(W.shape, dtype=torch.float32, device=x.device))
            buf = _grad_buffer(W)
            if buf is not None:
                buf.add_(gW)
            else:
                W.grad = gW.to(W.dtype) if W.grad is None else W.grad + gW.to(W.dtype)
        return dx, None, None, None, dA, dB, None


class RoutedLayout(GroupLayout):
    """Layout of a local (single-rank) MoE layer built from the router's top-k choice ``idx`` [T, k]:
    adds the slot <-> padded-row maps used by the dispatch / combine kernels."""

    def __init__(self, idx: torch.Tensor, E: int):
        T, k = idx.shape
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        # torch.bincount synchronises with the host (it sizes its output from the data): count with a
        # scatter-add instead so the layer stays free of host round trips
        counts = torch.zeros(E, dtype=torch.int64, device=idx.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))
        super().__init__(counts, T * k)
        self.k = k
        self.slot_row = torch.empty(T * k, dtype=torch.int32, device=idx.device)
        self.slot_row[order] = self.dest.to(torch.int32)
        self.row_token = torch.full((self.max_rows,), -1, dtype=torch.int32, device=idx.device)
        self.row_token[self.dest] = (order // k).to(torch.int32)


def _dispatch_rows(x, row_token, row_scale, n_rows):
    out = torch.empty((n_rows, x.shape[1]), dtype=x.dtype, device=x.device)
    _lib.check_rc(_lib.cuda_lib().axb_moe_dispatch_rows(
        x.data_ptr(), row_token.data_ptr(), row_scale.data_ptr() if row_scale is not None else None, out.data_ptr(),
        n_rows, x.shape[1], _lib.stream_ptr()), "moe_dispatch_rows")
    return out


def _combine_rows(ys, slot_row, w, n_tokens, k):
    out = torch.empty((n_tokens, ys.shape[1]), dtype=ys.dtype, device=ys.device)
    _lib.check_rc(_lib.cuda_lib().axb_moe_combine_rows(
        ys.data_ptr(), slot_row.data_ptr(), w.data_ptr() if w is not None else None, out.data_ptr(), n_tokens, k,
        ys.shape[1], _lib.stream_ptr()), "moe_combine_rows")
    return out


class _LocalDispatch(torch.autograd.Function):
    """x [T, H] -> padded expert-sorted rows [max_rows, H] (zeros in pad rows)."""

    @staticmethod
    def forward(ctx, x, lay):
        ctx.lay, ctx.T = lay, x.shape[0]
        return _dispatch_rows(x.contiguous(), lay.row_token, None, lay.max_rows)

    @staticmethod
    def backward(ctx, dxp):
        lay = ctx.lay
        return _combine_rows(dxp.contiguous(), lay.slot_row, None, ctx.T, lay.k), None


class _LocalCombine(torch.autograd.Function):
    """y[t] = sum_j w[t, j] * ys[row of slot (t, j)]."""

    @staticmethod
    def forward(ctx, ys, w, lay):
        ctx.lay = lay
        wf = w.detach().float().contiguous()
        ctx.save_for_backward(ys, wf)
        ctx.w_dtype = w.dtype
        return _combine_rows(ys.contiguous(), lay.slot_row, wf, w.shape[0], lay.k)

    @staticmethod
    def backward(ctx, dy):
        ys, wf = ctx.saved_tensors
        lay = ctx.lay
        dy = dy.contiguous()
        row_scale = torch.zeros(lay.max_rows, dtype=torch.float32, device=dy.device)
        row_scale[lay.slot_row.long()] = wf.reshape(-1)
        dys = _dispatch_rows(dy, lay.row_token, row_scale, lay.max_rows)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = torch.empty(wf.shape, dtype=torch.float32, device=dy.device)
            _lib.check_rc(_lib.cuda_lib().axb_moe_combine_dw(
                dy.data_ptr(), ys.data_ptr(), lay.slot_row.data_ptr(), dw.data_ptr(), wf.numel(), lay.k, dy.shape[1],
                _lib.stream_ptr()), "moe_combine_dw")
            dw = dw.to(ctx.w_dtype)
        return dys, dw, None


GEMV_MAX_SLOTS = 64     # decode steps: up to this many routed slots run as matrix-vector products


def _gemv(x, slot_token, slot_expert, experts, which):
    q = experts.nvfp4[which] if experts.nvfp4 is not None else None
    S = slot_expert.numel()
    if q is not None:
        E, N, Kh = q["qdata"].shape
        K = Kh * 2
        args = (q["qdata"].data_ptr(), q["scale"].data_ptr(), _pts32(q).data_ptr(), 1)
    else:
        W = experts.gate_up_proj if which == "gate_up" else experts.down_proj
        E, N, K = W.shape
        args = (W.data_ptr(), None, None, 0)
    out = torch.empty((S, N), dtype=torch.bfloat16, device=x.device)
    _lib.check_rc(_lib.cuda_lib().axb_moe_gemv(x.data_ptr(), slot_token.data_ptr(), slot_expert.data_ptr(), args[0], args[1],
                                               args[2], out.data_ptr(), S, E, N, K, args[3], _lib.stream_ptr()), "moe_gemv")
    return out


def _slot_lora(inp, slot_expert, experts, which):
    """s * B_e (A_e v) per slot, for the few slots of a decode step (batched small products)."""
    E = experts.E
    A16, Bt16 = _adapter_operands(experts, which, experts.lora[which + "_A"], experts.lora[which + "_B"], E)
    se = slot_expert.long()
    t = torch.bmm(A16.index_select(0, se), inp.unsqueeze(-1))                    # [S, r, 1]
    return float(experts.scaling) * torch.bmm(Bt16.index_select(0, se), t).squeeze(-1)


@torch.no_grad()
def moe_decode_forward(experts, x, w, idx):
    """Expert pass of a generation step (a few tokens, no autograd): every routed slot is a GEMV against its expert
    (``csrc/moe_gemv.cu``), NVFP4 weights decoded in registers; adapters are applied per slot."""
    T, k = idx.shape
    slot_expert = idx.reshape(-1).to(torch.int32).contiguous()
    slot_token = (torch.arange(T * k, device=x.device, dtype=torch.int32) // k).contiguous()
    x = x.contiguous()
    use_lora = experts.lora is not None and adapters_enabled()
    gu = _gemv(x, slot_token, slot_expert, experts, "gate_up")
    if use_lora:
        gu = gu + _slot_lora(x.index_select(0, slot_token.long()), slot_expert, experts, "gate_up").to(gu.dtype)
    if getattr(experts, "gate_up_bias", None) is not None:
        gu = gu + experts.gate_up_bias.to(gu.dtype).index_select(0, slot_expert.long())
    h = Fn.glu(gu, experts.act, getattr(experts, "glu_limit", None)).contiguous()
    own = torch.arange(T * k, device=x.device, dtype=torch.int32)
    y = _gemv(h, own, slot_expert, experts, "down")
    if use_lora:
        y = y + _slot_lora(h, slot_expert, experts, "down").to(y.dtype)
    if getattr(experts, "down_bias", None) is not None:
        y = y + experts.down_bias.to(y.dtype).index_select(0, slot_expert.long())
    return (y.view(T, k, -1).float() * w.float().unsqueeze(-1)).sum(1).to(x.dtype)


def moe_local_forward(experts, x, w, idx, E):
    """Whole local MoE expert pass on CUDA: dispatch -> grouped projections -> weighted combine."""
    if not torch.is_grad_enabled() and idx.numel() <= GEMV_MAX_SLOTS and x.dtype == torch.bfloat16:
        return moe_decode_forward(experts, x, w, idx)
    lay = RoutedLayout(idx, E)
    xp = _LocalDispatch.apply(x, lay)
    yp = grouped_experts_padded(experts, xp, lay)
    return _LocalCombine.apply(yp, w, lay)


def grouped_experts_forward(experts, x_sorted, counts):
    """x_sorted [M, H]: rows grouped by local expert; counts: per-expert row counts (device tensor,
    or a python list). Returns [M, H]."""
    if not torch.is_tensor(counts):
        counts = torch.tensor(counts, dtype=torch.int64, device=x_sorted.device)
    lay = GroupLayout(counts, x_sorted.shape[0])
    return lay.unpad(grouped_experts_padded(experts, lay.pad(x_sorted.contiguous()), lay))


def grouped_experts_padded(experts, x, lay):
    """x: padded expert-sorted rows [lay.max_rows, H] -> same layout [lay.max_rows, H]."""
    use_lora = experts.lora is not None and adapters_enabled()
    L = experts.lora if use_lora else None
    gu = _GroupedProj.apply(x, experts, "gate_up", lay, L["gate_up_A"] if L else None, L["gate_up_B"] if L else None,
                            float(experts.scaling))
    row_e = None
    if getattr(experts, "gate_up_bias", None) is not None:     # per-expert biases (gpt-oss): one row gather + add
        row_e = lay.blk_expert.long().repeat_interleave(BLOCK)
        gu = gu + experts.gate_up_bias.to(gu.dtype).index_select(0, row_e)
    h = Fn.glu(gu, experts.act, getattr(experts, "glu_limit", None),
               blocks_in_use=lay.n_blocks if getattr(lay, "prefix_only", False) else None)
    y = _GroupedProj.apply(h, experts, "down", lay, L["down_A"] if L else None, L["down_B"] if L else None,
                           float(experts.scaling))
    if row_e is not None:
        y = y + experts.down_bias.to(y.dtype).index_select(0, row_e)
    return y


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
