"""Expert parallelism: experts are sharded over the EP group, tokens travel to their experts and
back over NVLink peer memory.

Per MoE layer and micro batch:
1. routing is local (softmax -> top-k); every rank writes its routing table ([T, k] expert ids and
   weights) next to its hidden states in symmetric memory. After ONE flag barrier each rank reads all
   tables with peer loads and builds its plan on the device (which slots run on its experts, in
   expert-sorted padded order) with static shapes: buffers are sized by a capacity factor
   (``AXB_EP_CAPACITY``, default 2 x the mean load; never more than the worst case); an overflow is
   recorded on the device, the optimizer step it belongs to is skipped on every rank and the factor grows. No NCCL call and no host synchronisation
   happens on the layer path;
2. DISPATCH: the destination ranks *pull* the rows routed to their experts with peer loads: each needed token once
   into a local staging area (``axb_ep_stage_rows``; top-k routing puts several slots of a token on
   the same rank), then a local gather into the padded expert-sorted layout
   (``axb_ep_gather_rows``) -- no send buffers, no host barrier;
3. the local experts run as tcgen05 GEMMs (bf16, or NVFP4 weights dequantised by
   ``axb_nvfp4_dequant``) with their LoRA folded in;
4. COMBINE: expert outputs are scaled by their routing weight and summed per (source rank, token)
   into a local partial buffer (``axb_ep_scatter_add``); after one more flag barrier the source adds
   one partial row per contributing rank with peer loads (``axb_ep_reduce_rows``).
The backward pass is the mirror image (combine^T = gather of dY rows, dispatch^T = scatter-add of dX
rows). Expert weights and expert-LoRA slices follow the reference's layout rules
(src/axolotl/integrations/expert_parallel/shard.py:56-393): rank r owns experts
[r*E/ep, (r+1)*E/ep); A is expert-major ([E*r, in] rows), B is rank-major ([out, r, E] view).
On CPU (gloo) the plan and the payload move with ``all_to_all_single`` (host-side split sizes) so the same
logic is testable without GPUs.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _lib
from .symm import PeerSync, SymmBuffer


class _Plan:
    """Routing plan of one MoE layer call (shared by forward and backward)."""
    __slots__ = ("T", "k", "H", "send_order", "send_counts", "recv_counts", "recv_src_rank", "recv_src_row",
                 "recv_weight", "local_order", "expert_counts", "n_recv", "send_tok", "lay", "pad_src_rank", "pad_src_row",
                 "pad_weight", "pad_src_slot", "need", "sent", "x_buf")


class ExpertParallelGroup:
    def __init__(self, device, group, size, rank, num_experts):
        self.device, self.group, self.size, self.rank = torch.device(device), group, size, rank
        if num_experts % size:
            raise ValueError(f"{num_experts} experts are not divisible by expert_parallel_size={size}")
        self.E, self.E_local = num_experts, num_experts // size
        self.fused = self.device.type == "cuda"
        self.x_bufs = self.y_bufs = None
        self.p_bufs = self.staging = None
        self.kx = self.ky = 0
        # Deduplicated payload (default): a token with several slots on one rank crosses NVLink once in
        # each direction (rows are staged / partially summed per rank pair). AXB_EP_DEDUP=0 moves one row
        # per slot straight between the ranks instead.
        self.dedup = os.environ.get("AXB_EP_DEDUP", "1") != "0"
        # Transport of the staged rows: "sm" (default) = only the needed rows by a copy kernel; "ce" = whole
        # peer buffers by the copy engines (peer cudaMemcpyAsync). Measured on the 2-GPU Qwen3-MoE step:
        # 370.9 ms with the row kernels, 384.3 ms with the copy engines (more bytes, one copy per peer);
        # on 8 GPUs 442.7 ms against 592.1 ms.
        self.stage_by = os.environ.get("AXB_EP_STAGE", "sm")
        # Device-side plan: rows this rank may receive per layer call = capacity_factor x (its own slots), capped
        # at the worst case (every slot of every rank). AXB_EP_PLAN=host keeps the NCCL + host-sync plan.
        self.capacity_factor = float(os.environ.get("AXB_EP_CAPACITY", "2.0"))
        self.device_plan = self.fused and os.environ.get("AXB_EP_PLAN", "device") != "host"
        self.t_bufs = self.s_bufs = None
        self.kt = self.ks = 0
        self.overflow = torch.zeros(1, dtype=torch.int32, device=self.device) if self.fused else None
        if self.fused:
            self.sync = PeerSync(self.device, group)

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def shard_experts(self, model):
        from ..models.moe import Experts, SparseMoE

        r, n, El = self.rank, self.size, self.E_local
        for m in model.modules():
            if not isinstance(m, SparseMoE):
                continue
            ex: Experts = m.experts
            lo, hi = r * El, (r + 1) * El
            if ex.nvfp4 is not None:
                for which in ("gate_up", "down"):
                    q = ex.nvfp4[which]
                    ex.nvfp4[which] = {k: v[lo:hi].contiguous() for k, v in q.items()}
            else:
                ex.gate_up_proj = torch.nn.Parameter(ex.gate_up_proj.detach()[lo:hi].contiguous().clone(),
                                                     requires_grad=ex.gate_up_proj.requires_grad)
                ex.down_proj = torch.nn.Parameter(ex.down_proj.detach()[lo:hi].contiguous().clone(),
                                                  requires_grad=ex.down_proj.requires_grad)
            if ex.lora is not None:
                rr = ex.lora_r
                new = {}
                for which in ("gate_up", "down"):
                    A, B = ex.lora[which + "_A"], ex.lora[which + "_B"]
                    new[which + "_A"] = torch.nn.Parameter(A.detach()[lo * rr:hi * rr].contiguous().clone())
                    new[which + "_B"] = torch.nn.Parameter(
                        B.detach().view(B.shape[0], rr, self.E)[:, :, lo:hi].reshape(B.shape[0], rr * El).contiguous().clone())
                ex.lora = torch.nn.ParameterDict(new)
                for p in ex.lora.values():
                    p._tp_sharded = True   # unique per rank: never reduced over the EP group
            ex.E, ex.expert_offset = El, lo
            for p in ex.parameters():
                p._tp_sharded = True
            m.ep = self
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    @torch.no_grad()
    def gather_expert_lora(self, ex):
        """Full-size expert adapter tensors in PEFT layout (adapter saving)."""
        out = {}
        rr, El = ex.lora_r, self.E_local
        for which in ("gate_up", "down"):
            A, B = ex.lora[which + "_A"].detach().contiguous(), ex.lora[which + "_B"].detach().contiguous()
            As = [torch.empty_like(A) for _ in range(self.size)]
            Bs = [torch.empty_like(B) for _ in range(self.size)]
            dist.all_gather(As, A, group=self.group)
            dist.all_gather(Bs, B, group=self.group)
            out[which + "_A"] = torch.cat(As, 0)
            out[which + "_B"] = torch.cat([b.view(b.shape[0], rr, El) for b in Bs], 2).reshape(B.shape[0], rr * self.E)
        return out

    # ------------------------------------------------------------------ plan
    def _make_plan(self, idx, w, H):
        T, k = idx.shape
        dev = idx.device
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)                 # grouped by destination rank, then expert
        dest = (flat_e // self.E_local)
        # counts by scatter-add: torch.bincount synchronises with the host to size its output
        send_counts = torch.zeros(self.size, dtype=torch.int64, device=dev).scatter_add_(
            0, dest.long(), torch.ones_like(dest, dtype=torch.int64))
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # the ONE host synchronisation of the plan: NCCL needs the split sizes of the slot exchange
        both = torch.stack([send_counts, recv_counts]).tolist()
        sc, rc = both[0], both[1]
        n_recv = sum(rc)
        tok = (order // k).to(torch.int32)
        loc_e = (flat_e[order] % self.E_local).to(torch.int32)
        wt = w.reshape(-1)[order].float()
        # one exchange for the three per-slot fields: [token row, local expert, routing weight bits]
        send = torch.stack([tok, loc_e, wt.detach().contiguous().view(torch.int32)], 1).contiguous()
        recv = torch.empty((n_recv, 3), dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv, send, rc, sc, group=self.group)
        r_tok, r_e = recv[:, 0].contiguous(), recv[:, 1].contiguous()
        r_w = recv[:, 2].contiguous().view(torch.float32)
        src_rank = torch.repeat_interleave(torch.arange(self.size, device=dev, dtype=torch.int32),
                                           recv_counts, output_size=n_recv)
        local_order = torch.argsort(r_e, stable=True)
        p = _Plan()
        p.T, p.k, p.H = T, k, H
        p.send_order, p.send_counts, p.recv_counts = order, sc, rc
        p.recv_src_rank = src_rank[local_order].contiguous()
        p.recv_src_row = r_tok[local_order].contiguous()
        p.recv_weight = r_w[local_order].contiguous()
        p.local_order = local_order
        counts_dev = torch.zeros(self.E_local, dtype=torch.int64, device=dev).scatter_add_(
            0, r_e.long(), torch.ones(n_recv, dtype=torch.int64, device=dev))
        # host copy only where the per-expert loop of the unfused path needs it
        p.expert_counts = None if self.fused else counts_dev.tolist()
        p.n_recv = n_recv
        p.send_tok = tok
        p.lay = None
        if self.fused:
            # expert segments padded to 128 rows for the grouped GEMM; -1 marks pad rows
            from ..ops.grouped import GroupLayout

            lay = GroupLayout(counts_dev, n_recv)
            p.lay = lay
            p.pad_src_rank = torch.full((lay.max_rows,), -1, dtype=torch.int32, device=dev)
            p.pad_src_rank[lay.dest] = p.recv_src_rank
            p.pad_src_row = torch.zeros(lay.max_rows, dtype=torch.int32, device=dev)
            p.pad_src_row[lay.dest] = p.recv_src_row
            p.pad_weight = torch.zeros(lay.max_rows, dtype=torch.float32, device=dev)
            p.pad_weight[lay.dest] = p.recv_weight
            if self.dedup:
                # need[r*T + row]: this rank computes at least one slot of rank r's token `row`;
                # sent[r*T + row]: rank r computes at least one slot of this rank's token `row`
                p.need = torch.zeros(self.size * T, dtype=torch.uint8, device=dev)
                p.need[p.recv_src_rank.long() * T + p.recv_src_row.long()] = 1
                p.sent = torch.zeros(self.size * T, dtype=torch.uint8, device=dev)
                p.sent[dest.long() * T + torch.arange(T * k, device=dev) // k] = 1
        return p

    # ------------------------------------------------------------------ device-side plan
    def _capacity(self, n):
        cap = min(self.size * n, int(-(-self.capacity_factor * n // 1)))
        return max(128, (cap + 127) // 128 * 128)

    def _ensure_tables(self, n):
        if self.t_bufs is None or self.t_bufs[0].tensor.numel() < 2 * n:
            self.t_bufs = [SymmBuffer(2 * n, torch.int32, self.device, self.group, use_multicast=False) for _ in range(2)]
            self.s_bufs = [SymmBuffer(n, torch.float32, self.device, self.group, use_multicast=False) for _ in range(2)]
            dist.barrier(self.group)

    def _publish(self, x, idx, w):
        """This rank's token rows and routing table into symmetric memory; one barrier publishes both."""
        T, H = x.shape
        n = idx.numel()
        self._ensure(T, H)
        self._ensure_tables(n)
        buf = self.x_bufs[self.kx & 1]
        self.kx += 1
        buf.tensor[: T * H].view(T, H).copy_(x.detach())
        tab = self.t_bufs[self.kt & 1]
        self.kt += 1
        tab.tensor[:n].copy_(idx.reshape(-1))
        tab.tensor[n:2 * n].copy_(w.detach().reshape(-1).float().view(torch.int32))
        self.sync.barrier(channel=6)
        return buf, tab

    def _make_plan_device(self, idx, H, tab):
        """The plan from every rank's routing table, computed on the device with static shapes."""
        from ..ops.grouped import BLOCK, GroupLayout

        T, k = idx.shape
        n, W, El, dev = T * k, self.size, self.E_local, idx.device
        allt = torch.empty((W, 2, n), dtype=torch.int32, device=dev)
        _lib.check_rc(_lib.cuda_lib().axb_ep_gather_tables(tab.ptrs_c, W, 2 * n, allt.data_ptr(), _lib.stream_ptr()),
                      "ep_gather_tables")
        return self._plan_from_tables(allt[:, 0].reshape(-1), allt[:, 1].reshape(-1).view(torch.float32), idx, H)

    def _plan_from_tables(self, all_idx, all_w, idx, H):
        """``all_idx`` / ``all_w``: the routing tables of all ranks, rank-major, flattened [W * T * k]."""
        from ..ops.grouped import BLOCK, GroupLayout

        T, k = idx.shape
        n, W, El, dev = T * k, self.size, self.E_local, idx.device
        mine = torch.div(all_idx, El, rounding_mode="floor") == self.rank
        flat = torch.where(mine, all_idx % El, El)                      # local expert id, El = not for this rank
        cap = self._capacity(n)
        order = torch.argsort(flat, stable=True)[:cap]                  # expert-sorted, rank-major inside an expert
        e_sorted = flat[order]
        valid = e_sorted < El
        counts = torch.zeros(El + 1, dtype=torch.int64, device=dev).scatter_add_(
            0, flat.long(), torch.ones(flat.numel(), dtype=torch.int64, device=dev))[:El]
        if self.overflow is None:
            self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overflow += (counts.sum() > cap).to(torch.int32)
        padded = (counts + (BLOCK - 1)) // BLOCK * BLOCK
        seg_end = padded.cumsum(0)
        seg_start = seg_end - padded
        first = counts.cumsum(0) - counts
        lay = GroupLayout.__new__(GroupLayout)
        lay.E, lay.n_rows = El, cap
        lay.max_blocks = cap // BLOCK + El
        lay.max_rows = lay.max_blocks * BLOCK
        e_c = e_sorted.clamp(max=El - 1).long()
        dump = lay.max_rows                                              # rows beyond the received ones land here
        dest = torch.where(valid, seg_start[e_c] + (torch.arange(order.numel(), device=dev) - first[e_c]), dump)
        dest = dest.clamp(max=dump)                                      # (an overflowing call is reported, not trusted)
        lay.dest = dest
        blk_row = torch.arange(lay.max_blocks, device=dev) * BLOCK
        lay.blk_expert = torch.searchsorted(seg_end, blk_row, right=True).clamp(max=El - 1).to(torch.int32)
        lay.n_blocks = (seg_end[-1:] // BLOCK).clamp(max=lay.max_blocks).to(torch.int32)
        lay.seg_start = seg_start.to(torch.int32)
        lay.seg_rows = padded.to(torch.int32)
        lay.prefix_only = True      # rows beyond n_blocks * 128 are never written or read (capacity slack)
        src_rank = torch.div(order, n, rounding_mode="floor").to(torch.int32)
        src_slot = (order % n).to(torch.int32)
        p = _Plan()
        p.T, p.k, p.H, p.lay = T, k, H, lay
        p.n_recv = cap
        neg = torch.full((), -1, dtype=torch.int32, device=dev)
        p.pad_src_rank = torch.full((lay.max_rows + 1,), -1, dtype=torch.int32, device=dev)
        p.pad_src_rank[dest] = torch.where(valid, src_rank, neg)
        p.pad_src_rank = p.pad_src_rank[: lay.max_rows]
        p.pad_src_slot = torch.full((lay.max_rows + 1,), -1, dtype=torch.int32, device=dev)
        p.pad_src_slot[dest] = torch.where(valid, src_slot, neg)
        p.pad_src_slot = p.pad_src_slot[: lay.max_rows]
        p.pad_src_row = torch.div(p.pad_src_slot.clamp(min=0), k, rounding_mode="floor").to(torch.int32)
        p.pad_weight = torch.zeros(lay.max_rows + 1, dtype=torch.float32, device=dev)
        p.pad_weight[dest] = torch.where(valid, all_w[order], torch.zeros((), device=dev))
        p.pad_weight = p.pad_weight[: lay.max_rows]
        if self.dedup:
            lin = torch.where(valid, src_rank.long() * T + torch.div(src_slot, k, rounding_mode="floor").long(), W * T)
            p.need = torch.zeros(W * T + 1, dtype=torch.uint8, device=dev)
            p.need[lin] = 1
            dest_rank = torch.div(idx.reshape(-1), El, rounding_mode="floor").long()
            p.sent = torch.zeros(W * T, dtype=torch.uint8, device=dev)
            p.sent[dest_rank * T + torch.arange(n, device=dev) // k] = 1
        return p

    def take_overflow(self) -> bool:
        """True when ANY rank of the group received more rows than its capacity in a layer call since the last
        check (rows were dropped there, so this step's gradients are incomplete on every rank). The capacity factor
        then grows by half (up to the group size, where no overflow is possible) and the caller skips the update.
        One small device all-reduce and one host read per optimizer step."""
        if self.overflow is None:
            return False
        flag = self.overflow.to(torch.float32)
        if self.fused and self.size > 1:
            self.sync.all_reduce_(flag, channel=2)
        hit = float(flag.item()) > 0
        if hit:
            self.overflow.zero_()
            self.skipped_steps = getattr(self, "skipped_steps", 0) + 1
            old = self.capacity_factor
            self.capacity_factor = min(float(self.size), old * 1.5)
            from ..utils.logging import get_logger

            get_logger(__name__).warning(
                "expert parallelism: a rank received more than %.2f x its own slots in one layer call; this optimizer "
                "step is skipped and the capacity factor grows to %.2f (set expert_parallel_capacity_factor / "
                "AXB_EP_CAPACITY to start higher)", old, self.capacity_factor)
        return hit

    def check_overflow(self):
        """Raises when a layer call since the last check dropped rows (for callers that cannot skip a step)."""
        if self.take_overflow():
            raise RuntimeError("expert parallelism: rows were dropped in a layer call (capacity factor too small); "
                               "raise AXB_EP_CAPACITY (up to the group size)")

    def return_slot_scalars_fused(self, vals_pad, plan):
        """Per-slot scalars of the padded rows -> [T, k] at the rank that routed the slot (peer stores)."""
        n = plan.T * plan.k
        sb = self.s_bufs[self.ks & 1]
        self.ks += 1
        _lib.check_rc(_lib.cuda_lib().axb_ep_put_scalars(
            sb.ptrs_c, self.size, plan.pad_src_rank.data_ptr(), plan.pad_src_slot.data_ptr(),
            vals_pad.contiguous().data_ptr(), plan.lay.max_rows, n, _lib.stream_ptr()), "ep_put_scalars")
        self.sync.barrier(channel=8)
        return sb.tensor[:n].view(plan.T, plan.k).clone()

    def _ensure(self, T, H):
        if not self.fused:
            return
        need = T * H
        if self.x_bufs is None or self.x_bufs[0].tensor.numel() < need:
            self.x_bufs = [SymmBuffer(need, torch.bfloat16, self.device, self.group, use_multicast=False) for _ in range(2)]
            self.y_bufs = [SymmBuffer(need, torch.bfloat16, self.device, self.group, use_multicast=False) for _ in range(2)]
            if self.dedup:
                self.p_bufs = [SymmBuffer(self.size * need, torch.bfloat16, self.device, self.group, use_multicast=False)
                               for _ in range(2)]
                self.staging = torch.empty(self.size * need, dtype=torch.bfloat16, device=self.device)
            dist.barrier(self.group)

    def _slices(self, base, stride_bytes, own):
        """Pointer table for the row kernels: slice r of a local [world, T, H] buffer, this rank's own
        entry replaced by ``own`` (its rows need no staging)."""
        from .symm import _u64_array

        return _u64_array([own if r == self.rank else base + r * stride_bytes for r in range(self.size)])

    # ------------------------------------------------------------------ payload movement
    def pull_rows(self, x, plan, weighted=False, dot_with=None):
        """Rows routed to this rank's experts, expert-sorted. Fused path: the padded layout
        [lay.max_rows, H] (zeros in pad rows), optionally scaled by the routing weight, and
        optionally the per-row dot product of the unscaled row with ``dot_with``. Collective path:
        compact [n_recv, H]."""
        if not self.fused:
            return _a2a_rows(x[plan.send_tok.long()], plan.recv_counts, plan.send_counts, self.group)[plan.local_order]
        lib = _lib.cuda_lib()
        T, H = x.shape
        buf = getattr(plan, "x_buf", None)
        plan.x_buf = None
        if buf is None:      # (the forward dispatch of the device-side plan published x with the routing table)
            self._ensure(T, H)
            buf = self.x_bufs[self.kx & 1]
            self.kx += 1
            buf.tensor[: T * H].view(T, H).copy_(x)
            self.sync.barrier(channel=6)
        n = plan.lay.max_rows
        out = torch.empty((n, H), dtype=x.dtype, device=x.device)
        dots = torch.empty(n, dtype=torch.float32, device=x.device) if dot_with is not None else None
        src_ptrs = buf.ptrs_c
        if self.dedup:   # rows of every peer -> local staging, then a local gather
            if self.stage_by == "ce":
                for r in range(self.size):
                    if r != self.rank:
                        self.staging[r * T * H:(r + 1) * T * H].copy_(
                            buf.handle.get_buffer(r, (T * H,), torch.bfloat16, 0), non_blocking=True)
            else:
                _lib.check_rc(lib.axb_ep_stage_rows(buf.ptrs_c, self.size, self.rank, plan.need.data_ptr(),
                                                    self.staging.data_ptr(), T, H, _lib.stream_ptr()), "ep_stage_rows")
            src_ptrs = self._slices(self.staging.data_ptr(), T * H * 2, buf.tensor.data_ptr())
        args = (src_ptrs, self.size, plan.pad_src_rank.data_ptr(), plan.pad_src_row.data_ptr(),
                plan.pad_weight.data_ptr() if weighted else None, dot_with.data_ptr() if dot_with is not None else None,
                dots.data_ptr() if dots is not None else None, out.data_ptr(), n, H, H)
        if getattr(plan.lay, "prefix_only", False):
            _lib.check_rc(lib.axb_ep_gather_rows_n(*args, plan.lay.n_blocks.data_ptr(), _lib.stream_ptr()), "ep_gather_rows")
        else:
            _lib.check_rc(lib.axb_ep_gather_rows(*args, _lib.stream_ptr()), "ep_gather_rows")
        return out if dot_with is None else (out, dots)

    def push_rows(self, rows, plan, weighted):
        """sum over slots of (weight *) rows back at their source token: [T, H] on the source rank."""
        T, H = plan.T, plan.H
        if not self.fused:
            r = rows * plan.recv_weight[:, None].to(rows.dtype) if weighted else rows
            inv = torch.empty_like(plan.local_order)
            inv[plan.local_order] = torch.arange(len(inv), device=inv.device)
            back = _a2a_rows(r[inv], plan.send_counts, plan.recv_counts, self.group)
            y = torch.zeros(T, H, dtype=rows.dtype, device=rows.device)
            y.index_add_(0, plan.send_tok.long(), back)
            return y
        lib = _lib.cuda_lib()
        self._ensure(T, H)
        rows = rows.contiguous()
        if self.dedup:
            # Slots are summed per (source rank, token) locally; the source then pulls one partial row per
            # contributing rank. The partial buffer alternates between two allocations: by the time one is
            # zeroed again every peer has passed the barrier of the call in between, i.e. finished reading it.
            part = self.p_bufs[self.ky & 1]
            self.ky += 1
            part.tensor[: self.size * T * H].zero_()
            y = torch.zeros(T, H, dtype=rows.dtype, device=rows.device)
            dst_ptrs = self._slices(part.tensor.data_ptr(), T * H * 2, y.data_ptr())
            _lib.check_rc(lib.axb_ep_scatter_add(dst_ptrs, self.size, plan.pad_src_rank.data_ptr(),
                                                 plan.pad_src_row.data_ptr(),
                                                 plan.pad_weight.data_ptr() if weighted else None, rows.data_ptr(),
                                                 plan.lay.max_rows, H, H, _lib.stream_ptr()), "ep_scatter_add")
            self.sync.barrier(channel=7)
            part_ptrs = part.ptrs_c
            if self.stage_by == "ce":
                # every peer's partial slice for this rank -> local staging by the copy engines; the
                # reduce kernel then reads local memory (its pointer table is biased so that
                # "slice `rank` of peer r" lands on staging slice r)
                from .symm import _u64_array

                for r in range(self.size):
                    if r != self.rank:
                        self.staging[r * T * H:(r + 1) * T * H].copy_(
                            part.handle.get_buffer(r, (T * H,), torch.bfloat16, self.rank * T * H), non_blocking=True)
                base = self.staging.data_ptr()
                part_ptrs = _u64_array([base + (r - self.rank) * T * H * 2 for r in range(self.size)])
            _lib.check_rc(lib.axb_ep_reduce_rows(part_ptrs, self.size, self.rank, plan.sent.data_ptr(), y.data_ptr(),
                                                 T, H, _lib.stream_ptr()), "ep_reduce_rows")
            return y
        buf = self.y_bufs[self.ky & 1]     # zero on every rank since its last use
        self.ky += 1
        _lib.check_rc(lib.axb_ep_scatter_add(buf.ptrs_c, self.size, plan.pad_src_rank.data_ptr(),
                                             plan.pad_src_row.data_ptr(),
                                             plan.pad_weight.data_ptr() if weighted else None, rows.data_ptr(),
                                             plan.lay.max_rows, H, H, _lib.stream_ptr()), "ep_scatter_add")
        self.sync.barrier(channel=7)
        y = buf.tensor[: T * H].view(T, H).clone()
        buf.tensor[: T * H].zero_()
        return y

    def return_slot_scalars(self, vals, plan):
        """per-slot scalars computed at the expert rank -> [T, k] at the source rank."""
        inv = torch.empty_like(plan.local_order)
        inv[plan.local_order] = torch.arange(len(inv), device=inv.device)
        send = vals[inv].contiguous()
        back = torch.empty(plan.T * plan.k, dtype=vals.dtype, device=vals.device)
        dist.all_to_all_single(back, send, plan.send_counts, plan.recv_counts, group=self.group)
        out = torch.empty_like(back)
        out[plan.send_order] = back
        return out.view(plan.T, plan.k)

    # ------------------------------------------------------------------ layer entry
    def dispatch_compute_combine(self, experts, x, w, idx):
        if self.device_plan:
            x = x.contiguous()
            buf, tab = self._publish(x, idx.to(torch.int32), w)
            plan = self._make_plan_device(idx, x.shape[1], tab)
            plan.x_buf = buf
        else:
            plan = self._make_plan(idx, w, x.shape[1])
        xs = _Dispatch.apply(x, self, plan)
        if self.fused:
            from ..ops.grouped import grouped_experts_padded

            ys = grouped_experts_padded(experts, xs, plan.lay)
        else:
            ys = experts(xs, plan.expert_counts)
        return _Combine.apply(ys, w, self, plan)


def _a2a_rows(rows, out_counts, in_counts, group):
    out = torch.empty((sum(out_counts), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), out_counts, in_counts, group=group)
    return out


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep, plan):
        ctx.ep, ctx.plan = ep, plan
        return ep.pull_rows(x.contiguous(), plan)

    @staticmethod
    def backward(ctx, dxs):
        return ctx.ep.push_rows(dxs, ctx.plan, weighted=False), None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, w, ep, plan):
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(ys)
        ctx.w_dtype = w.dtype
        return ep.push_rows(ys, plan, weighted=True)

    @staticmethod
    def backward(ctx, dy):
        (ys,) = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        if ep.fused:   # one peer gather: weight-scaled dY rows and <dY row, expert output row>
            if ctx.needs_input_grad[1]:
                dys, dots = ep.pull_rows(dy.contiguous(), plan, weighted=True, dot_with=ys.contiguous())
                if ep.device_plan:
                    dw = ep.return_slot_scalars_fused(dots, plan).to(ctx.w_dtype)
                else:
                    dw = ep.return_slot_scalars(dots[plan.lay.dest], plan).to(ctx.w_dtype)
            else:
                dys, dw = ep.pull_rows(dy.contiguous(), plan, weighted=True), None
            return dys, dw, None, None
        dy_rows = ep.pull_rows(dy.contiguous(), plan)                     # dY of each slot's token
        dys = dy_rows * plan.recv_weight[:, None].to(dy_rows.dtype)
        dw = None
        if ctx.needs_input_grad[1]:
            dw_slots = (dy_rows.float() * ys.float()).sum(-1)
            dw = ep.return_slot_scalars(dw_slots, plan).to(ctx.w_dtype)
        return dys, dw, None, None
