"""FSDP-style sharding of the frozen base weights with the all-gather overlapped with the GEMMs.

Every ``FusedLinear`` weight [N, K] is row-sharded: rank r keeps rows [r*N/W, (r+1)*N/W) inside
one symmetric arena. Forward (x W^T) and input-gradient (dY W) GEMMs read the full weight from
one of two local staging buffers; while the GEMM on weight k runs, the shards of weight k+1 of the
layer schedule are pulled out of the peers' memory over NVLink into the other staging buffer.
Two transports exist for that pull. (a) The copy engines (default): one peer copy per rank on a
side stream, ordered by events after the last reader of the buffer and before its next reader; no
SM is taken from the MMAs. (b) Gather CTAs inside the GEMM launch (``axb_gemm_bf16_prefetch``):
a few extra CTAs of the same kernel copy the shards with bulk loads, so stream order is the only
synchronisation; this costs the tensor-core kernel some SMs (measured 6 % of the 2-GPU step).
A weight that was not predicted is fetched by a stand-alone all-gather launch. Per-GPU weight
memory is 1/W of the model plus two staging buffers of the largest weight. Because the base is
frozen its shards never change, so no inter-rank synchronisation is needed around the gathers.

This is the B200 counterpart of the reference's per-layer ``fully_shard`` units + NCCL all-gather
(src/axolotl/monkeypatch/accelerate/fsdp2.py:539-802).
"""
from __future__ import annotations

import os

import torch

from ..models.layers import FusedLinear
from ..utils.logging import get_logger
from .symm import SymmBuffer

LOG = get_logger(__name__)


class ShardInfo:
    __slots__ = ("rows", "cols", "world", "rank", "peer_bases_dev", "shard_offset", "shard_bytes", "ctx", "index")

    def __init__(self, rows, cols, world, rank, peer_bases_dev, shard_offset, shard_bytes, ctx):
        self.rows, self.cols, self.world, self.rank = rows, cols, world, rank
        self.peer_bases_dev, self.shard_offset, self.shard_bytes, self.ctx = peer_bases_dev, shard_offset, shard_bytes, ctx


class FSDPContext:
    """Owns the shard arena, the staging buffers and the prefetch state of one sharding group."""

    NS = 3   # staging buffers: the GEMM's own operand plus a prefetch distance of two

    def __init__(self, device, group, world, rank, reshard_after_forward=True):
        self.device, self.group, self.world, self.rank = device, group, world, rank
        # False: every weight gets a staging buffer of its own, so what the forward pass gathered is still
        # there when the backward pass needs it (one gather per step instead of two, at the price of a full
        # copy of the frozen weights); the copies are dropped when the step ends, as FSDP2 reshards them.
        self.reshard_after_forward = bool(reshard_after_forward)
        self.arena = None
        self.staging = [None] * self.NS   # full-size buffers; weight i of the schedule lives in buffer i % NS
        self.holds = [None] * self.NS     # weight (ShardInfo) each buffer holds, in stream order
        self.order = []               # sharded weights in forward execution order
        self.sharded = []
        self.stats = {"prefetched": 0, "standalone": 0}
        # Planning figures for the number of gather CTAs per launch. Swept on 2 GPUs (Llama-3-8B LoRA
        # step): under-provisioning exposes the gather (16 CTAs max / 80 GB/s assumed: 362 ms/step),
        # 32-64 CTAs max at 20-40 GB/s assumed all land at 333-335 ms/step.
        self.bytes_per_cta_s = float(os.environ.get("AXB_FSDP_CTA_GBS", "40")) * 1e9
        self.max_prefetch_ctas = int(os.environ.get("AXB_FSDP_MAX_CTAS", "40"))
        # Transport of the prefetch. Default: the copy engines (peer cudaMemcpyAsync on a side stream, ordered
        # by events against the GEMMs that read / reuse the staging buffers), which leaves every SM to the
        # MMAs: 316 ms/step against 335 ms with gather CTAs on the 2-GPU Llama-3-8B LoRA step.
        # AXB_FSDP_COPY_ENGINE=0 selects the gather CTAs inside the GEMM launch instead.
        self.copy_engine = os.environ.get("AXB_FSDP_COPY_ENGINE", "1") == "1"
        self.side_stream = None
        self.pending = [None] * self.NS   # copy-complete event of each staging buffer

    @staticmethod
    def shardable(m: FusedLinear, world: int) -> bool:
        N, K = m.weight.shape
        if m.weight.dtype != torch.bfloat16:
            return False
        row_bytes = 2 * K
        return N % world == 0 and ((N // world) * row_bytes) % 8192 == 0 and N // world >= 1

    @torch.no_grad()
    def shard_model(self, model):
        mods = [m for _, m in model.fused_linears() if self.shardable(m, self.world) and not m.weight.requires_grad
                and getattr(m.weight, "_axb_quant", None) is None]   # 4-bit weights stay replicated (already 4x smaller)
        total = sum(m.weight.numel() // self.world for m in mods)
        if total == 0:
            return 0
        buf = SymmBuffer(total, torch.bfloat16, self.device, self.group, use_multicast=False)
        self.arena = buf
        max_full = max(m.weight.numel() for m in mods)
        if self.reshard_after_forward:
            self.staging = [torch.empty(max_full, dtype=torch.bfloat16, device=self.device) for _ in range(self.NS)]
        else:
            self.NS = len(mods)
            self.staging = [torch.empty(m.weight.numel(), dtype=torch.bfloat16, device=self.device) for m in mods]
            self.holds, self.pending = [None] * self.NS, [None] * self.NS
        off = 0
        for m in mods:
            N, K = m.weight.shape
            rows = N // self.world
            n = rows * K
            shard = buf.tensor[off:off + n].view(rows, K)
            shard.copy_(m.weight[self.rank * rows:(self.rank + 1) * rows])
            info = ShardInfo(N, K, self.world, self.rank, buf.ptrs_dev, off * 2, n * 2, self)
            info.index = len(self.order)
            self.order.append(info)
            p = torch.nn.Parameter(shard, requires_grad=False)
            p._axb_shard = info
            m.weight = p
            m.full_out_features = N
            self.sharded.append(m)
            off += n
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()
        LOG.info("FSDP: sharded %d weights (%.2f GB/rank), staging %.0f MB", len(mods), total * 2 / 1e9,
                 max_full * 2 / 1e6)
        return len(mods)

    # ------------------------------------------------------------------ staging management
    def acquire(self, info: ShardInfo, backward: bool):
        """Returns (staging tensor holding ``info``'s full weight, list of prefetch plans).

        Called in stream order right before the GEMM that consumes the weight. Every plan names a
        weight predicted to be used soon and the buffer it must be gathered into."""
        from ..ops import _lib

        slot = info.index % self.NS
        hit = self.holds[slot] is info
        if self.pending[slot] is not None:   # copy engines are (or were) writing this buffer: order after them
            torch.cuda.current_stream(self.device).wait_event(self.pending[slot])
            self.pending[slot] = None
        if not hit:  # not predicted: fetch now with every SM
            lib = _lib.cuda_lib()
            _lib.check_rc(lib.axb_allgather_rows(info.peer_bases_dev.data_ptr(), info.shard_offset, info.shard_bytes,
                                                 info.world, self.staging[slot].data_ptr(), 0,
                                                 _lib.status_word(self.device).data_ptr(), _lib.stream_ptr()),
                          "allgather_rows")
            self.holds[slot] = info
            self.stats["standalone"] += 1
        # the next weights of the schedule that are not resident yet (distance 1, then 2): a large weight
        # that follows a short GEMM gets two GEMMs' worth of time to arrive
        plans = []
        for d in (1, 2):
            i = info.index + (-d if backward else d)
            if 0 <= i < len(self.order):
                nxt = self.order[i]
                if self.holds[i % self.NS] is not nxt:
                    plans.append((nxt, i % self.NS))
        return self.staging[slot], plans

    def end_of_step(self):
        """``reshard_after_forward: false``: the gathered copies are released with the step."""
        if not self.reshard_after_forward:
            self.holds = [None] * self.NS

    def prefetch_ctas(self, nxt: ShardInfo, gemm_flops: float) -> int:
        """Enough gather CTAs to finish the next weight within this GEMM's run time."""
        t_gemm = gemm_flops / 1.3e15
        need = nxt.shard_bytes * nxt.world / max(t_gemm, 1e-6) / self.bytes_per_cta_s
        return int(min(self.max_prefetch_ctas, max(2, round(need + 0.5))))

    def prefetch_by_copy(self, plan):
        """Issues the all-gather of the planned weight on the copy engines. Called right BEFORE the GEMM
        that reads the other staging buffer is launched: the copies wait for everything already queued on
        the compute stream (the last reader of the buffer they overwrite) and run beside that GEMM."""
        nxt, slot = plan
        main = torch.cuda.current_stream(self.device)
        if self.side_stream is None:
            self.side_stream = torch.cuda.Stream(self.device)
        if self.pending[slot] is not None:      # an earlier, never consumed prefetch into this buffer
            self.side_stream.wait_event(self.pending[slot])
        ev = torch.cuda.Event()
        ev.record(main)
        self.side_stream.wait_event(ev)
        n = nxt.shard_bytes // 2
        dst = self.staging[slot]
        with torch.cuda.stream(self.side_stream):
            for r in range(nxt.world):
                src = self.arena.handle.get_buffer(r, (n,), torch.bfloat16, nxt.shard_offset // 2)
                dst[r * n:(r + 1) * n].copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.side_stream)
        self.pending[slot] = done

    def committed(self, plan):
        nxt, slot = plan
        self.holds[slot] = nxt
        self.stats["prefetched"] += 1

    @torch.no_grad()
    def gather_full_weight(self, m: FusedLinear) -> torch.Tensor:
        """Full [N, K] weight assembled from all ranks (checkpoint saving; NCCL all-gather)."""
        import torch.distributed as dist

        info = m.weight._axb_shard
        out = torch.empty(info.rows, info.cols, dtype=m.weight.dtype, device=self.device)
        dist.all_gather_into_tensor(out, m.weight.data.contiguous(), group=self.group)
        return out
