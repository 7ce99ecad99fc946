"""FSDP-style sharding of the frozen base weights with the all-gather fused into the GEMM.

Every ``FusedLinear`` weight [N, K] is row-sharded: rank r keeps rows [r*N/W, (r+1)*N/W) inside
one symmetric arena. Forward (x W^T) and input-gradient (dY W) GEMMs run the
``axb_gemm_bf16_allgather`` kernel: while the tensor cores work on tile t, a gather warp in every
CTA pulls 8 KB chunks of the peers' shards over NVLink into a local staging buffer and flags
256-row blocks as ready for the TMA producer. Nothing is gathered ahead of time and nothing
stays resident: per-GPU weight memory is 1/W of the model plus one staging buffer of the largest
weight. Because the base is frozen its shards never change, so no inter-rank synchronisation is
needed around the gathers at all.

This is the B200 counterpart of the reference's per-layer ``fully_shard`` units + NCCL all-gather
(src/axolotl/monkeypatch/accelerate/fsdp2.py:539-802).
"""
from __future__ import annotations

import torch

from ..models.layers import FusedLinear
from ..utils.logging import get_logger
from .symm import SymmBuffer

LOG = get_logger(__name__)


class ShardInfo:
    __slots__ = ("rows", "cols", "world", "rank", "peer_bases_dev", "shard_offset", "shard_bytes", "ctx")

    def __init__(self, rows, cols, world, rank, peer_bases_dev, shard_offset, shard_bytes, ctx):
        self.rows, self.cols, self.world, self.rank = rows, cols, world, rank
        self.peer_bases_dev, self.shard_offset, self.shard_bytes, self.ctx = peer_bases_dev, shard_offset, shard_bytes, ctx


class FSDPContext:
    """Owns the shard arena, the staging buffer and the ready counters of one sharding group."""

    def __init__(self, device, group, world, rank):
        self.device, self.group, self.world, self.rank = device, group, world, rank
        self.arena = None
        self.staging = None
        self.ready = None
        self.sharded = []

    @staticmethod
    def shardable(m: FusedLinear, world: int) -> bool:
        N, K = m.weight.shape
        if m.weight.dtype != torch.bfloat16:
            return False
        row_bytes = 2 * K
        return (N % 256 == 0 and N % world == 0 and (256 * row_bytes) % 8192 == 0
                and ((N // world) * row_bytes) % 8192 == 0 and N // world >= 1)

    @torch.no_grad()
    def shard_model(self, model):
        mods = [m for _, m in model.fused_linears() if self.shardable(m, self.world) and not m.weight.requires_grad]
        total = sum(m.weight.numel() // self.world for m in mods)
        if total == 0:
            return 0
        buf = SymmBuffer(total, torch.bfloat16, self.device, self.group, use_multicast=False)
        self.arena = buf
        max_full = max(m.weight.numel() for m in mods)
        max_rows = max(m.weight.shape[0] for m in mods)
        self.staging = torch.empty(max_full, dtype=torch.bfloat16, device=self.device)
        self.ready = torch.zeros(max_rows // 256 + 1, dtype=torch.int32, device=self.device)
        off = 0
        for m in mods:
            N, K = m.weight.shape
            rows = N // self.world
            n = rows * K
            shard = buf.tensor[off:off + n].view(rows, K)
            shard.copy_(m.weight[self.rank * rows:(self.rank + 1) * rows])
            info = ShardInfo(N, K, self.world, self.rank, buf.ptrs_dev, off * 2, n * 2, self)
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

    @torch.no_grad()
    def gather_full_weight(self, m: FusedLinear) -> torch.Tensor:
        """Full [N, K] weight assembled from all ranks (checkpoint saving; NCCL all-gather)."""
        import torch.distributed as dist

        info = m.weight._axb_shard
        out = torch.empty(info.rows, info.cols, dtype=m.weight.dtype, device=self.device)
        dist.all_gather_into_tensor(out, m.weight.data.contiguous(), group=self.group)
        return out
