"""N-D device mesh with the axis order and sizing rules of the reference
(src/axolotl/monkeypatch/accelerate/parallelism_config.py:85-92, src/axolotl/utils/distributed.py:299-382):
axes ``(ep, dp_replicate, dp_shard, cp, tp)``, fastest-varying last; ``dp_shard`` is inferred from
the world size when left unset; expert-parallel ranks count as data-parallel for the dataloader;
TP and CP ranks do not multiply the global batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

AXES = ("ep", "dp_replicate", "dp_shard", "cp", "tp")


@dataclass
class MeshSpec:
    ep: int = 1
    dp_replicate: int = 1
    dp_shard: int = 1
    cp: int = 1
    tp: int = 1

    @classmethod
    def from_cfg(cls, world_size, *, tensor_parallel_size=1, context_parallel_size=1,
                 dp_shard_size=None, dp_replicate_size=None, expert_parallel_size=1):
        tp, cp, ep = tensor_parallel_size or 1, context_parallel_size or 1, expert_parallel_size or 1
        rep = dp_replicate_size or 1
        rest = tp * cp * ep * rep
        if world_size % rest:
            raise ValueError(f"world size {world_size} is not divisible by tp*cp*ep*dp_replicate = {rest}")
        shard = dp_shard_size if dp_shard_size else world_size // rest
        if shard * rest != world_size:
            raise ValueError(f"mesh {dict(ep=ep, dp_replicate=rep, dp_shard=shard, cp=cp, tp=tp)} "
                             f"does not cover world size {world_size}")
        return cls(ep=ep, dp_replicate=rep, dp_shard=shard, cp=cp, tp=tp)

    @property
    def shape(self):
        return tuple(getattr(self, a) for a in AXES)

    @property
    def world_size(self):
        return math.prod(self.shape)

    @property
    def data_parallel_size(self):
        """Ranks that consume distinct batches (ep counts, cp/tp do not)."""
        return self.ep * self.dp_replicate * self.dp_shard

    def coords(self, rank):
        out, r = {}, rank
        for a in reversed(AXES):
            n = getattr(self, a)
            out[a] = r % n
            r //= n
        return out

    def rank_of(self, **coords):
        r = 0
        for a in AXES:
            r = r * getattr(self, a) + coords.get(a, 0)
        return r

    def group_ranks(self, rank, axes):
        """Ranks that share every coordinate of ``rank`` except along ``axes`` (ordered)."""
        if isinstance(axes, str):
            axes = (axes,)
        base = self.coords(rank)
        ranks = [dict(base)]
        for a in AXES:
            if a in axes:
                ranks = [dict(c, **{a: i}) for c in ranks for i in range(getattr(self, a))]
        return sorted(self.rank_of(**c) for c in ranks)

    def all_groups(self, axes):
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(self.group_ranks(r, axes))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out


class DeviceMesh:
    """Process groups for every axis (and the fused axes FSDP needs) of a MeshSpec."""

    def __init__(self, spec: MeshSpec, rank: int, backend: str | None = None, timeout=None):
        import torch.distributed as dist

        self.spec, self.rank = spec, rank
        self.groups = {}
        self._ranks = {}
        combos = [(a,) for a in AXES] + [("dp_shard", "cp"), ("dp_replicate", "dp_shard"),
                                         ("ep", "dp_replicate", "dp_shard")]
        for axes in combos:
            size = math.prod(getattr(spec, a) for a in axes)
            key = "_".join(axes)
            mine = spec.group_ranks(rank, axes)
            self._ranks[key] = mine
            if size == 1:
                self.groups[key] = None
                continue
            if size == spec.world_size:
                self.groups[key] = dist.group.WORLD
                continue
            for g in spec.all_groups(axes):  # every rank must create every group, in the same order
                kw = {"timeout": timeout} if timeout is not None else {}
                pg = dist.new_group(g, backend=backend, **kw)
                if rank in g:
                    self.groups[key] = pg

    def group(self, *axes):
        return self.groups["_".join(axes)]

    def ranks(self, *axes):
        return self._ranks["_".join(axes)]

    def size(self, *axes):
        return math.prod(getattr(self.spec, a) for a in axes)

    def coord(self, axis):
        return self.spec.coords(self.rank)[axis]
