"""Process-group layout of a job: one rank per GPU arranged as ``pp x dp x sp x tp`` (``ep`` reuses the ``dp x sp``
ranks of a pipeline stage).  ``DistributedInterface`` builds the groups once and hands every subsystem its context
(the reference's experimental stack has the same role in ``v1/accelerator/interface.py:45-233`` with dims
``mp_replicate, mp_shard, dp, cp``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch.distributed as dist


@dataclass
class MeshDims:
    pp: int = 1
    dp: int = 1
    sp: int = 1
    tp: int = 1

    def size(self) -> int:
        return self.pp * self.dp * self.sp * self.tp


def coords(rank: int, dims: MeshDims) -> Dict[str, int]:
    """tp fastest, then sp, dp, pp."""
    tp = rank % dims.tp
    sp = (rank // dims.tp) % dims.sp
    dp = (rank // (dims.tp * dims.sp)) % dims.dp
    pp = rank // (dims.tp * dims.sp * dims.dp)
    return {"pp": pp, "dp": dp, "sp": sp, "tp": tp}


def group_ranks(dims: MeshDims, axis: str) -> List[List[int]]:
    """All groups along ``axis``: ranks that differ only in that coordinate."""
    world = dims.size()
    buckets: Dict[tuple, List[int]] = {}
    for r in range(world):
        c = coords(r, dims)
        key = tuple(v for k, v in c.items() if k != axis)
        buckets.setdefault(key, []).append(r)
    return [sorted(v, key=lambda r: coords(r, dims)[axis]) for v in buckets.values()]


@dataclass
class DistributedInterface:
    dims: MeshDims
    rank: int = 0
    groups: Dict[str, object] = field(default_factory=dict)
    ranks: Dict[str, List[int]] = field(default_factory=dict)

    @classmethod
    def create(cls, pp: int = 1, dp: Optional[int] = None, sp: int = 1, tp: int = 1) -> "DistributedInterface":
        world = dist.get_world_size() if dist.is_initialized() else 1
        if dp is None:
            assert world % (pp * sp * tp) == 0, "world size does not factor into pp * sp * tp"
            dp = world // (pp * sp * tp)
        dims = MeshDims(pp, dp, sp, tp)
        assert dims.size() == world, f"mesh {dims} does not match the world size {world}"
        me = dist.get_rank() if dist.is_initialized() else 0
        out = cls(dims, me)
        for axis in ("pp", "dp", "sp", "tp"):
            for ranks in group_ranks(dims, axis):
                g = dist.new_group(ranks) if world > 1 else None       # every rank creates every group
                if me in ranks:
                    out.groups[axis], out.ranks[axis] = g, ranks
        return out

    def coord(self, axis: str) -> int:
        return coords(self.rank, self.dims)[axis]

    def sp_context(self):
        from .sp import SPContext
        if self.dims.sp == 1:
            return None
        return SPContext(self.groups["sp"], self.coord("sp"), self.dims.sp, self.ranks["sp"])

    def tp_context(self):
        from .tp import TPContext
        return TPContext(self.groups.get("tp"), self.coord("tp"), self.dims.tp)

    def ep_context(self):
        from .ep import EPContext
        return EPContext(self.groups.get("dp"), self.coord("dp"), self.dims.dp)
