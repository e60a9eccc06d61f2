"""3-D process grid in the Megatron PTD-P order: ``rank = (dp * PP + pp) * TP + tp`` — tensor
parallel ranks are adjacent (same NVSwitch domain, the most communication), then pipeline, then
data parallel (reference: crates/model/src/grid.rs:32-80 ``Grid``, :91-136 ``LocalGroups``).
``ProcessGroups`` builds the matching ``torch.distributed`` groups (every rank creates every group,
as the API requires) and an optional expert-parallel axis laid over the data-parallel ranks."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple


@dataclass(frozen=True)
class Grid:
    tp: int = 1
    pp: int = 1
    dp: int = 1

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.dp

    def rank_of(self, tp: int, pp: int, dp: int) -> int:
        assert 0 <= tp < self.tp and 0 <= pp < self.pp and 0 <= dp < self.dp
        return (dp * self.pp + pp) * self.tp + tp

    def coord_of(self, rank: int) -> Tuple[int, int, int]:
        """(tp, pp, dp) of ``rank``."""
        assert 0 <= rank < self.world
        tp = rank % self.tp
        pp = (rank // self.tp) % self.pp
        dp = rank // (self.tp * self.pp)
        return tp, pp, dp

    def tp_group(self, rank: int) -> List[int]:
        _, pp, dp = self.coord_of(rank)
        return [self.rank_of(t, pp, dp) for t in range(self.tp)]

    def pp_group(self, rank: int) -> List[int]:
        tp, _, dp = self.coord_of(rank)
        return [self.rank_of(tp, p, dp) for p in range(self.pp)]

    def dp_group(self, rank: int) -> List[int]:
        tp, pp, _ = self.coord_of(rank)
        return [self.rank_of(tp, pp, d) for d in range(self.dp)]

    def all_groups(self, axis: str) -> List[List[int]]:
        fn = {"tp": self.tp_group, "pp": self.pp_group, "dp": self.dp_group}[axis]
        seen, out = set(), []
        for r in range(self.world):
            g = tuple(fn(r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out


class ProcessGroups:
    """``torch.distributed`` groups for one rank of a Grid."""

    def __init__(self, grid: Grid, rank: Optional[int] = None, backend: Optional[str] = None):
        import torch.distributed as dist
        self.grid = grid
        self.rank = dist.get_rank() if rank is None else rank
        assert dist.get_world_size() == grid.world, "world size does not match the grid"
        self.tp_coord, self.pp_coord, self.dp_coord = grid.coord_of(self.rank)
        self.groups = {}
        for axis in ("tp", "pp", "dp"):
            mine = None
            for ranks in grid.all_groups(axis):
                g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
                if self.rank in ranks:
                    mine = (g, ranks)
            self.groups[axis] = mine
        # pipeline p2p runs on two communicators of its own, one per direction: activations going
        # down and gradients coming up then never queue behind each other (or behind the
        # collectives of the default group) on one NCCL stream
        for name in ("pp_fwd", "pp_bwd"):
            mine = None
            for ranks in grid.all_groups("pp"):
                g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
                if self.rank in ranks:
                    mine = (g, ranks)
            self.groups[name] = mine

    def group(self, axis: str):
        return self.groups[axis][0]

    def ranks(self, axis: str) -> List[int]:
        return self.groups[axis][1]

    def prev_stage(self) -> Optional[int]:
        r = self.ranks("pp")
        return r[self.pp_coord - 1] if self.pp_coord > 0 else None

    def next_stage(self) -> Optional[int]:
        r = self.ranks("pp")
        return r[self.pp_coord + 1] if self.pp_coord + 1 < len(r) else None


class LocalGroups:
    """One ``HostCollective`` group per tensor / pipeline / data group of a Grid, for ranks that are
    threads of one process (reference: crates/model/src/grid.rs:91-136).  ``tp(r)`` / ``pp(r)`` /
    ``dp(r)`` return rank ``r``'s collective handle; its ``rank`` attribute is ``r``'s index inside
    that group."""

    def __init__(self, grid: Grid, timeout_s: float = 60.0):
        from .collective import HostCollective
        self.grid = grid
        self._by_axis = {}
        for axis in ("tp", "pp", "dp"):
            handles: List = [None] * grid.world
            for members in grid.all_groups(axis):
                group = HostCollective.group(len(members), timeout_s)
                for i, m in enumerate(members):
                    handles[m] = group[i]
            self._by_axis[axis] = handles

    def tp(self, rank: int):
        return self._by_axis["tp"][rank]

    def pp(self, rank: int):
        return self._by_axis["pp"][rank]

    def dp(self, rank: int):
        return self._by_axis["dp"][rank]
