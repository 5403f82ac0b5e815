"""Process-group layout for dp x pp x tp on one or more nodes.

Rank order (fastest to slowest): tp, dp, pp -- tensor-parallel peers are adjacent ranks (same
NVSwitch domain), data-parallel replicas next, pipeline stages outermost.  This replaces
Megatron-core's ``parallel_state`` that the reference initialises with tp hard-wired to 1
(``benchmarks_paper/bench_multi_gpu.py:72-77,624``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist


@dataclass(frozen=True)
class ParallelLayout:
    world_size: int
    dp: int = 1
    pp: int = 1
    tp: int = 1

    def __post_init__(self):
        if self.dp * self.pp * self.tp != self.world_size:
            raise ValueError(f"dp*pp*tp = {self.dp * self.pp * self.tp} != world size {self.world_size}")

    def coords(self, rank: int) -> tuple:
        """``(pp_rank, dp_rank, tp_rank)`` of a global rank."""
        tp_rank = rank % self.tp
        dp_rank = (rank // self.tp) % self.dp
        pp_rank = rank // (self.tp * self.dp)
        return pp_rank, dp_rank, tp_rank

    def rank_of(self, pp_rank: int, dp_rank: int, tp_rank: int) -> int:
        return (pp_rank * self.dp + dp_rank) * self.tp + tp_rank

    def tp_group_ranks(self, rank: int) -> list:
        p, d, _ = self.coords(rank)
        return [self.rank_of(p, d, t) for t in range(self.tp)]

    def dp_group_ranks(self, rank: int) -> list:
        p, _, t = self.coords(rank)
        return [self.rank_of(p, d, t) for d in range(self.dp)]

    def pp_group_ranks(self, rank: int) -> list:
        _, d, t = self.coords(rank)
        return [self.rank_of(p, d, t) for p in range(self.pp)]

    def all_groups(self, kind: str) -> list:
        fn = {"tp": self.tp_group_ranks, "dp": self.dp_group_ranks, "pp": self.pp_group_ranks}[kind]
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(fn(r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    @classmethod
    def parse(cls, spec: str, world_size: int) -> "ParallelLayout":
        """``"dp8"``, ``"tp4pp2"``, ``"pp4dp2"`` ... missing factors default to 1 (dp absorbs
        the remainder when it is not given)."""
        import re

        vals = {k: int(v) for k, v in re.findall(r"(dp|pp|tp)(\d+)", spec.lower())}
        tp, pp = vals.get("tp", 1), vals.get("pp", 1)
        dp = vals.get("dp", world_size // (tp * pp))
        return cls(world_size, dp, pp, tp)


@dataclass
class ParallelState:
    """Live process groups of this rank."""

    layout: ParallelLayout
    rank: int
    pp_rank: int
    dp_rank: int
    tp_rank: int
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    pp_group: Optional[object] = None

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.layout.pp - 1

    @property
    def prev_rank(self) -> Optional[int]:
        return None if self.is_first_stage else self.layout.rank_of(self.pp_rank - 1, self.dp_rank, self.tp_rank)

    @property
    def next_rank(self) -> Optional[int]:
        return None if self.is_last_stage else self.layout.rank_of(self.pp_rank + 1, self.dp_rank, self.tp_rank)


def initialize_parallel_state(layout: ParallelLayout, rank: Optional[int] = None) -> ParallelState:
    """Create every tp / dp / pp group (all ranks must call this in the same order)."""
    rank = dist.get_rank() if rank is None else rank
    mine = {}
    for kind in ("tp", "dp", "pp"):
        for ranks in layout.all_groups(kind):
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if rank in ranks:
                mine[kind] = g
    p, d, t = layout.coords(rank)
    return ParallelState(layout, rank, p, d, t, mine.get("tp"), mine.get("dp"), mine.get("pp"))
