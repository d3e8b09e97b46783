"""Named-axis process mesh.

Ranks are laid out row-major over the axis sizes with the last axis innermost, so
with axes ``(dp, cfg, ep, sp, cp, tp)`` a TP group is a block of consecutive ranks
and each CFG branch is a contiguous TP block (reference layout:
phyai/src/phyai/engine.py:252-278, phyai/src/phyai/parallel/mesh.py:20-79).

The mesh owns one ``torch.distributed`` group per axis the calling rank belongs
to. Building groups is collective: every rank must construct the same mesh.
"""

from __future__ import annotations

import math
from typing import Any, Sequence

from .backend import Topology


class Mesh:
    def __init__(self, sizes: Sequence[int], names: Sequence[str], *, rank: int = 0,
                 world_size: int | None = None, build_groups: bool = True, device_type: str = "cpu") -> None:
        if len(sizes) != len(names):
            raise ValueError("mesh: sizes and names differ in length")
        if len(set(names)) != len(names):
            raise ValueError(f"mesh: duplicate axis names in {tuple(names)}")
        self.sizes = tuple(int(s) for s in sizes)
        self.names = tuple(names)
        self.world_size = math.prod(self.sizes)
        if world_size is not None and world_size != self.world_size:
            raise ValueError(f"mesh {self.sizes} covers {self.world_size} ranks, world_size is {world_size}")
        if not 0 <= rank < self.world_size:
            raise ValueError(f"rank {rank} outside mesh of {self.world_size}")
        self.rank = rank
        self.device_type = device_type
        self._groups: dict[str, Any] = {}
        self._group_ranks: dict[str, tuple[int, ...]] = {n: self._ranks_along(n) for n in self.names}
        if build_groups and self.world_size > 1:
            self._build_groups()

    # ------------------------------------------------------------ coordinates
    def coords(self, rank: int | None = None) -> tuple[int, ...]:
        r = self.rank if rank is None else rank
        out = []
        for s in reversed(self.sizes):
            out.append(r % s)
            r //= s
        return tuple(reversed(out))

    def rank_of(self, coords: Sequence[int]) -> int:
        r = 0
        for c, s in zip(coords, self.sizes):
            r = r * s + c
        return r

    def _ranks_along(self, axis: str, rank: int | None = None) -> tuple[int, ...]:
        i = self.names.index(axis)
        c = list(self.coords(rank))
        out = []
        for k in range(self.sizes[i]):
            c[i] = k
            out.append(self.rank_of(c))
        return tuple(out)

    def _build_groups(self) -> None:
        import torch.distributed as dist

        for axis in self.names:
            i = self.names.index(axis)
            if self.sizes[i] == 1:
                continue
            seen: set[tuple[int, ...]] = set()
            for r in range(self.world_size):
                ranks = self._ranks_along(axis, r)
                if ranks in seen:
                    continue
                seen.add(ranks)
                g = dist.new_group(list(ranks))  # collective: every rank creates every group
                if self.rank in ranks:
                    self._groups[axis] = g

    # ----------------------------------------------------------------- queries
    def has_axis(self, axis: str) -> bool:
        return axis in self.names

    def axis_size(self, axis: str) -> int:
        return self.sizes[self.names.index(axis)] if axis in self.names else 1

    def axis_local_rank(self, axis: str) -> int:
        return self.coords()[self.names.index(axis)] if axis in self.names else 0

    def axis_ranks(self, axis: str) -> tuple[int, ...]:
        return self._group_ranks.get(axis, (self.rank,))

    def axis_group(self, axis: str) -> Any:
        """The process group of ``axis`` (``None`` for a size-1 axis)."""
        return self._groups.get(axis)

    def topology(self, axis: str) -> Topology:
        return Topology(world_size=self.world_size, axis_size=self.axis_size(axis))

    def __repr__(self) -> str:
        ax = ", ".join(f"{n}={s}" for n, s in zip(self.names, self.sizes))
        return f"Mesh({ax}; rank {self.rank}/{self.world_size})"


__all__ = ["Mesh"]
