"""Bump allocator over a contiguous slab of pool slots.

Reference: phyai/src/phyai/cache/static_cache.py:33-153.
"""

from __future__ import annotations

import torch

from .kv_cache_pool import KVCachePool


class StaticCacheError(RuntimeError):
    """The slab has fewer free slots than were asked for."""


class StaticCache:
    def __init__(self, pool: KVCachePool, *, base_offset: int, capacity: int) -> None:
        if base_offset < 0 or capacity <= 0 or base_offset + capacity > pool.num_slots:
            raise ValueError(f"slab [{base_offset}, {base_offset + capacity}) does not fit a pool of {pool.num_slots} slots")
        self.pool, self.base_offset, self.capacity = pool, base_offset, capacity
        self._used = 0

    @property
    def used(self) -> int:
        return self._used

    @property
    def free(self) -> int:
        return self.capacity - self._used

    def allocate(self, n: int) -> torch.Tensor:
        """The next ``n`` slots as an int64 tensor on the pool's device."""
        if n < 0:
            raise ValueError("allocate: n must be non-negative")
        if n > self.free:
            raise StaticCacheError(f"StaticCache out of slots: want {n}, free {self.free} of {self.capacity}")
        start = self.base_offset + self._used
        self._used += n
        return torch.arange(start, start + n, dtype=torch.int64, device=self.pool.device)

    def slot_range(self) -> tuple[int, int]:
        """``(first, one past last)`` slot of the slab in the pool."""
        return self.base_offset, self.base_offset + self.capacity

    def used_slot_range(self) -> tuple[int, int]:
        """The slots handed out so far."""
        return self.base_offset, self.base_offset + self._used

    def reset(self) -> None:
        self._used = 0


__all__ = ["StaticCache", "StaticCacheError"]
