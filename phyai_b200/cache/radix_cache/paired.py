"""Full-attention + sliding-window pair with window-driven eviction. Reference: phyai/src/phyai/cache/radix_cache/paired.py:24-96."""

from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple

from .config import CacheConfig
from .native import MatchResult, PrefixCache, Tier


@dataclass(frozen=True)
class PairedCacheConfig:
    full: CacheConfig
    swa: CacheConfig
    window_size: int   # atoms


class PairedMatchResult(NamedTuple):
    full: MatchResult
    swa: MatchResult


class PairedCache:
    def __init__(self, cfg: PairedCacheConfig) -> None:
        self.cfg = cfg
        self.full: PrefixCache = cfg.full.build()
        self.swa: PrefixCache = cfg.swa.build()
        self.window_size = int(cfg.window_size)

    cur_step = property(lambda s: s.full.current_step)

    def allocate_pair(self, n: int):
        full_units = self.full.allocate(Tier.DEVICE, n)
        return full_units, self.swa.allocate(Tier.DEVICE, n)   # a failure here drops full_units back into its pool

    def insert_pair(self, atoms: bytes, full_units, swa_units):
        return self.full.insert(Tier.DEVICE, atoms, full_units), self.swa.insert(Tier.DEVICE, atoms, swa_units)

    def match(self, atoms: bytes) -> PairedMatchResult:
        return PairedMatchResult(self.full.match(atoms), self.swa.match(atoms))

    def lock_pair(self, full_node: int, swa_node: int):
        return self.full.lock(Tier.DEVICE, full_node), self.swa.lock(Tier.DEVICE, swa_node)

    def advance(self, n_new_atoms: int) -> int:
        """Move both clocks; drop window-cache nodes last touched at or before ``now - window``. Returns units freed."""
        self.full.advance_step(int(n_new_atoms))
        self.swa.advance_step(int(n_new_atoms))
        return self.swa.evict_by_named_predicate(Tier.DEVICE, "step_le", max(0, self.swa.current_step - self.window_size))

    def stats(self) -> dict[str, int]:
        return {"full_avail": self.full.available(Tier.DEVICE), "full_active": self.full.active(Tier.DEVICE),
                "swa_avail": self.swa.available(Tier.DEVICE), "swa_active": self.swa.active(Tier.DEVICE),
                "cur_step": int(self.cur_step), "window_size": self.window_size}
