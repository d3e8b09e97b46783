"""Recurrent-state + attention cache with per-layer routing. Reference: phyai/src/phyai/cache/radix_cache/hybrid.py:22-74."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

from .config import CacheConfig
from .native import HybridMatchResult, HybridPrefixCache, MambaSlot, PrefixCache


@dataclass(frozen=True)
class HybridCacheConfig:
    kv: CacheConfig
    num_mamba_slots: int
    layer_kinds: tuple[Literal["attn", "mamba"], ...]


class HybridCache:
    def __init__(self, cfg: HybridCacheConfig) -> None:
        self.hybrid = HybridPrefixCache(cfg.kv.build(), cfg.num_mamba_slots)
        self.layer_kinds = tuple(cfg.layer_kinds)

    kv = property(lambda s: s.hybrid.kv)
    num_layers = property(lambda s: len(s.layer_kinds))
    available_slots = property(lambda s: s.hybrid.available_slots)
    total_slots = property(lambda s: s.hybrid.total_slots)
    active_slots = property(lambda s: s.hybrid.active_slots)

    def is_mamba_layer(self, layer_id: int) -> bool:
        return self.layer_kinds[layer_id] == "mamba"

    def match(self, atoms: bytes) -> HybridMatchResult:
        return self.hybrid.match(atoms)

    def allocate_mamba_slot(self) -> Optional[MambaSlot]:
        return self.hybrid.allocate_mamba_slot()

    def attach_mamba(self, node_handle: int, slot: MambaSlot) -> None:
        self.hybrid.attach_mamba(node_handle, slot)

    def detach_mamba(self, node_handle: int) -> Optional[MambaSlot]:
        return self.hybrid.detach_mamba(node_handle)

    def ensure_mamba_capacity_by_evict(self, n: int) -> bool:
        return self.hybrid.ensure_mamba_capacity_by_evict(n)
