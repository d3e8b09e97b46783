"""Declarative cache configuration. Reference: phyai/src/phyai/cache/radix_cache/config.py:11-56."""

from __future__ import annotations

import enum
from dataclasses import asdict, dataclass

from .native import PrefixCache


class Modality(str, enum.Enum):
    TEXT = "text"
    IMAGE = "image"
    VIDEO = "video"
    AUDIO = "audio"


@dataclass(frozen=True)
class CacheConfig:
    atom_bytes: int
    atoms_per_unit: int
    device_total_units: int
    host_total_units: int = 0
    disk_total_units: int = 0
    remote_total_units: int = 0
    eviction_policy: str = "lru"
    slru_threshold: int = 2
    max_events_buffered: int = 16384
    device_max_pending_units: int = 0
    host_max_pending_units: int = 0
    disk_max_pending_units: int = 0
    remote_max_pending_units: int = 0

    def build(self) -> PrefixCache:
        return PrefixCache(**asdict(self))
