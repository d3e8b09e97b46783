"""Routing facades: one cache per modality / attention pattern. Reference: phyai/src/phyai/cache/radix_cache/multimodal.py:13-99."""

from __future__ import annotations

from typing import Any, Mapping

from .config import CacheConfig, Modality
from .native import PrefixCache, Tier


class _Router:
    def __init__(self, children: Mapping[Any, Any]) -> None:
        self.children: dict[Any, Any] = dict(children)

    def __getitem__(self, key):
        return self.children[key]

    def __contains__(self, key) -> bool:
        return key in self.children

    def __iter__(self):
        return iter(self.children)

    def keys(self):
        return self.children.keys()

    def items(self):
        return self.children.items()

    def values(self):
        return self.children.values()


class MultimodalCache(_Router):
    def __init__(self, configs: Mapping[Modality, CacheConfig]) -> None:
        super().__init__({m: c.build() for m, c in configs.items()})
        self.configs = dict(configs)

    caches = property(lambda s: s.children)

    def stats(self) -> dict[Modality, dict[str, int]]:
        out = {}
        for m, c in self.children.items():
            row = {}
            for t in Tier:
                if c.tier_enabled(t):
                    row[f"{t.name.lower()}_avail"] = c.available(t)
                    row[f"{t.name.lower()}_active"] = c.active(t)
            out[m] = row
        return out


class MultiPatternCache(_Router):
    """Keyed by a free-form attention-pattern name such as "full" / "swa" / "sparse"."""

    def __init__(self, configs: Mapping[str, CacheConfig]) -> None:
        super().__init__({k: c.build() for k, c in configs.items()})

    caches = property(lambda s: s.children)

    def cache_of(self, pattern: str) -> PrefixCache:
        return self.children[pattern]


class NestedCache(_Router):
    """Router over arbitrary cache-like values, for layered compositions."""
