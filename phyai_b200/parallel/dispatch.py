"""Per-call backend choice with a small cache.

The cache key is ``(op, axis, mesh id, dtype, size bucket, mode, device, extra)``
(reference: phyai/src/phyai/parallel/dispatch.py:22-118).
"""

from __future__ import annotations

from ..env import envs
from .backend import Backend, Call
from .registry import DefaultPolicy, ForcedPolicy, Registry


def size_bucket(nbytes: int) -> int:
    return max(int(nbytes), 1).bit_length()


class Dispatcher:
    def __init__(self, registry: Registry, policy=None) -> None:
        self.registry = registry
        forced = envs.PHYAI_FORCE_BACKEND.get()
        self.policy = policy if policy is not None else (ForcedPolicy(forced) if forced else DefaultPolicy())
        self._cache: dict[tuple, Backend] = {}
        self.hits = 0
        self.misses = 0

    def select(self, call: Call) -> Backend:
        key = (call.op, call.axis, id(call.mesh), call.dtype, size_bucket(call.nbytes), call.mode,
               call.device_type, call.extra)
        hit = self._cache.get(key)
        if hit is not None:
            self.hits += 1
            return hit
        self.misses += 1
        chosen = self.policy.choose(call, self.registry.candidates(call))
        self._cache[key] = chosen
        return chosen

    def clear(self) -> None:
        self._cache.clear()


__all__ = ["Dispatcher", "size_bucket"]
