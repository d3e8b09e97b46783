"""Backend registry and selection policies.

Reference: phyai/src/phyai/parallel/registry.py:21-192.
"""

from __future__ import annotations

from typing import Iterable

from .backend import Backend, Call, Mode, Op
from .exceptions import CaptureUnsafeError, NoBackendError


class Registry:
    """Ordered list of backends with per-op preferences."""

    def __init__(self) -> None:
        self._backends: list[Backend] = []
        self._preferred: dict[Op, list[str]] = {}

    def register(self, backend: Backend, *, prefer_for: Iterable[Op] = ()) -> None:
        if any(b.name == backend.name for b in self._backends):
            raise ValueError(f"backend {backend.name!r} is already registered")
        self._backends.append(backend)
        for op in prefer_for:
            self._preferred.setdefault(op, []).append(backend.name)

    def names(self) -> list[str]:
        return [b.name for b in self._backends]

    def get(self, name: str) -> Backend:
        for b in self._backends:
            if b.name == name:
                return b
        raise KeyError(name)

    def candidates(self, call: Call) -> list[Backend]:
        """Backends able to run ``call``, preferred ones first; capture mode filters."""
        able = [b for b in self._backends if b.can_handle(call)]
        if call.mode is Mode.GRAPH_CAPTURING:
            safe = [b for b in able if b.supports_capture()]
            if able and not safe:
                raise CaptureUnsafeError(
                    f"{call.op.value} on axis {call.axis!r}: only capture-unsafe backends "
                    f"({[b.name for b in able]}) can run it")
            able = safe
        pref = self._preferred.get(call.op, [])
        able.sort(key=lambda b: pref.index(b.name) if b.name in pref else len(pref))
        return able

    def validate(self) -> None:
        if not self._backends:
            raise NoBackendError("no communication backend registered")


class DefaultPolicy:
    def choose(self, call: Call, candidates: list[Backend]) -> Backend:
        if not candidates:
            raise NoBackendError(f"no backend for {call.op.value} on axis {call.axis!r} "
                                 f"({call.dtype}, {call.nbytes} B, {call.mode.value})")
        return candidates[0]


class ForcedPolicy:
    """Always pick the named backend (``PHYAI_FORCE_BACKEND``)."""

    def __init__(self, name: str) -> None:
        self.name = name

    def choose(self, call: Call, candidates: list[Backend]) -> Backend:
        for b in candidates:
            if b.name == self.name:
                return b
        raise NoBackendError(f"forced backend {self.name!r} cannot run {call.op.value} on axis {call.axis!r}")


__all__ = ["Registry", "DefaultPolicy", "ForcedPolicy"]
