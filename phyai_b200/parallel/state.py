"""Process-wide state of the communication layer: capture mode and named meshes.

Reference: phyai/src/phyai/parallel/state.py:20-92.
"""

from __future__ import annotations

import contextlib
import contextvars
from typing import Any, Iterator

from .backend import Mode

_MODE: contextvars.ContextVar[Mode] = contextvars.ContextVar("phyai_b200_comm_mode", default=Mode.EAGER)
_MESHES: dict[str, Any] = {}
_DEFAULT_NAME = "model"
_ACTIVE: contextvars.ContextVar[str | None] = contextvars.ContextVar("phyai_b200_active_mesh", default=None)


def current_mode() -> Mode:
    return _MODE.get()


@contextlib.contextmanager
def graph_capture() -> Iterator[None]:
    """Inside this block collectives must be capturable; backends that are not are skipped."""
    tok = _MODE.set(Mode.GRAPH_CAPTURING)
    try:
        yield
    finally:
        _MODE.reset(tok)


def register_mesh(name: str, mesh: Any) -> None:
    _MESHES[name] = mesh


def unregister_mesh(name: str) -> None:
    _MESHES.pop(name, None)


def resolve_mesh(name: str | None = None) -> Any:
    key = name or _ACTIVE.get() or _DEFAULT_NAME
    if key not in _MESHES:
        raise KeyError(f"no mesh registered under {key!r}; call phyai_b200.parallel.init first")
    return _MESHES[key]


def mesh_name(mesh: Any) -> str | None:
    """The name a mesh object is registered under (None for an unregistered mesh)."""
    for k, v in _MESHES.items():
        if v is mesh:
            return k
    return None


def default_mesh() -> Any | None:
    return _MESHES.get(_ACTIVE.get() or _DEFAULT_NAME)


@contextlib.contextmanager
def use_mesh(name: str) -> Iterator[Any]:
    tok = _ACTIVE.set(name)
    try:
        yield resolve_mesh(name)
    finally:
        _ACTIVE.reset(tok)


def clear_meshes() -> None:
    _MESHES.clear()


__all__ = ["current_mode", "graph_capture", "register_mesh", "unregister_mesh", "resolve_mesh", "mesh_name",
           "default_mesh", "use_mesh", "clear_meshes"]
