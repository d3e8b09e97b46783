"""Collective entry points: ``all_reduce``, ``all_gather``, ``reduce_scatter``,
``all_to_all``, ``broadcast``, ``send``, ``recv``, ``barrier``.

Each call names a mesh axis. A size-1 axis (or no mesh at all) makes the op the
identity (a clone, so callers may mutate the result). Otherwise a backend is
chosen per call by the dispatcher (reference: phyai/src/phyai/parallel/ops.py:66-479).
"""

from __future__ import annotations

from typing import Any

import torch

from . import state
from .backend import Call, Op

_DISPATCHER = None


def set_dispatcher(d) -> None:
    global _DISPATCHER
    _DISPATCHER = d


def get_dispatcher():
    return _DISPATCHER


def _mesh(mesh):
    return mesh if mesh is not None and not isinstance(mesh, str) else (
        state.resolve_mesh(mesh) if (mesh is not None or state.default_mesh() is not None) else None)


def _trivial(mesh, axis: str) -> bool:
    return mesh is None or mesh.axis_size(axis) <= 1


def _run(op: Op, axis: str, mesh, x: torch.Tensor | None, extra: tuple = (), **kw: Any):
    if _DISPATCHER is None:
        raise RuntimeError("phyai_b200.parallel.init has not been called")
    dev = x.device.type if x is not None else mesh.device_type
    call = Call(op=op, axis=axis, mesh=mesh, dtype=x.dtype if x is not None else torch.uint8,
                nbytes=x.numel() * x.element_size() if x is not None else 0,
                mode=state.current_mode(), device_type=dev, extra=extra)
    backend = _DISPATCHER.select(call)
    args = (x,) if x is not None else ()
    return backend.execute(call, *args, **kw)


def all_reduce(x: torch.Tensor, axis: str = "tp", *, reduce: str = "sum", mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    return _run(Op.ALL_REDUCE, axis, m, x, (reduce,), reduce=reduce)


def all_gather(x: torch.Tensor, axis: str = "tp", *, dim: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    return _run(Op.ALL_GATHER, axis, m, x, (dim,), dim=dim)


def reduce_scatter(x: torch.Tensor, axis: str = "tp", *, dim: int = 0, reduce: str = "sum", mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    return _run(Op.REDUCE_SCATTER, axis, m, x, (dim, reduce), dim=dim, reduce=reduce)


def all_to_all(x: torch.Tensor, axis: str = "sp", *, split_dim: int = 0, concat_dim: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    return _run(Op.ALL_TO_ALL, axis, m, x, (split_dim, concat_dim), split_dim=split_dim, concat_dim=concat_dim)


def broadcast(x: torch.Tensor, axis: str = "tp", *, src: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    return _run(Op.BROADCAST, axis, m, x, (src,), src=src)


def send(x: torch.Tensor, dst: int, axis: str = "dp", *, mesh=None) -> None:
    """Point-to-point send to local rank ``dst`` of ``axis`` (NCCL p2p on CUDA)."""
    m = _mesh(mesh)
    if _trivial(m, axis):
        raise ValueError(f"send on axis {axis!r} of size 1")
    _run(Op.SEND, axis, m, x, (), dst=dst)


def recv(x: torch.Tensor, src: int, axis: str = "dp", *, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        raise ValueError(f"recv on axis {axis!r} of size 1")
    return _run(Op.RECV, axis, m, x, (), src=src)


def barrier(axis: str = "tp", *, mesh=None) -> None:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return
    _run(Op.BARRIER, axis, m, None)


__all__ = ["all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "send", "recv",
           "barrier", "set_dispatcher", "get_dispatcher"]
