"""Collective entry points: ``all_reduce``, ``all_gather``, ``reduce_scatter``,
``all_to_all``, ``broadcast``, ``send``, ``recv``, ``barrier``.

Each call names a mesh axis. A size-1 axis (or no mesh at all) makes the op the
identity (a clone, so callers may mutate the result). Otherwise a backend is
chosen per call by the dispatcher (reference: phyai/src/phyai/parallel/ops.py:66-479).

The tensor-valued collectives are also registered with ``torch.library`` as ``phyai_b200::all_reduce``
... ``phyai_b200::broadcast`` (mesh passed by its registered name) with shape-only fake implementations,
so code that calls them can be traced with fake tensors / exported (reference: ops.py:104-124). Calls on a
registered mesh go through those ops; a mesh object that was never registered is served directly.
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


# ---------------------------------------------------------------- registered ops (mesh by name)
def _axis_size(mesh_name: str, axis: str) -> int:
    return state.resolve_mesh(mesh_name).axis_size(axis)


@torch.library.custom_op("phyai_b200::all_reduce", mutates_args=())
def _all_reduce_op(x: torch.Tensor, mesh_name: str, axis: str, reduce: str) -> torch.Tensor:
    return _run(Op.ALL_REDUCE, axis, state.resolve_mesh(mesh_name), x, (reduce,), reduce=reduce)


@_all_reduce_op.register_fake
def _(x, mesh_name, axis, reduce):
    return torch.empty_like(x)


@torch.library.custom_op("phyai_b200::all_gather", mutates_args=())
def _all_gather_op(x: torch.Tensor, mesh_name: str, axis: str, dim: int) -> torch.Tensor:
    return _run(Op.ALL_GATHER, axis, state.resolve_mesh(mesh_name), x, (dim,), dim=dim)


@_all_gather_op.register_fake
def _(x, mesh_name, axis, dim):
    shape = list(x.shape)
    shape[dim] *= _axis_size(mesh_name, axis)
    return x.new_empty(shape)


@torch.library.custom_op("phyai_b200::reduce_scatter", mutates_args=())
def _reduce_scatter_op(x: torch.Tensor, mesh_name: str, axis: str, dim: int, reduce: str) -> torch.Tensor:
    return _run(Op.REDUCE_SCATTER, axis, state.resolve_mesh(mesh_name), x, (dim, reduce), dim=dim, reduce=reduce)


@_reduce_scatter_op.register_fake
def _(x, mesh_name, axis, dim, reduce):
    shape = list(x.shape)
    n = _axis_size(mesh_name, axis)
    if shape[dim] % n:
        raise ValueError(f"reduce_scatter: dim {dim} of size {shape[dim]} does not divide over {n} ranks")
    shape[dim] //= n
    return x.new_empty(shape)


@torch.library.custom_op("phyai_b200::all_to_all", mutates_args=())
def _all_to_all_op(x: torch.Tensor, mesh_name: str, axis: str, split_dim: int, concat_dim: int) -> torch.Tensor:
    return _run(Op.ALL_TO_ALL, axis, state.resolve_mesh(mesh_name), x, (split_dim, concat_dim), split_dim=split_dim,
                concat_dim=concat_dim)


@_all_to_all_op.register_fake
def _(x, mesh_name, axis, split_dim, concat_dim):
    shape = list(x.shape)
    n = _axis_size(mesh_name, axis)
    if shape[split_dim] % n:
        raise ValueError(f"all_to_all: dim {split_dim} of size {shape[split_dim]} does not divide over {n} ranks")
    shape[split_dim] //= n
    shape[concat_dim] *= n
    return x.new_empty(shape)


@torch.library.custom_op("phyai_b200::broadcast", mutates_args=())
def _broadcast_op(x: torch.Tensor, mesh_name: str, axis: str, src: int) -> torch.Tensor:
    return _run(Op.BROADCAST, axis, state.resolve_mesh(mesh_name), x, (src,), src=src)


@_broadcast_op.register_fake
def _(x, mesh_name, axis, src):
    return torch.empty_like(x)


def _named(m) -> str | None:
    return state.mesh_name(m)


def all_reduce(x: torch.Tensor, axis: str = "tp", *, reduce: str = "sum", mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    name = _named(m)
    if name is not None:
        return torch.ops.phyai_b200.all_reduce(x, name, axis, reduce)
    return _run(Op.ALL_REDUCE, axis, m, x, (reduce,), reduce=reduce)


def all_gather(x: torch.Tensor, axis: str = "tp", *, dim: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    name = _named(m)
    if name is not None:
        return torch.ops.phyai_b200.all_gather(x, name, axis, dim % x.dim())
    return _run(Op.ALL_GATHER, axis, m, x, (dim,), dim=dim)


def reduce_scatter(x: torch.Tensor, axis: str = "tp", *, dim: int = 0, reduce: str = "sum", mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    name = _named(m)
    if name is not None:
        return torch.ops.phyai_b200.reduce_scatter(x, name, axis, dim % x.dim(), reduce)
    return _run(Op.REDUCE_SCATTER, axis, m, x, (dim, reduce), dim=dim, reduce=reduce)


def all_to_all(x: torch.Tensor, axis: str = "sp", *, split_dim: int = 0, concat_dim: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    name = _named(m)
    if name is not None:
        return torch.ops.phyai_b200.all_to_all(x, name, axis, split_dim % x.dim(), concat_dim % x.dim())
    return _run(Op.ALL_TO_ALL, axis, m, x, (split_dim, concat_dim), split_dim=split_dim, concat_dim=concat_dim)


def broadcast(x: torch.Tensor, axis: str = "tp", *, src: int = 0, mesh=None) -> torch.Tensor:
    m = _mesh(mesh)
    if _trivial(m, axis):
        return x.clone()
    name = _named(m)
    if name is not None:
        return torch.ops.phyai_b200.broadcast(x, name, axis, src)
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
