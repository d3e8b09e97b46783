"""Distributed communication layer.

``init`` builds the named mesh, registers the backends that fit the device and
installs a dispatcher; the collective functions then work on any axis name. On a
single rank everything degenerates to identities, so model code is written once.

Backends: ``nccl`` / ``gloo`` (``torch.distributed``, plumbing and fallback) and,
on CUDA, ``peer`` — this repository's own kernels over IPC-mapped peer memory
(one-shot all-reduce, CFG exchange), preferred for small messages because they
avoid the NCCL launch path and are captured into CUDA graphs. The kernels that
fuse a GEMM with its collective are reached through ``phyai_b200.parallel.symm`` (``PeerStream.linear_reduce``,
``ops.gemm(wait=...)``).

Reference: phyai/src/phyai/parallel/__init__.py:78-249.
"""

from __future__ import annotations

import contextlib
from typing import Sequence

import torch

from . import state
from ..env import envs
from .backend import Backend, Call, Mode, Op, Topology
from .dispatch import Dispatcher
from .dist import destroy_dist, init_dist
from .exceptions import (CaptureUnsafeError, CommTimeoutError, NoBackendError, PeerLostError,
                         PhyaiDistError)
from .mesh import Mesh
from .ops import (all_gather, all_reduce, all_to_all, barrier, broadcast, get_dispatcher, recv,
                  reduce_scatter, send, set_dispatcher)
from .registry import DefaultPolicy, ForcedPolicy, Registry
from .backends.torch_dist import GlooBackend, NcclBackend
from .backends.torch_dist import _TorchDistBackend as TorchDistBackend
from .state import current_mode, default_mesh, graph_capture, register_mesh, resolve_mesh, use_mesh

AXES = ("dp", "cfg", "ep", "sp", "cp", "tp")
Policy = DefaultPolicy | ForcedPolicy       # anything with ``choose(call, candidates) -> Backend``


def __getattr__(name: str):
    # backends with heavier imports (ctypes binding of libnccl, the CUDA extension) load on first use
    if name in ("PyNcclBackend", "PyNCCLBackend"):
        from .backends.pynccl import PyNcclBackend

        return PyNcclBackend
    if name == "PeerBackend":
        from .backends.peer import PeerBackend

        return PeerBackend
    raise AttributeError(name)


def init(layout: Sequence[int] = (1,), mesh_dim_names: Sequence[str] = ("tp",), *, device: str = "cuda",
         backend: str | None = None, name: str = "model", enable_peer: bool = True, enable_pynccl: bool | None = None,
         pynccl_axes: Sequence[str] | None = None, pynccl_library_path: str | None = None) -> Mesh:
    """Create and register the mesh ``name`` and install the dispatcher.

    ``layout`` gives the size of every axis in ``mesh_dim_names`` (outermost first).
    With more than one rank a default process group must already exist
    (:func:`init_dist`).
    """
    import math

    import torch.distributed as dist

    ws = math.prod(layout)
    device_type = torch.device(device).type
    registry = Registry()
    if ws <= 1 or not (dist.is_available() and dist.is_initialized()):
        if ws > 1:
            raise RuntimeError(f"mesh of {ws} ranks needs an initialised process group")
        mesh = Mesh(layout, mesh_dim_names, rank=0, build_groups=False, device_type=device_type)
    else:
        if dist.get_world_size() != ws:
            raise ValueError(f"layout {tuple(layout)} covers {ws} ranks, the process group has {dist.get_world_size()}")
        mesh = Mesh(layout, mesh_dim_names, rank=dist.get_rank(), device_type=device_type)
        from .backends.torch_dist import GlooBackend, NcclBackend

        kind = backend or ("nccl" if device_type == "cuda" else "gloo")
        if kind == "nccl":
            if enable_peer:
                try:
                    from .backends.peer import PeerBackend

                    peer = PeerBackend.create(mesh)
                    if peer is not None:
                        registry.register(peer, prefer_for=(Op.ALL_REDUCE,))
                except Exception as e:  # peer memory is an optimisation; NCCL still serves every op
                    import logging

                    logging.getLogger(__name__).warning("peer-memory backend unavailable: %s", e)
            if enable_pynccl if enable_pynccl is not None else envs.PHYAI_USE_PYNCCL.get():
                # NCCL through ctypes: one communicator per axis, ops enqueue on the current stream
                try:
                    from .backends.pynccl import PyNcclBackend

                    registry.register(PyNcclBackend(mesh, list(pynccl_axes) if pynccl_axes is not None else None, pynccl_library_path))
                except Exception as e:
                    import logging

                    logging.getLogger(__name__).warning("pynccl backend unavailable: %s", e)
            registry.register(NcclBackend())
            registry.register(GlooBackend())
        elif kind == "gloo":
            registry.register(GlooBackend())
        else:
            raise ValueError(f"unknown communication backend {kind!r}")
        registry.validate()
    register_mesh(name, mesh)
    set_dispatcher(Dispatcher(registry))
    return mesh


def shutdown(name: str = "model") -> None:
    """Collective: closes the backends and the peer-memory groups of this process (their process groups belong to the
    mesh that goes away here: a group left open would be asked to agree on the step status by the next engine), then
    forgets the mesh."""
    from .symm import PeerGroup

    for g in PeerGroup.open_groups():
        try:
            g.close()
        except Exception:  # noqa: BLE001 - a rank that lost its peers still has to get through shutdown
            g._closed = True
    d = get_dispatcher()
    if d is not None:
        for n in d.registry.names():
            b = d.registry.get(n)
            if hasattr(b, "close"):
                b.close()
    state.unregister_mesh(name)
    set_dispatcher(None)


@contextlib.contextmanager
def on_stream(stream: "torch.cuda.Stream"):
    """Run the enclosed collectives on ``stream`` (they enqueue on the current stream)."""
    with torch.cuda.stream(stream):
        yield


def warmup(axes: Sequence[str] = AXES, *, mesh=None) -> None:
    """One tiny all-reduce per multi-rank axis so lazy communicator setup happens before capture."""
    m = mesh or default_mesh()
    if m is None:
        return
    for ax in axes:
        if m.has_axis(ax) and m.axis_size(ax) > 1:
            t = torch.ones(1, device="cuda" if m.device_type == "cuda" else "cpu")
            all_reduce(t, ax, mesh=m)
    if m.device_type == "cuda":
        torch.cuda.synchronize()


__all__ = ["GlooBackend", "NcclBackend", "TorchDistBackend", "PyNcclBackend", "PyNCCLBackend", "PeerBackend", "Policy",
           "get_dispatcher", "set_dispatcher", "AXES", "init", "shutdown", "on_stream", "warmup", "Mesh", "Op", "Mode", "Topology", "Call",
           "Backend", "Registry", "Dispatcher", "DefaultPolicy", "ForcedPolicy", "init_dist", "destroy_dist",
           "all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "send", "recv", "barrier",
           "graph_capture", "current_mode", "default_mesh", "resolve_mesh", "register_mesh", "use_mesh",
           "PhyaiDistError", "NoBackendError", "CommTimeoutError", "CaptureUnsafeError", "PeerLostError"]
