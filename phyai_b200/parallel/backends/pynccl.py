"""``pynccl`` backend: NCCL collectives enqueued straight from ctypes, one communicator per mesh axis.

The unique id of an axis communicator travels over the axis' torch process group (any backend:
it is 128 bytes of host data). Every op runs on the current CUDA stream, so ``P.on_stream`` and
CUDA-graph capture work as with any kernel; a warm-up all-reduce on a side stream at construction
takes NCCL's lazy connection setup out of the first captured step.

Reference: phyai/src/phyai/parallel/backends/pynccl.py:46-426.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from ..backend import Call, Op
from .nccl_binding import DTYPES, NcclLibrary, ncclUniqueId


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0


class PyNcclCommunicator:
    def __init__(self, lib: NcclLibrary, world: int, rank: int, uid: ncclUniqueId) -> None:
        self.lib, self.world, self.rank = lib, world, rank
        self.comm = lib.comm_init_rank(world, uid, rank)

    def close(self) -> None:
        if self.comm is not None:
            self.lib.comm_destroy(self.comm)
            self.comm = None


class PyNcclBackend:
    name = "pynccl"

    def __init__(self, mesh, axes: list[str] | None = None, library_path: str | None = None, *, warmup: bool = True) -> None:
        self.mesh, self.lib = mesh, NcclLibrary(library_path)
        self.comms: dict[str, PyNcclCommunicator] = {}
        for axis in axes if axes is not None else list(mesh.names):
            n = mesh.axis_size(axis)
            if n <= 1:
                continue
            group, ranks, pos = mesh.axis_group(axis), mesh.axis_ranks(axis), mesh.axis_local_rank(axis)
            box = [bytes(self.lib.unique_id().internal) if pos == 0 else None]
            dist.broadcast_object_list(box, src=ranks[0], group=group)
            uid = ncclUniqueId()
            ctypes.memmove(ctypes.byref(uid), box[0], 128)
            self.comms[axis] = PyNcclCommunicator(self.lib, n, pos, uid)
        if warmup and self.comms and torch.cuda.is_available():
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for axis, c in self.comms.items():
                    t = torch.ones(8, device="cuda")
                    self.lib.all_reduce(t.data_ptr(), t.data_ptr(), 8, t.dtype, "sum", c.comm, side.cuda_stream)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()

    def can_handle(self, call: Call) -> bool:
        return call.device_type == "cuda" and call.axis in self.comms and call.mesh is self.mesh and call.dtype in DTYPES \
            and call.op is not Op.BARRIER and call.op is not Op.ALL_TO_ALL

    def supports_capture(self) -> bool:
        return True

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        c = self.comms[call.axis]
        n, op, s = c.world, call.op, _stream()
        if op is Op.ALL_REDUCE:
            x = tensors[0].contiguous()
            out = torch.empty_like(x)
            self.lib.all_reduce(x.data_ptr(), out.data_ptr(), x.numel(), x.dtype, kw.get("reduce", "sum"), c.comm, s)
            return out
        if op is Op.ALL_GATHER:
            x = tensors[0]
            dim = kw.get("dim", 0) % max(x.dim(), 1)
            xm = x.movedim(dim, 0).contiguous()
            out = torch.empty((n * xm.shape[0], *xm.shape[1:]), dtype=x.dtype, device=x.device)
            self.lib.all_gather(xm.data_ptr(), out.data_ptr(), xm.numel(), x.dtype, c.comm, s)
            return out.movedim(0, dim) if dim else out
        if op is Op.REDUCE_SCATTER:
            x = tensors[0]
            dim = kw.get("dim", 0) % max(x.dim(), 1)
            xm = x.movedim(dim, 0).contiguous()
            if xm.shape[0] % n:
                raise ValueError(f"reduce_scatter: dim {dim} of size {xm.shape[0]} is not divisible by {n}")
            out = torch.empty((xm.shape[0] // n, *xm.shape[1:]), dtype=x.dtype, device=x.device)
            self.lib.reduce_scatter(xm.data_ptr(), out.data_ptr(), out.numel(), x.dtype, kw.get("reduce", "sum"), c.comm, s)
            return out.movedim(0, dim) if dim else out
        if op is Op.BROADCAST:
            x = tensors[0].contiguous()
            out = torch.empty_like(x)
            self.lib.broadcast(x.data_ptr(), out.data_ptr(), x.numel(), x.dtype, kw.get("src", 0), c.comm, s)
            return out
        if op is Op.SEND:
            x = tensors[0].contiguous()
            self.lib.send(x.data_ptr(), x.numel(), x.dtype, kw["dst"], c.comm, s)
            return None
        if op is Op.RECV:
            x = tensors[0]
            self.lib.recv(x.data_ptr(), x.numel(), x.dtype, kw["src"], c.comm, s)
            return x
        raise NotImplementedError(op)

    def close(self) -> None:
        for c in self.comms.values():
            c.close()
        self.comms.clear()


__all__ = ["PyNcclBackend", "PyNcclCommunicator"]
