"""ctypes binding of the NCCL C API (no torch in between).

``torch.distributed`` brings its own watchdog threads and Python dispatch; for collectives inside a
latency-critical or graph-captured step it is enough to enqueue ``ncclAllReduce`` on the current
stream. The library is ``libnccl.so.2`` next to torch's CUDA libraries unless ``PHYAI_NCCL_SO_PATH``
names another one.

Reference: phyai/src/phyai/parallel/backends/pynccl_wrapper.py:31-330.
"""

from __future__ import annotations

import ctypes
import glob
import os
from pathlib import Path

import torch

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p
cudaStream_t = ctypes.c_void_p
buffer_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


# ncclDataType_t / ncclRedOp_t values of NCCL 2.x
DTYPES = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
          torch.float64: 8, torch.bfloat16: 9}
REDOPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


class NcclError(RuntimeError):
    pass


def find_library() -> str:
    from ...env import envs

    override = envs.PHYAI_NCCL_SO_PATH.get()
    if override:
        return override
    here = Path(torch.__file__).resolve().parent
    for pat in (str(here / "lib" / "libnccl.so*"), str(here.parent / "nvidia" / "nccl" / "lib" / "libnccl.so*")):
        hits = sorted(glob.glob(pat))
        if hits:
            return hits[0]
    return "libnccl.so.2"


class NcclLibrary:
    _SIGS = {
        "ncclGetErrorString": (ctypes.c_char_p, [ncclResult_t]),
        "ncclGetVersion": (ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
        "ncclGetUniqueId": (ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
        "ncclCommInitRank": (ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int]),
        "ncclAllReduce": (ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclAllGather": (ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclReduceScatter": (ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclBroadcast": (ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclSend": (ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclRecv": (ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        "ncclGroupStart": (ncclResult_t, []),
        "ncclGroupEnd": (ncclResult_t, []),
        "ncclCommDestroy": (ncclResult_t, [ncclComm_t]),
    }

    def __init__(self, path: str | None = None) -> None:
        self.path = path or find_library()
        try:
            self.lib = ctypes.CDLL(self.path)
        except OSError as e:
            raise NcclError(f"cannot load NCCL from {self.path!r}: {e}") from e
        for name, (res, args) in self._SIGS.items():
            f = getattr(self.lib, name)
            f.restype, f.argtypes = res, args

    def check(self, code: int, what: str) -> None:
        if code != 0:
            msg = self.lib.ncclGetErrorString(code)
            raise NcclError(f"{what}: {msg.decode() if msg else code}")

    def version(self) -> tuple[int, int, int]:
        v = ctypes.c_int()
        self.check(self.lib.ncclGetVersion(ctypes.byref(v)), "ncclGetVersion")
        n = v.value
        return (n // 10000, (n // 100) % 100, n % 100) if n >= 10000 else (n // 1000, (n // 100) % 10, n % 100)

    def unique_id(self) -> ncclUniqueId:
        uid = ncclUniqueId()
        self.check(self.lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
        return uid

    def comm_init_rank(self, world: int, uid: ncclUniqueId, rank: int) -> ncclComm_t:
        comm = ncclComm_t()
        self.check(self.lib.ncclCommInitRank(ctypes.byref(comm), world, uid, rank), "ncclCommInitRank")
        return comm

    # every call below enqueues on `stream` (a raw cudaStream_t value) and returns at once
    def all_reduce(self, send: int, recv: int, count: int, dtype: torch.dtype, op: str, comm, stream: int) -> None:
        self.check(self.lib.ncclAllReduce(send, recv, count, DTYPES[dtype], REDOPS[op], comm, stream), "ncclAllReduce")

    def all_gather(self, send: int, recv: int, count: int, dtype: torch.dtype, comm, stream: int) -> None:
        self.check(self.lib.ncclAllGather(send, recv, count, DTYPES[dtype], comm, stream), "ncclAllGather")

    def reduce_scatter(self, send: int, recv: int, count: int, dtype: torch.dtype, op: str, comm, stream: int) -> None:
        self.check(self.lib.ncclReduceScatter(send, recv, count, DTYPES[dtype], REDOPS[op], comm, stream), "ncclReduceScatter")

    def broadcast(self, send: int, recv: int, count: int, dtype: torch.dtype, root: int, comm, stream: int) -> None:
        self.check(self.lib.ncclBroadcast(send, recv, count, DTYPES[dtype], root, comm, stream), "ncclBroadcast")

    def send(self, buf: int, count: int, dtype: torch.dtype, peer: int, comm, stream: int) -> None:
        self.check(self.lib.ncclSend(buf, count, DTYPES[dtype], peer, comm, stream), "ncclSend")

    def recv(self, buf: int, count: int, dtype: torch.dtype, peer: int, comm, stream: int) -> None:
        self.check(self.lib.ncclRecv(buf, count, DTYPES[dtype], peer, comm, stream), "ncclRecv")

    def group_start(self) -> None:
        self.check(self.lib.ncclGroupStart(), "ncclGroupStart")

    def group_end(self) -> None:
        self.check(self.lib.ncclGroupEnd(), "ncclGroupEnd")

    def comm_destroy(self, comm) -> None:
        self.check(self.lib.ncclCommDestroy(comm), "ncclCommDestroy")


__all__ = ["NcclLibrary", "NcclError", "ncclUniqueId", "DTYPES", "REDOPS", "find_library"]
