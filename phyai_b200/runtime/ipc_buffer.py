"""Buffers shared between processes: device memory through CUDA IPC, host memory through POSIX shm.

``CudaIpcBuffer.create`` allocates a slab and exports a 64-byte handle; another process ``attach``es
it and both see the same bytes (this is also what the peer-memory collectives are built on, see
``phyai_b200.parallel.symm``). ``HostShmBuffer`` is the host-side twin for staging inputs between a
front-end process and the engine; with ``pin=True`` the mapping is registered with CUDA so copies
from it are asynchronous.

Reference: phyai/src/phyai/runtime/ipc_buffer.py:252-830 (there built on cuda-python; here on the
allocation calls of this repository's extension, which the GPU box always has).
"""

from __future__ import annotations

import base64
import json
import math
import secrets
from dataclasses import asdict, dataclass
from multiprocessing import shared_memory
from typing import Any, Sequence

import numpy as np
import torch


def _nbytes(shape: Sequence[int], dtype: torch.dtype) -> int:
    return math.prod(shape) * torch.empty((), dtype=dtype).element_size()


@dataclass(frozen=True)
class CudaIpcHandle:
    handle_b64: str
    nbytes: int
    device_index: int

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, s: str) -> "CudaIpcHandle":
        return cls(**json.loads(s))


@dataclass(frozen=True)
class HostShmHandle:
    name: str
    nbytes: int

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, s: str) -> "HostShmHandle":
        return cls(**json.loads(s))


class CudaIpcBuffer:
    def __init__(self, slab: torch.Tensor | None, ptr: int, nbytes: int, device: torch.device, handle: CudaIpcHandle, creator: bool) -> None:
        self._slab, self._ptr, self._nbytes, self._device, self._handle, self._creator = slab, ptr, nbytes, device, handle, creator
        self._closed = False

    @classmethod
    def create(cls, nbytes: int, device: int | torch.device | None = None) -> "CudaIpcBuffer":
        from .. import ops

        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device if not isinstance(device, int) else f"cuda:{device}")
        with torch.cuda.device(dev):
            slab, raw, ptr = ops.ext().ipc_alloc(int(nbytes))
        h = CudaIpcHandle(base64.b64encode(raw).decode(), int(nbytes), dev.index or 0)
        return cls(slab, ptr, int(nbytes), dev, h, True)

    @classmethod
    def attach(cls, handle: CudaIpcHandle, device: int | torch.device | None = None) -> "CudaIpcBuffer":
        """Map a buffer created by ANOTHER process (CUDA refuses to open a handle in the process that made it)."""
        from .. import ops

        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device if not isinstance(device, int) else f"cuda:{device}")
        with torch.cuda.device(dev):
            ptr = ops.ext().ipc_open(base64.b64decode(handle.handle_b64))
        return cls(None, ptr, handle.nbytes, dev, handle, False)

    handle = property(lambda s: s._handle)
    is_creator = property(lambda s: s._creator)
    local_ptr = property(lambda s: s._ptr)
    device = property(lambda s: s._device)
    nbytes = property(lambda s: s._nbytes)

    def tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.uint8, offset: int = 0) -> torch.Tensor:
        """A view of the buffer (no copy). Valid until ``close``."""
        need = _nbytes(shape, dtype)
        if offset < 0 or offset + need > self._nbytes:
            raise ValueError(f"view of {need} bytes at {offset} does not fit a buffer of {self._nbytes}")
        if self._slab is None:
            # attached side: wrap the mapped pointer
            class _Wrap:
                pass
            w = _Wrap()
            w.__cuda_array_interface__ = {"shape": (self._nbytes,), "typestr": "|u1", "data": (self._ptr, False), "version": 2}
            self._slab = torch.as_tensor(w, device=self._device)
        return self._slab[offset:offset + need].view(dtype).view(*shape)

    def close(self) -> None:
        if self._closed:
            return
        from .. import ops

        self._slab = None
        with torch.cuda.device(self._device):
            (ops.ext().ipc_free if self._creator else ops.ext().ipc_close)(self._ptr)
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()


class HostShmBuffer:
    def __init__(self, shm: shared_memory.SharedMemory, nbytes: int, creator: bool, pinned: bool) -> None:
        self._shm, self._nbytes, self._creator, self._pinned, self._closed = shm, nbytes, creator, pinned, False

    @classmethod
    def create(cls, nbytes: int, *, name: str | None = None, pin: bool = False) -> "HostShmBuffer":
        shm = shared_memory.SharedMemory(name=name or f"phyai_b200_{secrets.token_hex(6)}", create=True, size=int(nbytes))
        return cls(shm, int(nbytes), True, _register(shm, int(nbytes)) if pin else False)

    @classmethod
    def attach(cls, handle: HostShmHandle, *, pin: bool = False) -> "HostShmBuffer":
        shm = shared_memory.SharedMemory(name=handle.name, create=False)
        if shm.size < handle.nbytes:
            shm.close()
            raise ValueError(f"segment {handle.name!r} holds {shm.size} bytes, the handle says {handle.nbytes}")
        return cls(shm, handle.nbytes, False, _register(shm, handle.nbytes) if pin else False)

    handle = property(lambda s: HostShmHandle(s._shm.name, s._nbytes))
    is_creator = property(lambda s: s._creator)
    name = property(lambda s: s._shm.name)
    nbytes = property(lambda s: s._nbytes)
    pinned = property(lambda s: s._pinned)

    def as_numpy(self, shape: Sequence[int], dtype=np.uint8, offset: int = 0) -> np.ndarray:
        need = int(np.prod(shape)) * np.dtype(dtype).itemsize
        if offset < 0 or offset + need > self._nbytes:
            raise ValueError(f"view of {need} bytes at {offset} does not fit a buffer of {self._nbytes}")
        return np.ndarray(tuple(shape), dtype=dtype, buffer=self._shm.buf, offset=offset)

    def as_tensor(self, shape: Sequence[int], dtype: torch.dtype = torch.uint8, offset: int = 0) -> torch.Tensor:
        need = _nbytes(shape, dtype)
        if offset < 0 or offset + need > self._nbytes:
            raise ValueError(f"view of {need} bytes at {offset} does not fit a buffer of {self._nbytes}")
        flat = torch.frombuffer(self._shm.buf, dtype=torch.uint8, count=need, offset=offset)
        return flat.view(dtype).view(*shape)

    def close(self) -> None:
        if self._closed:
            return
        if self._pinned and torch.cuda.is_available():
            try:
                torch.cuda.cudart().cudaHostUnregister(_addr(self._shm))
            except Exception:
                pass
        try:
            self._shm.close()
        except BufferError:
            pass            # views are still alive: the mapping goes with the last of them
        if self._creator:
            try:
                self._shm.unlink()
            except FileNotFoundError:
                pass
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()


def _addr(shm: shared_memory.SharedMemory) -> int:
    return np.frombuffer(shm.buf, dtype=np.uint8, count=1).__array_interface__["data"][0]


def _register(shm: shared_memory.SharedMemory, nbytes: int) -> bool:
    if not torch.cuda.is_available():
        return False
    try:
        return int(torch.cuda.cudart().cudaHostRegister(_addr(shm), nbytes, 0)) == 0
    except Exception:
        return False


__all__ = ["CudaIpcBuffer", "CudaIpcHandle", "HostShmBuffer", "HostShmHandle"]
