"""``peer`` backend: small-message all-reduce over IPC-mapped peer memory.

One launch pushes this rank's tensor into every peer's slots, a second sums the arrivals; both
are ordinary kernels on the current stream, so the pair is captured into CUDA graphs and costs
no NCCL launch path. Large tensors stay on NCCL, whose ring / in-switch reductions move fewer
bytes per rank. The reference's small-message fast path is a ctypes NCCL binding
(phyai/src/phyai/parallel/backends/pynccl.py:196-426); this is the peer-memory equivalent.
"""

from __future__ import annotations

from typing import Any

import torch

from ..backend import Call, Op


class PeerBackend:
    name = "peer"
    max_bytes = 4 << 20
    #: every call is laid out as rows of this many bf16 values, so one slot geometry serves all shapes
    COLS = 1024

    def __init__(self, mesh) -> None:
        self.mesh = mesh
        self._groups: dict[str, Any] = {}
        self._streams: dict[str, Any] = {}
        self._failed: set[str] = set()

    @classmethod
    def create(cls, mesh) -> "PeerBackend | None":
        if mesh.device_type != "cuda" or not torch.cuda.is_available():
            return None
        from ... import ops

        if not ops.available():
            return None
        return cls(mesh)

    @property
    def max_rows(self) -> int:
        return -(-(self.max_bytes // 2) // self.COLS)

    def can_handle(self, call: Call) -> bool:
        if call.op is not Op.ALL_REDUCE or call.device_type != "cuda" or call.dtype != torch.bfloat16:
            return False
        if call.extra and call.extra[0] != "sum":
            return False
        n = call.mesh.axis_size(call.axis)
        # decisions are cached per power-of-two size bucket, so the limit sits on a bucket edge
        if not (1 < n <= 8 and call.nbytes < self.max_bytes and call.mesh is self.mesh):
            return False
        # the stream is created here (every rank asks in the same order), so that a heap or channel
        # shortage sends the call to the next backend instead of failing in the middle of a forward
        return self._stream(call.axis) is not None

    def supports_capture(self) -> bool:
        return True

    def _open_group(self, axis: str):
        from ..symm import PeerGroup

        return PeerGroup.for_axis(self.mesh, axis, heap_bytes=256 << 20)

    def _stream(self, axis: str):
        """The one stream of an axis: ``max_rows x COLS`` slots, which every call up to ``max_bytes`` fits."""
        st = self._streams.get(axis)
        if st is not None or axis in self._failed:
            return st
        try:
            pg = self._groups.get(axis)
            if pg is None:
                pg = self._open_group(axis)
                self._groups[axis] = pg
            st = pg.stream(f"ar:{axis}", self.max_rows, self.COLS)
        except (MemoryError, RuntimeError) as e:
            import logging

            logging.getLogger(__name__).warning("peer backend unavailable on axis %r (%s): calls go to the next backend", axis, e)
            self._failed.add(axis)
            return None
        self._streams[axis] = st
        return st

    @classmethod
    def flatten(cls, x: torch.Tensor) -> torch.Tensor:
        """``x`` as rows of ``COLS`` values (a view when the size divides, else a zero-padded copy)."""
        n = x.numel()
        x = x.contiguous()
        if n % cls.COLS == 0:
            return x.view(-1, cls.COLS)
        flat = x.new_zeros(-(-n // cls.COLS), cls.COLS)
        flat.view(-1)[:n] = x.view(-1)
        return flat

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        if kw.get("reduce", "sum") != "sum":
            raise NotImplementedError("peer backend reduces with sum only")
        x = tensors[0]
        st = self._stream(call.axis)
        if st is None:
            raise RuntimeError(f"peer backend has no stream on axis {call.axis!r}")
        flat = self.flatten(x)
        out = st.all_reduce(flat)
        return out.view(-1)[: x.numel()].view(x.shape)

    def close(self) -> None:
        for pg in self._groups.values():
            pg.close()
        self._groups.clear()
        self._streams.clear()
        self._failed.clear()


__all__ = ["PeerBackend"]
