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

    def __init__(self, mesh) -> None:
        self.mesh = mesh
        self._groups: dict[str, Any] = {}
        self._streams: dict[tuple[str, int, int], Any] = {}

    @classmethod
    def create(cls, mesh) -> "PeerBackend | None":
        if mesh.device_type != "cuda" or not torch.cuda.is_available():
            return None
        from ... import ops

        if not ops.available():
            return None
        return cls(mesh)

    def can_handle(self, call: Call) -> bool:
        if call.op is not Op.ALL_REDUCE or call.device_type != "cuda" or call.dtype != torch.bfloat16:
            return False
        if call.extra and call.extra[0] != "sum":
            return False
        n = call.mesh.axis_size(call.axis)
        # decisions are cached per power-of-two size bucket, so the limit sits on a bucket edge
        return 1 < n <= 8 and call.nbytes < self.max_bytes and call.mesh is self.mesh

    def supports_capture(self) -> bool:
        return True

    def _stream(self, axis: str, rows: int, cols: int):
        key = (axis, rows, cols)
        st = self._streams.get(key)
        if st is None:
            from ..symm import PeerGroup

            pg = self._groups.get(axis)
            if pg is None:
                pg = PeerGroup.for_axis(self.mesh, axis, heap_bytes=256 << 20)
                self._groups[axis] = pg
            st = pg.stream(f"ar:{rows}x{cols}", rows, cols)
            self._streams[key] = st
        return st

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any):
        if kw.get("reduce", "sum") != "sum":
            raise NotImplementedError("peer backend reduces with sum only")
        x = tensors[0].contiguous()
        n = x.numel()
        if n % 8:  # the kernels move 16-byte vectors: pad the tail
            flat = x.new_zeros((n + 7) // 8, 8)
            flat.view(-1)[:n] = x.view(-1)
        else:
            cols = x.shape[-1] if x.dim() > 1 and x.shape[-1] % 8 == 0 else 8
            flat = x.view(-1, cols)
        out = self._stream(call.axis, flat.shape[0], flat.shape[1]).all_reduce(flat)
        return out.view(-1)[:n].view(x.shape)

    def close(self) -> None:
        for pg in self._groups.values():
            pg.close()
        self._groups.clear()
        self._streams.clear()


__all__ = ["PeerBackend"]
