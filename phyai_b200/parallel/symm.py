"""Symmetric peer memory and the collectives built on it.

``PeerGroup`` gives the ranks of one mesh axis (all on one NVSwitch node) a slab of device
memory each, mapped into every peer through CUDA IPC, plus an array of per-channel signal
words at its start. A ``PeerStream`` is one ordered sequence of collective calls that all
ranks issue identically; it owns a channel and a double-buffered slot area sized for its
largest call. Because a stream's calls are ordered, its slots can serve every row-parallel
linear of a model in turn (call ``e + 2`` reuses the buffers of call ``e``, which every peer
has provably finished reading by then), so the memory cost is per model, not per layer.

Collectives (each is one or two launches of this repository's kernels, no NCCL):

* ``linear_reduce``   GEMM whose epilogue stores its tiles straight into the peers' slots,
  then a kernel that sums the partials, adds bias / gated residual and applies the norm.
  ``scatter=True`` is the two-step form for large token counts: tiles go only to the rank
  that owns those rows, the owner reduces + norms them and stores the result into every
  rank's gathered matrix; the next GEMM waits for the arrivals itself (``ops.gemm(wait=)``).
* ``all_reduce``      push + reduce without a GEMM in front.
* ``all_gather_rows`` push shards, wait, copy out.
* ``cfg_exchange``    classifier-free-guidance pair combine.

Every device-side wait gives up after about a second and records a status the host can read
(``ops.kernel_status()``); ranks are expected to be in step, and ``PeerGroup.sync()`` aligns
them on the host before first use. The reference has no counterpart: its collectives are
NCCL calls (phyai/src/phyai/layers/linear/layers.py:628-630).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import ops

_ALIGN = 256
_NORM_NONE = -1
_GUARD_BYTE = 0xA5


class PeerGuardError(RuntimeError):
    """A guard band of the symmetric heap was written: some kernel, on this rank or on a peer, stored outside its buffer."""


def _up(n: int, a: int = _ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass
class GatherTicket:
    """What the consumer of a gathered matrix needs: the matrix (a view of local symmetric memory)
    and the ``wait`` triple for ``ops.gemm``."""

    y: torch.Tensor
    wait: tuple[int, int, int]


class PeerGroup:
    _registry: dict[tuple[int, str], "PeerGroup"] = {}

    def __init__(self, ranks: tuple[int, ...], pos: int, group, *, heap_bytes: int = 1 << 30, n_channels: int = 256,
                 device: torch.device | None = None) -> None:
        self.ext = ops.ext()
        self.ranks, self.pos, self.world, self.group = tuple(ranks), int(pos), len(ranks), group
        if self.world > 8:
            raise ValueError("a peer group spans at most 8 ranks (one NVSwitch node)")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.n_channels = n_channels
        self.sig_bytes = _up(n_channels * self.ext.CHANNEL_SIG_BYTES)
        self.heap_bytes = _up(self.sig_bytes + heap_bytes)
        self.slab, handle, self.local_ptr = self.ext.ipc_alloc(self.heap_bytes)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, (self.pos, handle), group=group)
        self.ptrs: list[int] = [0] * self.world
        for p, h in handles:
            self.ptrs[p] = self.local_ptr if p == self.pos else self.ext.ipc_open(h)
        self._top = self.sig_bytes
        self._next_channel = 0
        self._streams: dict[str, PeerStream] = {}
        self._closed = False
        # PHYAI_PEER_GUARD=1: every allocation of the heap sits between two bands of a known byte, which
        # check_guards() reads back. Peers store into this rank's buffers, so the bands of a rank catch the
        # overruns of every rank. All ranks must agree on the setting (the offsets are part of the protocol).
        from ..env import envs

        self.guard_bytes = _ALIGN if envs.PHYAI_PEER_GUARD.get() else 0
        self._guards: list[tuple[int, int]] = []
        self.sync()

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def for_axis(cls, mesh, axis: str, **kw) -> "PeerGroup":
        key = (id(mesh), axis)
        g = cls._registry.get(key)
        if g is None or g._closed:
            if mesh.axis_size(axis) < 2:
                raise ValueError(f"axis {axis!r} has a single rank: nothing to share")
            g = cls(mesh.axis_ranks(axis), mesh.axis_local_rank(axis), mesh.axis_group(axis), **kw)
            cls._registry[key] = g
        return g

    def sync(self) -> None:
        """Host-side alignment of the ranks (drains this rank's stream first)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    @classmethod
    def open_groups(cls) -> list["PeerGroup"]:
        """Every peer group of this process that has not been closed."""
        return [g for g in cls._registry.values() if not g._closed]

    def reset_channels(self) -> None:
        """Collective: bring every channel back to its initial state after a device wait gave up.

        A consumer that timed out has already closed its call (counter cleared, epoch bumped), so an
        arrival that lands afterwards would be counted for a later call. All ranks drain their streams,
        meet on the host, clear their signal words, and meet again before anyone launches."""
        self.sync()
        self.slab[: self.sig_bytes].zero_()
        self.sync()

    def close(self) -> None:
        if self._closed:
            return
        self.sync()
        for p, ptr in enumerate(self.ptrs):
            if p != self.pos:
                self.ext.ipc_close(ptr)
        self.sync()
        self.ext.ipc_free(self.local_ptr)
        self._closed = True

    # ------------------------------------------------------------------ allocation (identical on every rank)
    def alloc(self, nbytes: int) -> int:
        g = self.guard_bytes
        if g and not self._guards:
            self._band(self._top)          # in front of the first allocation
            self._top += g
        off = self._top
        end = _up(off + nbytes)
        if end + g > self.heap_bytes:
            raise MemoryError(f"symmetric heap exhausted: {end + g} > {self.heap_bytes} bytes")
        if g:
            self._band(off + nbytes, end + g)   # from the last byte asked for: behind this allocation, in front of the next
        self._top = end + g
        return off

    def _band(self, lo: int, hi: int | None = None) -> None:
        hi = lo + self.guard_bytes if hi is None else hi
        if hi > self.heap_bytes:
            raise MemoryError("symmetric heap exhausted by a guard band")
        self.slab[lo:hi].fill_(_GUARD_BYTE)
        self._guards.append((lo, hi))

    def check_guards(self) -> None:
        """Raise :class:`PeerGuardError` if a guard band of this rank's heap no longer holds its fill byte
        (no-op without ``PHYAI_PEER_GUARD=1``). Call it between steps, after ``sync()``."""
        bad = []
        for lo, hi in self._guards:
            wrong = (self.slab[lo:hi] != _GUARD_BYTE).nonzero()
            if wrong.numel():
                bad.append((lo + int(wrong[0]), int(wrong.numel())))
        if bad:
            raise PeerGuardError("symmetric heap guard bands overwritten on rank position %d: %s"
                                 % (self.pos, ", ".join(f"{n} byte(s) from offset {o}" for o, n in bad)))

    def new_channel(self) -> int:
        c = self._next_channel
        if c >= self.n_channels:
            raise RuntimeError("out of signal channels")
        self._next_channel += 1
        return c

    def view(self, byte_off: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        return self.slab[byte_off:byte_off + n].view(dtype).view(*shape)

    def stream(self, name: str, max_rows: int, max_cols: int, *, gather_rows: int = 0, gather_cols: int = 0) -> "PeerStream":
        s = self._streams.get(name)
        if s is None:
            s = PeerStream(self, max_rows, max_cols, gather_rows, gather_cols)
            self._streams[name] = s
        elif s.max_rows < max_rows or s.max_cols < max_cols or s.gather_rows < gather_rows or s.gather_cols < gather_cols:
            raise ValueError(f"stream {name!r} exists with a smaller geometry")
        return s

    # ------------------------------------------------------------------ CFG pair
    def cfg_exchange(self, v: torch.Tensor, *, is_cond: bool, g: float, out: torch.Tensor | None = None,
                     x_fp32: torch.Tensor | None = None, dt: float = 0.0) -> torch.Tensor:
        """Both ranks of a guidance pair end with ``uncond + g (cond - uncond)``; with ``x_fp32`` the
        Euler update ``x += dt * v`` happens in the same kernel."""
        if self.world != 2:
            raise ValueError("cfg_exchange pairs exactly two ranks")
        n = v.numel()
        key = f"cfg:{n}"
        st = self._streams.get(key)
        if st is None:
            st = _CfgInbox(self, n)
            self._streams[key] = st  # type: ignore[assignment]
        if out is None:
            out = torch.empty_like(v)
        self.ext.cfg_exchange(v, self.ptrs, self.pos, 1 - self.pos, st.off // 2, bool(is_cond), float(g), out, x_fp32,
                              float(dt), 0, st.channel)
        return out


class _CfgInbox:
    def __init__(self, pg: PeerGroup, n: int) -> None:
        self.off = pg.alloc(2 * n * 2)  # two parities of n bf16
        self.channel = pg.new_channel()


class PeerStream:
    def __init__(self, pg: PeerGroup, max_rows: int, max_cols: int, gather_rows: int, gather_cols: int) -> None:
        self.pg, self.max_rows, self.max_cols = pg, int(max_rows), _up(int(max_cols), 8)
        self.gather_rows, self.gather_cols = int(gather_rows), _up(int(gather_cols), 8) if gather_cols else 0
        self.slot_stride = self.max_rows * self.max_cols                    # elements per source rank
        self.slots_off = pg.alloc(2 * pg.world * self.slot_stride * 2)      # bytes: [parity][src][rows][cols] bf16
        self.channel = pg.new_channel()
        self.y_off = pg.alloc(self.gather_rows * self.gather_cols * 2) if gather_rows else -1
        self.y_channel = pg.new_channel() if gather_rows else -1
        self.single_launches = 0          # linear_reduce calls served by one launch (GEMM with the reduce tail)

    # ---- producers
    def _check(self, rows: int, cols: int, scatter: bool) -> int:
        per = -(-rows // self.pg.world) if scatter else 0
        if cols > self.max_cols or (per if scatter else rows) > self.max_rows:
            raise ValueError(f"call of {rows}x{cols} exceeds the stream's slots ({self.max_rows}x{self.max_cols})")
        return per

    def push(self, x: torch.Tensor) -> int:
        self._check(x.shape[0], x.shape[1], False)
        pg = self.pg
        return pg.ext.push_partial(x, pg.ptrs, pg.pos, self.slots_off // 2, self.slot_stride, self.max_cols, 0, self.channel)

    def gemm_push(self, x: torch.Tensor, w: torch.Tensor, *, scatter: bool = False, force_bn: int = 0,
                  force_swap: int = -1, force_splits: int = 0) -> tuple[int, int]:
        per = self._check(x.shape[0], w.shape[0], scatter)
        pg = self.pg
        expect = pg.ext.gemm_push(x, w, pg.ptrs, pg.pos, self.slots_off // 2, self.slot_stride, self.max_cols, 0,
                                  self.channel, per, force_bn, force_swap, force_splits)
        return expect, per

    # ---- consumer
    def reduce(self, expect: int, rows: int, cols: int, *, rows_per_rank: int = 0, residual: torch.Tensor | None = None,
               col_gate: torch.Tensor | None = None, bias: torch.Tensor | None = None, h_out: torch.Tensor | None = None,
               y: torch.Tensor | None = None, norm: str | None = None, weight: torch.Tensor | None = None,
               mod: torch.Tensor | None = None, eps: float = 1e-6, gather: bool = False, max_ctas: int = 592):
        """Sum the partials of the pending call; ``h = residual + (sum + bias) * gate`` goes to ``residual``
        (in place) or ``h_out``; ``y = norm(h)`` goes to ``y`` or, with ``gather``, to every rank's
        gathered matrix (returns a :class:`GatherTicket`)."""
        pg = self.pg
        mode = _NORM_NONE if norm is None else ops.NORM[norm]
        y_off, y_ld = -1, 0
        if gather:
            if self.y_off < 0 or rows > self.gather_rows or cols > self.gather_cols:
                raise ValueError("stream was created without (enough) gather space")
            y_off, y_ld = self.y_off // 2, self.gather_cols
        pg.ext.reduce_norm(pg.ptrs, pg.pos, self.slots_off // 2, self.slot_stride, rows, cols, self.max_cols, 0,
                                      self.channel, expect, residual, col_gate, bias, h_out, y, mode, weight, mod, eps,
                                      max_ctas, rows_per_rank, y_off, y_ld, max(self.y_channel, 0))
        if not gather:
            return None
        # one arrival per CTA of every rank's reduce kernel; ranks own different numbers of rows
        arrivals = 0
        for r in range(pg.world):
            n_r = max(0, min(rows_per_rank, rows - r * rows_per_rank)) if rows_per_rank > 0 else rows
            arrivals += max(1, min(n_r, max_ctas))
        full = pg.view(self.y_off, (self.gather_rows, self.gather_cols))[:rows, :cols]
        return GatherTicket(full, (pg.local_ptr, self.y_channel, arrivals))

    def wait_gather(self, ticket: GatherTicket) -> torch.Tensor:
        """For a consumer that is not ``ops.gemm(wait=...)``: block the stream until the rows arrived."""
        pg = self.pg
        rows, cols = ticket.y.shape
        pg.ext.gather_consume(pg.ptrs, pg.pos, 0, 0, rows, _up(cols, 8), self.gather_cols, None, 0, self.y_channel,
                              ticket.wait[2])
        return ticket.y

    # ---- composed collectives
    def linear_reduce(self, x: torch.Tensor, w: torch.Tensor, *, scatter: bool = False, **kw):
        """Row-parallel ``x @ w.T`` summed over the ranks, with the residual / gate / norm of :meth:`reduce`.
        Whole-partial calls that gather nothing go through one native entry, which on few rows runs the
        consumer half in the GEMM's own CTAs (one launch, one peer round trip)."""
        if not scatter and not kw.get("gather", False):
            return self._linear_reduce_local(x, w, **kw)
        expect, per = self.gemm_push(x, w, scatter=scatter)
        return self.reduce(expect, x.shape[0], w.shape[0], rows_per_rank=per, **kw)

    def _linear_reduce_local(self, x: torch.Tensor, w: torch.Tensor, *, residual=None, col_gate=None, bias=None, h_out=None,
                             y=None, norm: str | None = None, weight=None, mod=None, eps: float = 1e-6, gather: bool = False,
                             max_ctas: int = 592, allow_tail: bool = True) -> None:
        self._check(x.shape[0], w.shape[0], False)
        pg = self.pg
        mode = _NORM_NONE if norm is None else ops.NORM[norm]
        self.single_launches += int(pg.ext.linear_reduce(x, w, pg.ptrs, pg.pos, self.slots_off // 2, self.slot_stride, self.max_cols, 0,
                                                         self.channel, residual, col_gate, bias, h_out, y, mode, weight, mod, eps,
                                                         max_ctas, allow_tail))

    def all_reduce(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of a (rows, cols) bf16 matrix over the ranks."""
        if out is None:
            out = torch.empty_like(x)
        self.reduce(self.push(x), x.shape[0], x.shape[1], h_out=out)
        return out

    def all_gather_rows(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        pg = self.pg
        rows, cols = x.shape
        if out is None:
            out = torch.empty(pg.world * rows, cols, dtype=x.dtype, device=x.device)
        expect = self.push(x)
        pg.ext.gather_consume(pg.ptrs, pg.pos, self.slots_off // 2, self.slot_stride, rows, cols, self.max_cols, out, 0,
                              self.channel, expect)
        return out


__all__ = ["PeerGroup", "PeerStream", "GatherTicket"]
