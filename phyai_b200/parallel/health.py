"""Failure detection on the host: rank heartbeats over a key-value store and device-wait time-outs.

The fused communication kernels never hang: a wait that runs out records a status word
(``ops.kernel_status()``) and the kernel returns. ``raise_for_kernel_status`` turns that word into
:class:`CommTimeoutError` so a scheduler can tear the communicator down. Between steps a
:class:`Heartbeat` publishes ``(counter, wall time)`` under ``hb/<rank>`` in a store shared by the
job (``torch.distributed.TCPStore`` or anything with ``set``/``get``); ``check_peers`` reports ranks
whose beat is older than the deadline *before* the next launch, which is where a lost rank must be
noticed: a kernel already waiting on it would only time out.

The reference defines ``CommTimeoutError`` and never raises it (phyai/src/phyai/parallel/exceptions.py:18-19)
and documents a hang where peers block in ``recv`` (phyai/src/phyai/models/pi05/scheduler_wn_pi05.py:113-124).
"""

from __future__ import annotations

import threading
import time
from typing import Iterable

from .exceptions import CommTimeoutError, PeerLostError

STATUS_TEXT = {1: "TMA data never arrived (full barrier)", 2: "a pipeline stage was never released (empty barrier)",
               3: "the accumulator barrier never completed", 4: "a peer rank's arrival flag never came"}


def raise_for_kernel_status(status: int | None = None, *, what: str = "step") -> None:
    """0 -> nothing. 4 -> :class:`CommTimeoutError` (a peer did not show up). Other codes -> ``RuntimeError``."""
    if status is None:
        from .. import ops

        status = ops.kernel_status()
    if status == 0:
        return
    msg = f"{what}: device wait timed out ({STATUS_TEXT.get(status, f'status {status}')})"
    if status == 4:
        raise CommTimeoutError(msg)
    raise RuntimeError(msg)


def check_step_status(*, what: str = "step", force: bool = False) -> None:
    """The per-step sync point of a serving loop: read the device status word where the step's outputs
    leave the device anyway and turn a device-wait time-out into an exception BEFORE the next step runs
    on stale data.

    With peer groups open the ranks first agree on the worst status (one tiny all-reduce over each group),
    so that either every rank raises or none does; on a non-zero status every rank resets the channel
    state of its groups (:meth:`PeerGroup.reset_channels`, a collective) and raises. Without peer groups
    nothing is read unless ``force`` (or ``PHYAI_CHECK_KERNEL_STATUS=1``) asks for it: single-GPU
    kernels wait only on their own copies."""
    import os

    import torch

    from .symm import PeerGroup

    groups = PeerGroup.open_groups() if torch.cuda.is_available() else []
    if not groups and not force and os.environ.get("PHYAI_CHECK_KERNEL_STATUS", "0") in ("0", "", "false", "off"):
        return
    from .. import ops

    status = int(ops.kernel_status())
    if groups:
        import torch.distributed as dist

        t = torch.tensor([status], dtype=torch.int32, device=groups[0].device)
        for g in groups:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=g.group)
        status = int(t.item())
        if status != 0:
            for g in groups:
                g.reset_channels()
    raise_for_kernel_status(status, what=what)


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process runs)."""

    def __init__(self) -> None:
        self._d: dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            if key not in self._d:
                raise KeyError(key)
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, *, interval_s: float = 0.5, prefix: str = "hb", clock=time.time) -> None:
        self.store, self.rank, self.world, self.interval_s, self.prefix, self.clock = store, rank, world, interval_s, prefix, clock
        self._n = 0
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._n += 1
        self.store.set(self._key(self.rank), f"{self._n}:{self.clock():.6f}")

    def start(self) -> "Heartbeat":
        self.beat()
        if self.interval_s > 0 and self._thread is None:
            def loop():
                while not self._stop.wait(self.interval_s):
                    try:
                        self.beat()
                    except Exception:   # the store went away with the job
                        return
            self._thread = threading.Thread(target=loop, name="phyai-heartbeat", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * max(self.interval_s, 0.1))
            self._thread = None

    def last_seen(self, r: int) -> float | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            raw = self.store.get(self._key(r))
        except Exception:
            return None
        try:
            return float(raw.decode().split(":")[1])
        except (IndexError, ValueError):
            return None

    def stale_peers(self, deadline_s: float, ranks: Iterable[int] | None = None) -> list[int]:
        now = self.clock()
        out = []
        for r in (range(self.world) if ranks is None else ranks):
            if r == self.rank:
                continue
            seen = self.last_seen(r)
            if seen is None or now - seen > deadline_s:
                out.append(r)
        return out

    def check_peers(self, deadline_s: float, ranks: Iterable[int] | None = None) -> None:
        lost = self.stale_peers(deadline_s, ranks)
        if lost:
            raise PeerLostError(f"rank {self.rank}: no heartbeat from ranks {lost} within {deadline_s:.1f} s")


__all__ = ["Heartbeat", "DictStore", "raise_for_kernel_status", "check_step_status", "STATUS_TEXT"]
