"""vGPU: carve one GPU's SMs into partitions (CUDA green contexts), each with its own stream.

A latency-critical graph (the action expert) can then run beside a throughput job (vision for the
next request) without the two fighting over SMs. Work submitted to a partition's stream only ever
occupies that partition's SMs; CUDA graphs captured on it inherit the restriction
(``runtime.capture_on_stream``).

The driver calls go through a small ``DriverApi`` object so the partitioning arithmetic and the
life-cycle are testable without a GPU. Two real backends: ``CudaDriver`` binds the green-context
entry points of cuda-python and supports disjoint splits plus a remainder; ``TorchGreenDriver``
wraps ``torch.cuda.green_contexts`` and, like the reference's torch backend, serves one shard per
call (several of its contexts may share SMs). ``PHYAI_VGPU_BACKEND`` = ``cuda`` | ``torch`` picks one.
Every :class:`vGPU` owns a ``torch.cuda.MemPool`` (on CUDA): allocations made inside ``activate()``
come from that pool, so a partition's activations never fragment its neighbour's.
Reference: phyai/src/phyai/vgpu/{vgpu,partition,topology,backend,state}.py, backends/torch.py:27-90.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Any, Iterator, Protocol, Sequence


class VGPUError(Exception):
    pass


class VGPUNotApplicableError(VGPUError):
    """Multi-rank job, CPU build, or a GPU older than compute capability 8.0."""


class VGPURuntimeError(VGPUError):
    pass


class VGPUDriverError(VGPUError):
    pass


def get_sm_count_constraint(cc: tuple[int, int]) -> tuple[int, int]:
    """(minimum, granularity) of an SM partition for a compute capability."""
    major = cc[0]
    if major == 6:
        return 1, 1
    if major == 7:
        return 2, 2
    if major == 8:
        return 4, 2
    if major >= 9:
        return 8, 8
    raise VGPURuntimeError(f"compute capability {cc[0]}.{cc[1]} has no green contexts")


def round_up_sm_count(req: int, cc: tuple[int, int]) -> int:
    if req <= 0:
        raise VGPURuntimeError(f"sm_count must be positive, got {req}")
    lo, step = get_sm_count_constraint(cc)
    return -(-max(req, lo) // step) * step


def validate_total(rounded: Sequence[int], total_sms: int) -> None:
    if sum(rounded) > total_sms:
        raise VGPURuntimeError(f"requested {sum(rounded)} SMs (rounded {list(rounded)}) of {total_sms}")


class DriverApi(Protocol):
    """What the partitioner needs from CUDA. ``split`` returns one opaque resource per count plus the remainder."""

    def capability(self, device: int) -> tuple[int, int]: ...
    def sm_count(self, device: int) -> int: ...
    def split(self, device: int, counts: Sequence[int]) -> list[tuple[Any, int]]: ...
    def make_stream(self, device: int, resource: Any) -> tuple[Any, Any]: ...   # -> (green context, stream object)
    def destroy(self, ctx: Any) -> None: ...


class CudaDriver:
    """Green contexts through cuda-python's driver bindings."""

    def __init__(self) -> None:
        from cuda.bindings import driver as drv   # cuda-python >= 12.6

        self.d = drv

    def _ok(self, res, what: str):
        err, *vals = res
        if int(err) != 0:
            raise VGPUDriverError(f"{what} failed with CUDA error {int(err)}")
        return vals[0] if len(vals) == 1 else vals

    def capability(self, device: int) -> tuple[int, int]:
        import torch

        return torch.cuda.get_device_capability(device)

    def sm_count(self, device: int) -> int:
        import torch

        return torch.cuda.get_device_properties(device).multi_processor_count

    def split(self, device: int, counts: Sequence[int]) -> list[tuple[Any, int]]:
        d = self.d
        dev = self._ok(d.cuDeviceGet(device), "cuDeviceGet")
        res = self._ok(d.cuDeviceGetDevResource(dev, d.CUdevResourceType.CU_DEV_RESOURCE_TYPE_SM), "cuDeviceGetDevResource")
        out = []
        remaining = res
        for c in counts:
            groups, _n, rem = self._ok(d.cuDevSmResourceSplitByCount(1, remaining, 0, c), "cuDevSmResourceSplitByCount")
            out.append((groups[0], int(groups[0].sm.smCount)))
            remaining = rem
        out.append((remaining, int(remaining.sm.smCount)))
        return out

    def make_stream(self, device: int, resource: Any) -> tuple[Any, Any]:
        import torch

        d = self.d
        dev = self._ok(d.cuDeviceGet(device), "cuDeviceGet")
        desc = self._ok(d.cuDevResourceGenerateDesc([resource], 1), "cuDevResourceGenerateDesc")
        ctx = self._ok(d.cuGreenCtxCreate(desc, dev, d.CUgreenCtxCreate_flags.CU_GREEN_CTX_DEFAULT_STREAM), "cuGreenCtxCreate")
        raw = self._ok(d.cuGreenCtxStreamCreate(ctx, d.CUstream_flags.CU_STREAM_NON_BLOCKING, 0), "cuGreenCtxStreamCreate")
        return ctx, torch.cuda.ExternalStream(int(raw), device=device)

    def destroy(self, ctx: Any) -> None:
        self._ok(self.d.cuGreenCtxDestroy(ctx), "cuGreenCtxDestroy")


class TorchGreenDriver:
    """One shard per call through ``torch.cuda.green_contexts.GreenContext`` (no disjointness guarantee
    between calls, no remainder: ``split`` with more than one count is refused)."""

    def capability(self, device: int) -> tuple[int, int]:
        import torch

        return torch.cuda.get_device_capability(device)

    def sm_count(self, device: int) -> int:
        import torch

        return torch.cuda.get_device_properties(device).multi_processor_count

    def split(self, device: int, counts: Sequence[int]) -> list[tuple[Any, int]]:
        if len(counts) != 1:
            raise VGPURuntimeError("the torch backend makes one shard per call (its contexts may share SMs); "
                                   "use the cuda backend for disjoint splits")
        return [(("torch", int(counts[0])), int(counts[0])), (None, 0)]

    def make_stream(self, device: int, resource: Any) -> tuple[Any, Any]:
        import torch
        from torch.cuda.green_contexts import GreenContext

        _, n = resource
        g = GreenContext.create(num_sms=n, device_id=device)
        try:
            stream = g.Stream()
        except AttributeError:           # older binding: make a stream while the context is current
            g.set_context()
            try:
                stream = torch.cuda.Stream(device=device)
            finally:
                g.pop_context()
        return g, stream

    def destroy(self, ctx: Any) -> None:
        return None                      # released with the last reference


class BackendCapabilityError(VGPUError):
    """The chosen backend cannot do what was asked on this machine (no cuda-python, a torch build without green contexts)."""


# name -> factory of a DriverApi; out-of-tree backends join with ``register_vgpu_backend``
_BACKENDS: dict[str, Any] = {"cuda": CudaDriver, "torch": TorchGreenDriver}
_CHOSEN: dict[str, str | None] = {"name": None}
GreenCtxBackend = TorchGreenDriver


def register_vgpu_backend(name: str):
    """Decorator: make a :class:`DriverApi` factory selectable by name (``set_backend`` / ``PHYAI_VGPU_BACKEND``).
    Reference: phyai/src/phyai/vgpu/backend.py."""
    def deco(factory):
        if name in _BACKENDS and _BACKENDS[name] is not factory:
            raise ValueError(f"vGPU backend {name!r} is already registered")
        _BACKENDS[name] = factory
        return factory
    return deco


register = register_vgpu_backend


def known_backends() -> list[str]:
    return sorted(_BACKENDS)


def set_backend(name: str | None) -> None:
    """Choose the backend the next ``init()`` builds (``None``: back to ``PHYAI_VGPU_BACKEND`` / automatic)."""
    if name is not None and name not in _BACKENDS:
        raise VGPURuntimeError(f"unknown vGPU backend {name!r}; known: {known_backends()}")
    _CHOSEN["name"] = name


def get_backend() -> str:
    """The name ``default_driver()`` resolves now: an explicit choice, else the environment, else ``"auto"``."""
    from ..env import envs

    if _CHOSEN["name"]:
        return _CHOSEN["name"]
    from ..engine_config import get_engine_config

    try:
        configured = get_engine_config().backends.vgpu          # EngineConfig already overlays PHYAI_VGPU_BACKEND
    except Exception:  # noqa: BLE001 - no engine configuration installed yet
        configured = None
    return (configured or envs.PHYAI_VGPU_BACKEND.get() or "auto").lower()


def default_driver() -> DriverApi:
    """The chosen backend's driver (``set_backend`` / ``PHYAI_VGPU_BACKEND``: a registered name; ``auto`` or unset:
    cuda-python when importable, else torch green contexts)."""
    want = get_backend()
    want = {"driver": "cuda", "green_ctx": "torch", "greenctx": "torch"}.get(want, want)     # spellings of EngineConfig / the reference
    if want in ("", "auto"):
        try:
            return CudaDriver()
        except ImportError:
            return TorchGreenDriver()
    if want not in _BACKENDS:
        raise VGPURuntimeError(f"unknown vGPU backend {want!r}; known: {known_backends()}")
    try:
        return _BACKENDS[want]()
    except ImportError as e:
        raise BackendCapabilityError(f"vGPU backend {want!r} is not usable here: {e}") from e


@dataclass(frozen=True)
class Shard:
    name: str
    device: int
    sm_count: int
    requested_sm_count: int
    is_remainder: bool
    stream: Any
    backend: str
    _ctx: Any


_STATE: dict[str, Any] = {"driver": None, "device": None, "open": []}


def init(device: int = 0, *, driver: DriverApi | None = None, world_size: int = 1) -> DriverApi:
    """Once per process, before any split. Refuses multi-rank jobs (each rank owns a whole GPU) and pre-Ampere GPUs."""
    if world_size > 1:
        raise VGPUNotApplicableError("SM partitioning is for single-GPU serving; multi-rank jobs own whole GPUs")
    drv = driver if driver is not None else default_driver()
    if drv.capability(device)[0] < 8:
        raise VGPUNotApplicableError(f"green contexts need compute capability >= 8.0, device has {drv.capability(device)}")
    _STATE.update(driver=drv, device=device)
    return drv


def _driver() -> DriverApi:
    if _STATE["driver"] is None:
        raise VGPURuntimeError("call phyai_b200.vgpu.init() first")
    return _STATE["driver"]


def split_device_by_sm_count(sm_counts: Sequence[int], *, device: int | None = None) -> list[Shard]:
    """One shard per requested count (rounded up to the hardware granularity) and a trailing remainder shard."""
    drv = _driver()
    dev = _STATE["device"] if device is None else device
    cc, total = drv.capability(dev), drv.sm_count(dev)
    rounded = [round_up_sm_count(c, cc) for c in sm_counts]
    validate_total(rounded, total)
    shards = []
    parts = drv.split(dev, rounded)
    for i, ((res, n), req) in enumerate(zip(parts, [*sm_counts, None])):
        rem = i == len(parts) - 1
        if rem and n == 0:
            continue
        ctx, stream = drv.make_stream(dev, res)
        shards.append(Shard(f"shard_{i}{'_rem' if rem else ''}", dev, n, n if rem else int(req), rem, stream, type(drv).__name__, ctx))
    return shards


def split_device(num_groups: int, min_count: int, *, device: int | None = None) -> list[Shard]:
    """``num_groups`` equal shards of at least ``min_count`` SMs, plus the remainder."""
    if num_groups <= 0:
        raise VGPURuntimeError("num_groups must be positive")
    return split_device_by_sm_count([min_count] * num_groups, device=device)


class vGPU:
    """A shard in use: ``with v.activate():`` makes its stream current; ``close`` destroys the green context."""

    def __init__(self, shard: Shard) -> None:
        self.shard, self._closed = shard, False
        self.mem_pool = None
        try:
            import torch

            if isinstance(shard.stream, torch.cuda.Stream) and hasattr(torch.cuda, "MemPool"):
                self.mem_pool = torch.cuda.MemPool()
        except ImportError:  # pragma: no cover
            pass
        _STATE["open"].append(self)

    name = property(lambda s: s.shard.name)
    sm_count = property(lambda s: s.shard.sm_count)
    stream = property(lambda s: s.shard.stream)

    @classmethod
    def from_shard(cls, shard: Shard) -> "vGPU":
        return cls(shard)

    @contextlib.contextmanager
    def activate(self) -> Iterator["vGPU"]:
        if self._closed:
            raise VGPURuntimeError(f"{self.name} is closed")
        from ..runtime import capture_on_stream

        cm, pool = contextlib.nullcontext(), contextlib.nullcontext()
        try:
            import torch

            if isinstance(self.stream, torch.cuda.Stream):
                cm = torch.cuda.stream(self.stream)
                if self.mem_pool is not None:
                    pool = torch.cuda.use_mem_pool(self.mem_pool)
        except ImportError:  # pragma: no cover
            pass
        with cm, pool, capture_on_stream(self.stream):
            yield self

    def close(self) -> None:
        if self._closed:
            return
        _driver().destroy(self.shard._ctx)
        self.mem_pool = None
        self._closed = True
        if self in _STATE["open"]:
            _STATE["open"].remove(self)


def create_vgpus(sm_counts: Sequence[int], *, device: int | None = None, include_remainder: bool = True) -> list[vGPU]:
    return [vGPU(s) for s in split_device_by_sm_count(sm_counts, device=device) if include_remainder or not s.is_remainder]


def close_all() -> None:
    for v in list(_STATE["open"]):
        v.close()


def _reset_for_tests() -> None:
    _STATE.update(driver=None, device=None, open=[])
    _CHOSEN["name"] = None


__all__ = ["VGPUError", "VGPUNotApplicableError", "VGPURuntimeError", "VGPUDriverError", "get_sm_count_constraint", "round_up_sm_count",
           "validate_total", "DriverApi", "CudaDriver", "TorchGreenDriver", "default_driver", "Shard", "init", "split_device", "split_device_by_sm_count", "vGPU", "create_vgpus",
           "close_all", "BackendCapabilityError", "GreenCtxBackend", "register_vgpu_backend", "register", "known_backends", "set_backend",
           "get_backend"]
