"""Profiler front-end: named scopes around pipeline stages.

``event_scope("pi05.forward")`` is free when no profiler is installed. Installable
back-ends (reference: phyai/src/phyai/utils/profile.py:81-533):

* ``NoOpProfiler``   default
* ``TorchProfiler``  ``torch.profiler`` chrome/perfetto trace per rank
* ``NvtxProfiler``   NVTX ranges + ``cudaProfilerStart/Stop`` window for an external
                     capture tool, optional per-module ranges via forward hooks
* ``TimelineProfiler`` CUDA-event timers per scope, dumped as a JSON timeline (no
                     external tool needed; feeds the metrics registry)
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterator

import torch


@dataclass
class ProfilerConfig:
    kind: str = "none"                 # none | torch | nvtx | timeline
    output_dir: str = "./profiles_out"
    prefix: str = "phyai_b200"
    only_rank: int | None = None
    record_shapes: bool = False
    with_stack: bool = False
    profile_memory: bool = False
    module_ranges: bool = False

    def __post_init__(self) -> None:
        if self.kind == "nsys":
            self.kind = "nvtx"
        if self.kind not in ("none", "torch", "nvtx", "timeline"):
            raise ValueError(f"unknown profiler kind {self.kind!r}")


class NoOpProfiler:
    active = False

    def start(self) -> None: ...
    def stop(self) -> None: ...

    def scope(self, name: str):
        return contextlib.nullcontext()

    def mark(self, name: str) -> None: ...


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


class TorchProfiler(NoOpProfiler):
    active = True

    def __init__(self, cfg: ProfilerConfig) -> None:
        self.cfg = cfg
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, record_shapes=cfg.record_shapes,
                                            with_stack=cfg.with_stack, profile_memory=cfg.profile_memory)
        self._run = 0

    def start(self) -> None:
        self._prof.start()

    def stop(self) -> None:
        self._prof.stop()
        out = Path(self.cfg.output_dir)
        out.mkdir(parents=True, exist_ok=True)
        self._prof.export_chrome_trace(str(out / f"{self.cfg.prefix}_{self._run}_rank{_rank()}.trace.json.gz"))
        self._run += 1

    def scope(self, name: str):
        return torch.profiler.record_function(name)


class NvtxProfiler(NoOpProfiler):
    active = True

    def __init__(self, cfg: ProfilerConfig) -> None:
        self.cfg = cfg
        self._hooks: list[Any] = []

    def start(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStart()

    def stop(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    @contextlib.contextmanager
    def scope(self, name: str) -> Iterator[None]:
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()

    def mark(self, name: str) -> None:
        torch.cuda.nvtx.mark(name)

    def attach_modules(self, root: torch.nn.Module, prefix: str = "") -> None:
        for n, m in root.named_modules():
            label = f"{prefix}{n}" if n else (prefix or type(root).__name__)
            self._hooks.append(m.register_forward_pre_hook(lambda _m, _i, _l=label: torch.cuda.nvtx.range_push(_l)))
            self._hooks.append(m.register_forward_hook(lambda _m, _i, _o: torch.cuda.nvtx.range_pop()))


class TimelineProfiler(NoOpProfiler):
    """CUDA-event (or wall-clock on CPU) timing of every scope; ``summary()`` aggregates per name."""

    active = True

    def __init__(self, cfg: ProfilerConfig | None = None) -> None:
        self.cfg = cfg or ProfilerConfig(kind="timeline")
        self._events: list[tuple[str, Any, Any]] = []
        self._wall: list[tuple[str, float]] = []
        self.enabled = False

    def start(self) -> None:
        self.enabled = True

    def stop(self) -> None:
        self.enabled = False

    @contextlib.contextmanager
    def scope(self, name: str) -> Iterator[None]:
        if not self.enabled:
            yield
            return
        if torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._events.append((name, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._wall.append((name, (time.perf_counter() - t0) * 1e3))

    def summary(self) -> dict[str, dict[str, float]]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        rows = [(n, a.elapsed_time(b)) for n, a, b in self._events] + list(self._wall)
        out: dict[str, dict[str, float]] = {}
        for n, ms in rows:
            d = out.setdefault(n, {"count": 0, "total_ms": 0.0, "max_ms": 0.0})
            d["count"] += 1
            d["total_ms"] += ms
            d["max_ms"] = max(d["max_ms"], ms)
        for d in out.values():
            d["mean_ms"] = d["total_ms"] / max(d["count"], 1)
        return out

    def dump(self, path: str | Path | None = None) -> Path:
        p = Path(path) if path else Path(self.cfg.output_dir) / f"{self.cfg.prefix}_timeline_rank{_rank()}.json"
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(json.dumps(self.summary(), indent=2))
        return p


_PROFILER: NoOpProfiler = NoOpProfiler()


Profiler = NoOpProfiler          # the interface every profiler here implements (scope, mark, start, stop, step)
NsysProfiler = NvtxProfiler      # Nsight Systems reads the NVTX ranges and the cudaProfilerStart / Stop window


def make_profiler(cfg: ProfilerConfig | None) -> NoOpProfiler:
    """A profiler for ``cfg`` without installing it (``install_profiler`` does both)."""
    if cfg is None or cfg.kind == "none":
        return NoOpProfiler()
    kinds = {"torch": TorchProfiler, "nvtx": NvtxProfiler, "nsys": NvtxProfiler, "timeline": TimelineProfiler}
    if cfg.kind not in kinds:
        raise ValueError(f"unknown profiler kind {cfg.kind!r}; known: none, {', '.join(kinds)}")
    return kinds[cfg.kind](cfg)


def set_profiler(profiler: NoOpProfiler | None) -> NoOpProfiler:
    """Install a profiler object as the process-wide one (``None``: the no-op profiler)."""
    global _PROFILER
    _PROFILER = profiler if profiler is not None else NoOpProfiler()
    return _PROFILER


def install_profiler(cfg: ProfilerConfig | None) -> NoOpProfiler:
    global _PROFILER
    if cfg is None or cfg.kind == "none" or (cfg.only_rank is not None and cfg.only_rank != _rank()):
        _PROFILER = NoOpProfiler()
    elif cfg.kind == "torch":
        _PROFILER = TorchProfiler(cfg)
    elif cfg.kind in ("nvtx", "nsys"):
        _PROFILER = NvtxProfiler(cfg)
    else:
        _PROFILER = TimelineProfiler(cfg)
    return _PROFILER


def get_profiler() -> NoOpProfiler:
    return _PROFILER


def event_scope(name: str):
    return _PROFILER.scope(name)


def mark_instant(name: str) -> None:
    _PROFILER.mark(name)


def add_profile_cli_args(parser: argparse.ArgumentParser) -> None:
    g = parser.add_argument_group("profiling")
    g.add_argument("--profile", default="none", choices=["none", "torch", "nvtx", "nsys", "timeline"])
    g.add_argument("--profile-dir", default="./profiles_out")
    g.add_argument("--profile-prefix", default="phyai_b200")
    g.add_argument("--profile-only-rank", type=int, default=None)
    g.add_argument("--profile-start-step", type=int, default=0)
    g.add_argument("--profile-num-steps", type=int, default=0)
    g.add_argument("--profile-record-shapes", action="store_true")
    g.add_argument("--profile-with-stack", action="store_true")
    g.add_argument("--profile-memory", action="store_true")
    g.add_argument("--profile-module-ranges", action="store_true")


def profile_config_from_args(args: argparse.Namespace) -> ProfilerConfig:
    return ProfilerConfig(kind=args.profile, output_dir=args.profile_dir, prefix=args.profile_prefix,
                          only_rank=args.profile_only_rank, record_shapes=args.profile_record_shapes,
                          with_stack=args.profile_with_stack, profile_memory=args.profile_memory,
                          module_ranges=args.profile_module_ranges)


__all__ = ["Profiler", "NsysProfiler", "make_profiler", "set_profiler", "ProfilerConfig", "NoOpProfiler", "TorchProfiler", "NvtxProfiler", "TimelineProfiler", "install_profiler",
           "get_profiler", "event_scope", "mark_instant", "add_profile_cli_args", "profile_config_from_args"]
