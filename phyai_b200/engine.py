"""Engine: configuration resolution, device / process-group / mesh bring-up, plugin host.

``Engine(EngineArgs(plugin="pi05", plugin_args=PI05Args(...), config=EngineConfig(...)))``
then ``engine.step(request)`` and ``engine.close()``. Plugins register with
``@Engine.register`` and implement :class:`Entry`. Same public surface as the reference
(phyai/src/phyai/engine.py:83-400).
"""

from __future__ import annotations

import abc
import dataclasses
import importlib
import logging
import time
from dataclasses import dataclass, field
from typing import Any, ClassVar

import torch

from . import parallel as P
from .engine_config import EngineConfig, init_engine_config
from .layers import linear as L
from .utils.cuda import init_cublas, init_cuda
from .utils.logging import this_rank_log
from .utils.metrics import metrics

logger = logging.getLogger(__name__)


@dataclass
class EntryArgs:
    """Base class of every plugin's argument bundle."""


class Entry(abc.ABC):
    """One servable model family."""

    name: ClassVar[str]
    args_cls: ClassVar[type[EntryArgs]]

    @abc.abstractmethod
    def setup(self, args: EntryArgs) -> None: ...

    @abc.abstractmethod
    def step(self, request: Any) -> Any: ...

    def close(self) -> None:
        pass

    def dump_targets(self) -> dict[str, torch.nn.Module]:
        """Modules whose leaf outputs the tensor dumper records (name -> module)."""
        return {}


@dataclass
class EngineArgs:
    plugin: str
    plugin_args: EntryArgs
    config: EngineConfig | None = None


_BUILTIN_PLUGINS = {
    "pi05": "phyai_b200.models.pi05.main_pi05",
    "pi05_wn": "phyai_b200.models.pi05.main_pi05_wn",
    "pi05_tp": "phyai_b200.models.pi05.main_pi05_tp",
    "pi0": "phyai_b200.models.pi0.main_pi0",
    "pi0_wn": "phyai_b200.models.pi0.main_pi0_wn",
    "cosmos3": "phyai_b200.models.cosmos3.main_cosmos3",
    "cosmos3_wn": "phyai_b200.models.cosmos3.main_cosmos3_wn",
    "cosmos3_policy": "phyai_b200.models.cosmos3.main_cosmos3_policy",
    "cosmos3_policy_wn": "phyai_b200.models.cosmos3.main_cosmos3_policy_wn",
}


class Engine:
    _plugins: ClassVar[dict[str, type[Entry]]] = {}

    @classmethod
    def register(cls, entry_cls: type[Entry]) -> type[Entry]:
        name = getattr(entry_cls, "name", None)
        if not isinstance(name, str) or not name:
            raise TypeError(f"{entry_cls.__name__} needs a non-empty class attribute `name`")
        if not isinstance(getattr(entry_cls, "args_cls", None), type) or not issubclass(entry_cls.args_cls, EntryArgs):
            raise TypeError(f"{entry_cls.__name__}.args_cls must subclass EntryArgs")
        prev = cls._plugins.get(name)
        if prev is not None and prev is not entry_cls:
            raise ValueError(f"plugin name {name!r} is already taken by {prev.__name__}")
        cls._plugins[name] = entry_cls
        return entry_cls

    @classmethod
    def plugin_names(cls) -> list[str]:
        return sorted(set(cls._plugins) | set(_BUILTIN_PLUGINS))

    @classmethod
    def _resolve_plugin(cls, name: str) -> type[Entry]:
        if name not in cls._plugins and name in _BUILTIN_PLUGINS:
            importlib.import_module(_BUILTIN_PLUGINS[name])     # registers itself on import
        if name not in cls._plugins:
            raise KeyError(f"unknown plugin {name!r}; available: {cls.plugin_names()}")
        return cls._plugins[name]

    def __init__(self, args: EngineArgs) -> None:
        explicit = args.config
        cfg = EngineConfig.from_env(base=explicit if explicit is not None else EngineConfig.auto(), explicit=explicit)
        self._dumper = None
        if cfg.runtime.debug_tensor_dump_dir and cfg.runtime.use_cuda_graph:
            # hooks cannot observe kernels replayed from a graph: dumping forces the eager path
            cfg = cfg.replace(runtime={"use_cuda_graph": False})
            this_rank_log(logger, logging.WARNING, "tensor dump enabled: CUDA graphs switched off")
        self.config = init_engine_config(cfg)
        self.device = init_cuda(cfg.device.target, cfg.device.params_dtype)
        init_cublas()
        p = cfg.parallel
        self._owns_pg = P.init_dist(p.world_size, self.device.type)
        self.mesh = P.init(p.layout, P.AXES, device=self.device.type)
        L.init()
        entry_cls = self._resolve_plugin(args.plugin)
        if not isinstance(args.plugin_args, entry_cls.args_cls):
            raise TypeError(f"plugin {args.plugin!r} expects {entry_cls.args_cls.__name__}, "
                            f"got {type(args.plugin_args).__name__}")
        self.plugin_name = args.plugin
        self.entry: Entry = entry_cls()
        self.entry.setup(args.plugin_args)
        if cfg.runtime.debug_tensor_dump_dir:
            from .runtime.tensor_dump import TensorDumper

            self._dumper = TensorDumper.from_config(cfg.runtime)
            for name, mod in self.entry.dump_targets().items():
                self._dumper.attach(mod, prefix=name)
        self._closed = False

    def step(self, request: Any) -> Any:
        if self._closed:
            raise RuntimeError("Engine.step after close()")
        t0 = time.perf_counter()
        out = self.entry.step(request)
        if self.device.type == "cuda":
            # the step's sync point: a device wait that gave up (a late or lost peer) must surface here,
            # with the channels reset, not as stale rows in the next step
            from .parallel.health import check_step_status

            check_step_status(what=f"{self.plugin_name}.step")
        if self._dumper is not None:
            self._dumper.flush()
        m = metrics()
        m.inc(f"engine.steps.{self.plugin_name}")
        m.observe(f"engine.step_host_ms.{self.plugin_name}", (time.perf_counter() - t0) * 1e3)   # host side: launch + any sync the plugin does
        return out

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            self.entry.close()
        finally:
            if self._dumper is not None:
                self._dumper.detach()
            P.shutdown()
            if self._owns_pg:
                P.destroy_dist()

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


__all__ = ["Engine", "EngineArgs", "Entry", "EntryArgs"]
