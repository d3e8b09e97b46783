"""Tensor dumper: records the output of selected leaf modules, one file per engine step.

Forward hooks on leaf modules copy outputs to the CPU under their dotted names (a module
called more than once in a step gets ``::call1``, ``::call2`` ... suffixes). ``flush()``
writes ``<dir>/rank{R}_pid{P}/pass{N:05d}.pt`` and starts the next pass. Selection is by
a list of regexes or by a predicate ``"pkg.mod:func"`` / ``"/path/file.py:func"`` that is
called as ``predicate(name)`` or, when it takes two arguments, ``predicate(name, module)``.
Only tensors are kept: other leaves of an output are dropped and a sequence left with one
tensor (a linear's ``(out, bias)`` pair with no bias) is stored as that tensor, so files
written here and by the reference from the same module tree have the same keys and values.
Dumping needs the eager path (hooks cannot see kernels replayed from a CUDA graph); the
engine switches graphs off when a dump directory is configured.
Reference: phyai/src/phyai/runtime/tensor_dump.py:112-429.
"""

from __future__ import annotations

import importlib
import importlib.util
import inspect
import os
import re
from collections.abc import Mapping
from pathlib import Path
from typing import Any, Callable

import torch


def _load_predicate(spec: str) -> Callable[..., bool]:
    target, _, func = spec.rpartition(":")
    if not target or not func:
        raise ValueError(f"dump filter function {spec!r} must look like 'pkg.mod:func' or '/path.py:func'")
    if target.endswith(".py") or os.sep in target:
        if not Path(target).is_file():
            raise FileNotFoundError(f"dump filter file not found: {target}")
        s = importlib.util.spec_from_file_location("_phyai_b200_dump_filter", target)
        mod = importlib.util.module_from_spec(s)
        s.loader.exec_module(mod)  # type: ignore[union-attr]
    else:
        mod = importlib.import_module(target)
    fn = getattr(mod, func)
    if not callable(fn):
        raise TypeError(f"dump filter {spec!r} is not callable")
    return fn


def _takes_module(fn: Callable[..., bool]) -> bool:
    """Whether a predicate wants ``(name, module)`` rather than ``(name)``."""
    try:
        params = [p for p in inspect.signature(fn).parameters.values()
                  if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD) and p.default is p.empty]
        return len(params) >= 2 or any(p.kind is p.VAR_POSITIONAL for p in inspect.signature(fn).parameters.values())
    except (TypeError, ValueError):
        return False


def _to_cpu(obj: Any) -> Any:
    """Tensors of ``obj`` detached on the CPU; ``None`` when it holds none."""
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, (tuple, list)):
        items = [x for x in (_to_cpu(o) for o in obj) if x is not None]
        return None if not items else items[0] if len(items) == 1 else items
    if isinstance(obj, Mapping):
        out = {k: x for k, x in ((k, _to_cpu(v)) for k, v in obj.items()) if x is not None}
        return out or None
    return None


class TensorDumper:
    """``TensorDumper(out_dir, patterns=..., predicate=...)`` followed by ``attach(module, prefix)``; or, in the reference's
    form, ``TensorDumper({"name": module, ...}, dump_dir=..., filter=None | [regex, ...] | predicate, rank=...)``, which
    attaches at once."""

    def __init__(self, out_dir: "str | Path | Mapping[str, torch.nn.Module] | None" = None, *, patterns: "tuple[str, ...] | list[str] | None" = None,
                 predicate: Callable[..., bool] | None = None, dump_dir: str | Path | None = None, filter: Any = None,
                 rank: int | None = None, world_size: int | None = None) -> None:
        targets = None
        if isinstance(out_dir, Mapping):
            targets, out_dir = out_dir, None
            if not targets:
                raise ValueError("TensorDumper needs at least one target module")
        if out_dir is None:
            out_dir = dump_dir
        if out_dir is None:
            raise ValueError("TensorDumper needs a directory (out_dir or dump_dir)")
        if filter is not None:
            if patterns is not None or predicate is not None:
                raise ValueError("pass filter, or patterns / predicate, not both")
            if isinstance(filter, str):
                raise TypeError(f"filter is None, a sequence of regex strings or a callable; wrap a single pattern in a list: [{filter!r}]")
            if callable(filter):
                predicate = filter
            else:
                patterns = tuple(filter)
        if patterns is not None and predicate is not None:
            raise ValueError("pass regex patterns or a predicate, not both")
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else int(rank)
        self.world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else int(world_size)
        self.dir = Path(out_dir) / f"rank{self.rank}_pid{os.getpid()}"
        self.dir.mkdir(parents=True, exist_ok=True)
        self._regex = [re.compile(p) for p in patterns] if patterns is not None else None
        self._predicate = predicate
        self._predicate_takes_module = predicate is not None and _takes_module(predicate)
        self._hooks: list[Any] = []
        self._records: dict[str, Any] = {}
        self._calls: dict[str, int] = {}
        self.pass_index = 0
        for name, module in (targets or {}).items():
            self.attach(module, prefix=name)

    @classmethod
    def from_config(cls, runtime) -> "TensorDumper":
        pred = _load_predicate(runtime.debug_tensor_dump_filter_fn) if runtime.debug_tensor_dump_filter_fn else None
        return cls(runtime.debug_tensor_dump_dir, patterns=runtime.debug_tensor_dump_filter, predicate=pred)

    @property
    def process_dir(self) -> Path:
        return self.dir

    def wants(self, name: str, module: torch.nn.Module | None = None) -> bool:
        if self._predicate is not None:
            return bool(self._predicate(name, module) if self._predicate_takes_module else self._predicate(name))
        if self._regex is not None:
            return any(r.search(name) for r in self._regex)      # an empty list selects nothing
        return True

    def attach(self, root: torch.nn.Module, prefix: str = "") -> int:
        n = 0
        for name, mod in root.named_modules():
            if any(True for _ in mod.children()):
                continue  # leaves only
            full = f"{prefix}.{name}" if prefix and name else (prefix or name)
            if not self.wants(full, mod):
                continue
            self._hooks.append(mod.register_forward_hook(self._make_hook(full)))
            n += 1
        return n

    def _store(self, name: str, value: Any) -> None:
        value = _to_cpu(value)
        if value is None:
            return
        k = self._calls.get(name, 0)
        self._calls[name] = k + 1
        self._records[name if k == 0 else f"{name}::call{k}"] = value

    def _make_hook(self, name: str):
        def hook(_mod, _inp, out):
            self._store(name, out)
        return hook

    def record(self, name: str, value: Any) -> None:
        """Manual entry for values that are not module outputs (e.g. sampler state)."""
        if self.wants(name):
            self._store(name, value)

    def flush(self) -> Path | None:
        if not self._records:
            self._calls.clear()
            return None
        path = self.dir / f"pass{self.pass_index:05d}.pt"
        torch.save(self._records, path)
        self._records, self._calls = {}, {}
        self.pass_index += 1
        return path

    flush_pass = flush

    def detach(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    @staticmethod
    def load_pass(directory: str | Path, index: int | None = None) -> dict[str, Any]:
        """One pass file: ``load_pass(process_dir, index)`` or ``load_pass(path_of_the_file)``."""
        path = Path(directory) if index is None else Path(directory) / f"pass{index:05d}.pt"
        return torch.load(path, map_location="cpu", weights_only=False)


load_filter_fn = _load_predicate
load_pass = TensorDumper.load_pass


def register_tensor_dumper(module: "torch.nn.Module | Mapping[str, torch.nn.Module]", out_dir: str | Path | None = None, *, prefix: str = "",
                           patterns: tuple[str, ...] | None = None, filter_fn: str | Callable[..., bool] | None = None,
                           dump_dir: str | Path | None = None, filter: Any = None, rank: int | None = None,
                           world_size: int | None = None) -> TensorDumper:
    """A dumper hooked onto ``module``'s leaf modules in one call (``filter_fn``: a predicate or its ``"pkg.mod:func"`` spec).
    With a mapping of named modules and ``dump_dir=`` / ``filter=`` it is the reference's call."""
    if isinstance(module, Mapping):
        return TensorDumper(module, dump_dir=dump_dir if dump_dir is not None else out_dir, filter=filter, rank=rank, world_size=world_size)
    pred = _load_predicate(filter_fn) if isinstance(filter_fn, str) else filter_fn
    dumper = TensorDumper(out_dir if out_dir is not None else dump_dir, patterns=patterns, predicate=pred, filter=filter, rank=rank, world_size=world_size)
    dumper.attach(module, prefix=prefix)
    return dumper


__all__ = ["TensorDumper", "load_filter_fn", "load_pass", "register_tensor_dumper"]
