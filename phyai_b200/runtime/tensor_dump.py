"""Tensor dumper: records the output of selected leaf modules, one file per engine step.

Forward hooks on leaf modules copy outputs to the CPU under their dotted names (a module
called more than once in a step gets ``::call1``, ``::call2`` ... suffixes). ``flush()``
writes ``<dir>/rank{R}_pid{P}/pass{N:05d}.pt`` and starts the next pass. Selection is by
a list of regexes or by a predicate ``"pkg.mod:func"`` / ``"/path/file.py:func"``.
Dumping needs the eager path (hooks cannot see kernels replayed from a CUDA graph); the
engine switches graphs off when a dump directory is configured.
Reference: phyai/src/phyai/runtime/tensor_dump.py:137-429.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import re
from pathlib import Path
from typing import Any, Callable

import torch


def _load_predicate(spec: str) -> Callable[[str], bool]:
    target, _, func = spec.rpartition(":")
    if not target or not func:
        raise ValueError(f"dump filter function {spec!r} must look like 'pkg.mod:func' or '/path.py:func'")
    if target.endswith(".py") or os.sep in target:
        s = importlib.util.spec_from_file_location("_phyai_b200_dump_filter", target)
        mod = importlib.util.module_from_spec(s)
        s.loader.exec_module(mod)  # type: ignore[union-attr]
    else:
        mod = importlib.import_module(target)
    return getattr(mod, func)


def _to_cpu(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, (tuple, list)):
        return type(obj)(_to_cpu(o) for o in obj)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    return obj


class TensorDumper:
    def __init__(self, out_dir: str | Path, *, patterns: tuple[str, ...] | None = None,
                 predicate: Callable[[str], bool] | None = None) -> None:
        if patterns is not None and predicate is not None:
            raise ValueError("pass regex patterns or a predicate, not both")
        rank = int(os.environ.get("RANK", "0"))
        self.dir = Path(out_dir) / f"rank{rank}_pid{os.getpid()}"
        self.dir.mkdir(parents=True, exist_ok=True)
        self._regex = [re.compile(p) for p in patterns] if patterns else None
        self._predicate = predicate
        self._hooks: list[Any] = []
        self._records: dict[str, Any] = {}
        self._calls: dict[str, int] = {}
        self.pass_index = 0

    @classmethod
    def from_config(cls, runtime) -> "TensorDumper":
        pred = _load_predicate(runtime.debug_tensor_dump_filter_fn) if runtime.debug_tensor_dump_filter_fn else None
        return cls(runtime.debug_tensor_dump_dir, patterns=runtime.debug_tensor_dump_filter, predicate=pred)

    def wants(self, name: str) -> bool:
        if self._predicate is not None:
            return bool(self._predicate(name))
        if self._regex is not None:
            return any(r.search(name) for r in self._regex)
        return True

    def attach(self, root: torch.nn.Module, prefix: str = "") -> int:
        n = 0
        for name, mod in root.named_modules():
            if any(True for _ in mod.children()):
                continue  # leaves only
            full = f"{prefix}.{name}" if prefix and name else (prefix or name)
            if not self.wants(full):
                continue
            self._hooks.append(mod.register_forward_hook(self._make_hook(full)))
            n += 1
        return n

    def _make_hook(self, name: str):
        def hook(_mod, _inp, out):
            k = self._calls.get(name, 0)
            self._calls[name] = k + 1
            self._records[name if k == 0 else f"{name}::call{k}"] = _to_cpu(out)
        return hook

    def record(self, name: str, value: Any) -> None:
        """Manual entry for values that are not module outputs (e.g. sampler state)."""
        if self.wants(name):
            self._records[name] = _to_cpu(value)

    def flush(self) -> Path | None:
        if not self._records:
            self._calls.clear()
            return None
        path = self.dir / f"pass{self.pass_index:05d}.pt"
        torch.save(self._records, path)
        self._records, self._calls = {}, {}
        self.pass_index += 1
        return path

    def detach(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    @staticmethod
    def load_pass(directory: str | Path, index: int) -> dict[str, Any]:
        return torch.load(Path(directory) / f"pass{index:05d}.pt", map_location="cpu", weights_only=False)


load_filter_fn = _load_predicate


def register_tensor_dumper(module: torch.nn.Module, out_dir: str | Path, *, prefix: str = "", patterns: tuple[str, ...] | None = None,
                           filter_fn: str | Callable[[str], bool] | None = None) -> TensorDumper:
    """A dumper hooked onto ``module``'s leaf modules in one call (``filter_fn``: a predicate or its ``"pkg.mod:func"`` spec)."""
    pred = _load_predicate(filter_fn) if isinstance(filter_fn, str) else filter_fn
    dumper = TensorDumper(out_dir, patterns=patterns, predicate=pred)
    dumper.attach(module, prefix=prefix)
    return dumper


__all__ = ["TensorDumper", "load_filter_fn", "register_tensor_dumper"]
