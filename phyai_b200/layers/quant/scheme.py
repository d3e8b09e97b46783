"""Quantisation IR: what a tensor is stored as, and which modules get which scheme.

Reference: phyai/src/phyai/layers/quant/{scheme,granularity,plan,materialize,active}.py.
"""

from __future__ import annotations

import contextlib
import contextvars
import enum
import fnmatch
import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterator, Sequence


class QDType(enum.Enum):
    BF16 = "bf16"
    FP16 = "fp16"
    FP8_E4M3 = "fp8_e4m3"
    FP8_E5M2 = "fp8_e5m2"
    NVFP4 = "nvfp4"


class Granularity(enum.Enum):
    PER_TENSOR = "per_tensor"
    PER_CHANNEL = "per_channel"
    PER_TOKEN = "per_token"
    BLOCK = "block"
    GROUP = "group"


@dataclass(frozen=True)
class TensorQuant:
    dtype: QDType
    granularity: Granularity = Granularity.PER_TENSOR
    block_shape: tuple[int, ...] | None = None   # (rows, cols) for BLOCK, (group,) for GROUP
    dynamic: bool = False                        # scales computed at run time (activations)

    def __post_init__(self) -> None:
        if self.granularity in (Granularity.BLOCK, Granularity.GROUP) and not self.block_shape:
            raise ValueError(f"{self.granularity.value} quantisation needs a block_shape")


@dataclass(frozen=True)
class QuantScheme:
    weight: TensorQuant
    activation: TensorQuant | None = None
    name: str = ""

    @property
    def spec_id(self) -> str:
        w = self.weight
        if w.dtype in (QDType.BF16, QDType.FP16):
            return w.dtype.value
        if w.dtype is QDType.NVFP4:
            return f"nvfp4_block_{(w.block_shape or (16,))[0]}"
        base = "fp8"
        if w.granularity is Granularity.BLOCK:
            r, c = w.block_shape  # type: ignore[misc]
            return f"{base}_block_{r}_{c}"
        return f"{base}_{w.granularity.value}"


FP8_BLOCK_128 = QuantScheme(
    weight=TensorQuant(QDType.FP8_E4M3, Granularity.BLOCK, (128, 128)),
    activation=TensorQuant(QDType.FP8_E4M3, Granularity.GROUP, (128,), dynamic=True), name="fp8_block_128_128")
FP8_PER_TENSOR = QuantScheme(weight=TensorQuant(QDType.FP8_E4M3, Granularity.PER_TENSOR),
                             activation=TensorQuant(QDType.FP8_E4M3, Granularity.PER_TOKEN, dynamic=True),
                             name="fp8_per_tensor")
FP8_PER_CHANNEL = QuantScheme(weight=TensorQuant(QDType.FP8_E4M3, Granularity.PER_CHANNEL),
                              activation=TensorQuant(QDType.FP8_E4M3, Granularity.PER_TOKEN, dynamic=True),
                              name="fp8_per_channel")
NVFP4_BLOCK_16 = QuantScheme(weight=TensorQuant(QDType.NVFP4, Granularity.GROUP, (16,)),
                             activation=TensorQuant(QDType.NVFP4, Granularity.GROUP, (16,), dynamic=True),
                             name="nvfp4_block_16")


@dataclass(frozen=True)
class Matcher:
    """Selects modules by exact name, glob, regex or class (any given criterion must match)."""

    name: str | None = None
    glob: str | None = None
    regex: str | None = None
    module_cls: str | type | None = None

    def matches(self, module_name: str, module_cls: type | None = None) -> bool:
        if self.name is not None and module_name != self.name:
            return False
        if self.glob is not None and not fnmatch.fnmatchcase(module_name, self.glob):
            return False
        if self.regex is not None and re.search(self.regex, module_name) is None:
            return False
        if self.module_cls is not None:
            if module_cls is None:
                return False
            want = self.module_cls if isinstance(self.module_cls, str) else self.module_cls.__name__
            if want not in {c.__name__ for c in module_cls.__mro__}:
                return False
        return True


@dataclass(frozen=True)
class Rule:
    matcher: Matcher
    scheme: QuantScheme | None      # None = leave unquantised (an "ignore" rule)


@dataclass(frozen=True)
class QuantPlan:
    """Ordered rules; the first match wins; no match falls back to ``default``."""

    rules: tuple[Rule, ...] = ()
    default: QuantScheme | None = None

    def resolve(self, module_name: str, module_cls: type | None = None) -> QuantScheme | None:
        for r in self.rules:
            if r.matcher.matches(module_name, module_cls):
                return r.scheme
        return self.default


_ACTIVE: contextvars.ContextVar[QuantPlan | None] = contextvars.ContextVar("phyai_b200_quant_plan", default=None)


def get_active_plan() -> QuantPlan | None:
    return _ACTIVE.get()


@contextlib.contextmanager
def use_quant_plan(plan: QuantPlan | None) -> Iterator[QuantPlan | None]:
    """Linears constructed inside the block resolve their scheme from ``plan``."""
    tok = _ACTIVE.set(plan)
    try:
        yield plan
    finally:
        _ACTIVE.reset(tok)


def load_quant_plan(checkpoint_dir: str | Path | None) -> QuantPlan | None:
    """Read ``quantization_config`` / ``compression_config`` from ``config.json`` or
    ``hf_quant_config.json`` and run the importers over it; ``None`` for a plain checkpoint."""
    if checkpoint_dir is None:
        return None
    from .importers import import_plan

    d = Path(checkpoint_dir)
    blobs: list[dict[str, Any]] = []
    cfg = d / "config.json"
    if cfg.is_file():
        j = json.loads(cfg.read_text())
        for k in ("quantization_config", "compression_config"):
            if isinstance(j.get(k), dict):
                blobs.append(j[k])
    mo = d / "hf_quant_config.json"
    if mo.is_file():
        blobs.append(json.loads(mo.read_text()))
    for b in blobs:
        plan = import_plan(b)
        if plan is not None:
            return plan
    return None


__all__ = ["QDType", "Granularity", "TensorQuant", "QuantScheme", "Matcher", "Rule", "QuantPlan",
           "get_active_plan", "use_quant_plan", "load_quant_plan", "FP8_BLOCK_128", "FP8_PER_TENSOR",
           "FP8_PER_CHANNEL", "NVFP4_BLOCK_16"]
