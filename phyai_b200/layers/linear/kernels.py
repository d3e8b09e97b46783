"""Linear kernel providers, registry and per-shape dispatcher.

A kernel declares the spec ids it can run, the minimum SM it needs and whether it
is CUDA-graph capturable. The registry prefers kernels per ``(spec_id, regime)``
where the regime is ``"decode"`` for M <= 4 and ``"prefill"`` otherwise; the
dispatcher caches the choice per M bucket. SM support is checked when a kernel is
selected, not when a layer is built, so a config can be constructed anywhere.

Reference: phyai/src/phyai/layers/linear/{backend,registry,dispatch,__init__}.py and
backends/{flashinfer,torch}.py. The CUDA provider here is this repository's tcgen05
GEMM (``phyai_b200.ops.gemm``) instead of FlashInfer / cuBLAS.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Protocol

import torch
import torch.nn.functional as F

from ... import ops
from ...engine_config import get_engine_config
from ...utils.cuda import sm_arch
from ..quant.scheme import Granularity


@dataclass(frozen=True)
class KernelProbe:
    spec_id: str
    M: int
    N: int
    K: int
    in_dtype: torch.dtype
    out_dtype: torch.dtype
    device_type: str = "cuda"
    capturing: bool = False

    @property
    def regime(self) -> str:
        return "decode" if self.M <= 4 else "prefill"


class LinearKernel(Protocol):
    name: str
    specs: frozenset[str]
    min_sm: int
    device_types: frozenset[str]

    def supports_capture(self) -> bool: ...

    def apply(self, layer, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor: ...


class TorchKernel:
    """Plain PyTorch: ``F.linear`` for bf16/fp16/fp32, dequantise + matmul for quantised specs."""

    name = "torch"
    specs = frozenset({"bf16", "fp16", "fp8_per_tensor", "fp8_per_channel", "fp8_block_128_128", "nvfp4_block_16"})
    min_sm = 0
    device_types = frozenset({"cpu", "cuda"})

    def supports_capture(self) -> bool:
        return True

    def apply(self, layer, x, bias):
        if layer.spec.spec_id in ("bf16", "fp16"):
            return F.linear(x, layer.weight, bias)
        return layer.spec.reference_apply(layer, x, bias)


class B200Kernel:
    """tcgen05 GEMM with fused bias; fp8 specs quantise the activation with the CUDA quant kernel."""

    name = "b200"
    specs = frozenset({"bf16", "fp8_per_tensor", "fp8_per_channel", "fp8_block_128_128", "nvfp4_block_16"})
    min_sm = 100
    device_types = frozenset({"cuda"})

    def supports_capture(self) -> bool:
        return True

    def apply(self, layer, x, bias):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        spec = layer.spec
        if spec.spec_id == "bf16":
            w = layer.weight
            if x2.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x2.shape[1] % 8 or w.shape[0] % 8:
                # fp32 / fp16 operands or odd widths (timestep embedders, action heads): the CUDA-core kernel
                b = bias if bias is None or bias.dtype == w.dtype else bias.to(w.dtype)
                y = ops.linear_simt(x2, w, b)
            else:
                y = ops.gemm(x2, w, bias=bias)
        elif spec.spec_id == "nvfp4_block_16":
            from ...ops import nvfp4

            if not nvfp4.available() or x2.shape[1] % 32 or layer.weight.shape[0] % 8:
                return spec.reference_apply(layer, x, bias)     # the block-scaled GEMM module is not built here
            y = nvfp4.linear(x2.to(torch.bfloat16), layer, bias).to(x.dtype)
        elif spec.granularity is Granularity.BLOCK:
            from ...ops import fp8_block

            q, s = ops.quant_fp8(x2.to(torch.bfloat16), 128)
            y = fp8_block.gemm_fp8_block(q, s, layer.weight, layer.weight_scale, bias=bias)
        else:
            q, s = ops.quant_fp8(x2.to(torch.bfloat16), 0)
            ws = layer.weight_scale
            if ws.numel() == 1:
                ws = ws.expand(layer.weight.shape[0]).contiguous()
            y = ops.gemm(q, layer.weight, a_scale=s, w_scale=ws, bias=bias)
        return y.reshape(*lead, -1)


class Registry:
    def __init__(self) -> None:
        self._kernels: list[LinearKernel] = []
        self._prefer: dict[tuple[str, str], list[str]] = {}

    def register(self, kernel: LinearKernel, *, prefer_for: Iterable[tuple[str, str]] = ()) -> None:
        if any(k.name == kernel.name for k in self._kernels):
            raise ValueError(f"linear kernel {kernel.name!r} already registered")
        self._kernels.append(kernel)
        for key in prefer_for:
            self._prefer.setdefault(key, []).append(kernel.name)

    def names(self) -> list[str]:
        return [k.name for k in self._kernels]

    def candidates(self, probe: KernelProbe, sm: int) -> list[LinearKernel]:
        ok = [k for k in self._kernels
              if probe.spec_id in k.specs and probe.device_type in k.device_types
              and (probe.device_type != "cuda" or sm >= k.min_sm)
              and (not probe.capturing or k.supports_capture())]
        pref = self._prefer.get((probe.spec_id, probe.regime), [])
        ok.sort(key=lambda k: pref.index(k.name) if k.name in pref else len(pref))
        return ok

    def validate(self) -> None:
        if not self._kernels:
            raise RuntimeError("no linear kernel registered")

    def supported_specs_for_sm(self, sm: int, device_type: str = "cuda") -> set[str]:
        out: set[str] = set()
        for k in self._kernels:
            if device_type in k.device_types and (device_type != "cuda" or sm >= k.min_sm):
                out |= set(k.specs)
        return out


class DefaultPolicy:
    """The first candidate: kernels preferred for the probe's (spec, regime), then registration order."""

    def choose(self, probe: KernelProbe, candidates: list[LinearKernel]) -> LinearKernel | None:
        return candidates[0] if candidates else None


class ForcedPolicy:
    """Only the named kernel (``RuntimeConfig.force_linear_kernel`` / ``PHYAI_FORCE_LINEAR_KERNEL``)."""

    def __init__(self, name: str) -> None:
        self.name = name

    def choose(self, probe: KernelProbe, candidates: list[LinearKernel]) -> LinearKernel | None:
        return next((k for k in candidates if k.name == self.name), None)


Policy = DefaultPolicy | ForcedPolicy

# kernel classes declared by ``register_linear_kernel`` (out-of-tree providers): instantiated by ``init`` behind the built-in ones
_DECLARED: list[tuple[type, frozenset[tuple[str, str]]]] = []


def register_linear_kernel(*, prefer_for: Iterable[tuple[str, str]] | None = None):
    """Class decorator: declare a :class:`LinearKernel` for the next ``init``. The class is not instantiated here, so
    importing a provider module has no side effects; ``prefer_for`` lists the ``(spec_id, regime)`` pairs it should win.
    Reference: phyai/src/phyai/layers/linear/registry.py:34-58."""
    def deco(cls: type) -> type:
        if not any(c is cls for c, _ in _DECLARED):
            _DECLARED.append((cls, frozenset(prefer_for or ())))
        return cls
    return deco


def list_registered_linear_kernels() -> list[tuple[type, frozenset[tuple[str, str]]]]:
    return list(_DECLARED)


def supported_specs_for_sm(sm: int, device_type: str = "cuda") -> list[str]:
    """Spec ids some kernel of the installed registry can run on this SM (0 with ``device_type="cpu"``: the CPU)."""
    return sorted(get_linear_dispatcher().registry.supported_specs_for_sm(sm, device_type))


class Dispatcher:
    def __init__(self, registry: Registry, forced: str | None = None, *, policy: "Policy | None" = None) -> None:
        self.registry = registry
        self.forced = forced if policy is None else getattr(policy, "name", None)
        self.policy = policy if policy is not None else (ForcedPolicy(forced) if forced is not None else DefaultPolicy())
        self._cache: dict[tuple, LinearKernel] = {}

    def select(self, *, spec_id: str, M: int, N: int, K: int, in_dtype: torch.dtype, out_dtype: torch.dtype,
               device_type: str = "cuda", capturing: bool = False) -> LinearKernel:
        key = (spec_id, max(M, 1).bit_length(), N, K, in_dtype, out_dtype, device_type, capturing)
        hit = self._cache.get(key)
        if hit is not None:
            return hit
        probe = KernelProbe(spec_id, M, N, K, in_dtype, out_dtype, device_type, capturing)
        sm = sm_arch() if device_type == "cuda" else 0
        cands = self.registry.candidates(probe, sm)
        chosen = self.policy.choose(probe, cands)
        if chosen is None:
            raise RuntimeError(
                f"no linear kernel for spec {spec_id!r} on {device_type} sm_{sm} (M={M}, N={N}, K={K}, "
                f"regime={probe.regime}, forced={self.forced!r}); registered: {self.registry.names()}")
        self._cache[key] = chosen
        return chosen


_DISPATCHER: Dispatcher | None = None


def init(force: str | None = None) -> Dispatcher:
    """Register the kernels for this process and install the dispatcher."""
    global _DISPATCHER
    cfg = get_engine_config()
    reg = Registry()
    b200_pref = [(s, r) for s in B200Kernel.specs for r in ("decode", "prefill")]
    reg.register(B200Kernel(), prefer_for=b200_pref)
    reg.register(TorchKernel())
    for cls, pref in _DECLARED:
        reg.register(cls(), prefer_for=pref)
    reg.validate()
    forced = force or cfg.runtime.force_linear_kernel or (
        cfg.backends.linear if cfg.backends.linear not in (None, "auto") else None)
    _DISPATCHER = Dispatcher(reg, forced)
    return _DISPATCHER


def get_linear_dispatcher() -> Dispatcher:
    if _DISPATCHER is None:
        return init()
    return _DISPATCHER


def _reset_for_test() -> None:
    global _DISPATCHER
    _DISPATCHER = None


KernelDispatcher, LinearKernelRegistry = Dispatcher, Registry

__all__ = ["KernelProbe", "LinearKernel", "TorchKernel", "B200Kernel", "Registry", "Dispatcher", "KernelDispatcher", "LinearKernelRegistry",
           "DefaultPolicy", "ForcedPolicy", "Policy", "register_linear_kernel", "list_registered_linear_kernels", "supported_specs_for_sm",
           "init", "get_linear_dispatcher"]
