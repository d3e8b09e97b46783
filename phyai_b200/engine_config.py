"""Layered, frozen engine configuration.

``EngineConfig`` = ``backends`` + ``device`` + ``parallel`` + ``runtime``; every
level is a frozen dataclass validated on construction. Precedence when the
engine resolves its config: explicit field > ``PHYAI_*`` environment variable >
model recommendation > auto default. A process-wide singleton is installed by
the engine and read by constructors that were not handed explicit values
(:func:`resolve_engine_defaults`).

Same public surface as the reference (phyai/src/phyai/engine_config.py:79-632);
the backend vocabulary differs because the compute path here is this
repository's own sm_100a kernels: ``"b200"`` (CUDA kernels of ``phyai_b200._C``)
and ``"torch"`` (plain PyTorch, used on CPU). ``"auto"`` picks by device. The
reference's names (``flashinfer``, ``phyai-kernel``, ``sdpa``, ``eager``) are
accepted as aliases so existing configs load.
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any

import torch

from .env import envs

ATTN_BACKENDS = ("auto", "b200", "torch")
NORM_BACKENDS = ("auto", "b200", "torch")
LINEAR_BACKENDS = (None, "auto", "b200", "torch")
VGPU_BACKENDS = (None, "auto", "torch", "driver")
_ALIASES = {
    "flashinfer": "b200", "phyai-kernel": "b200", "triton": "b200", "cuda": "b200",
    "sdpa": "torch", "eager": "torch",
}
PREFILL_BACKENDS = (None, "auto", "fa2", "fa3", "cudnn", "trtllm-gen", "b200")
AXES = ("dp", "cfg", "ep", "sp", "cp", "tp")


def _canon(name: str | None) -> str | None:
    if name is None:
        return None
    return _ALIASES.get(name, name)


@dataclass(frozen=True)
class BackendConfig:
    """Which implementation family each op class uses."""

    attn: str = "auto"
    norm: str = "auto"
    linear: str | None = None
    vgpu: str | None = None

    def __post_init__(self) -> None:
        for f, allowed in (("attn", ATTN_BACKENDS), ("norm", NORM_BACKENDS),
                           ("linear", LINEAR_BACKENDS), ("vgpu", VGPU_BACKENDS)):
            v = _canon(getattr(self, f))
            if v not in allowed:
                raise ValueError(f"backends.{f}={getattr(self, f)!r} is not one of {allowed}")
            object.__setattr__(self, f, v)


@dataclass(frozen=True)
class DeviceConfig:
    target: str = "cuda"
    params_dtype: torch.dtype = field(default=torch.bfloat16)

    def __post_init__(self) -> None:
        kind = str(self.target).split(":")[0]
        if kind not in ("cuda", "cpu"):
            raise ValueError(f"device.target={self.target!r}: expected 'cuda[:i]' or 'cpu'")
        if self.params_dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise ValueError(f"device.params_dtype={self.params_dtype} is not a floating dtype the engine serves")


@dataclass(frozen=True)
class ParallelConfig:
    """Six-axis layout, ``tp`` innermost, ``cfg`` just outside it."""

    world_size: int = 1
    dp_size: int = 1
    cfg_size: int = 1
    ep_size: int = 1
    sp_size: int = 1
    cp_size: int = 1
    tp_size: int = 1

    def __post_init__(self) -> None:
        for ax in AXES:
            v = getattr(self, f"{ax}_size")
            if not isinstance(v, int) or v < 1:
                raise ValueError(f"parallel.{ax}_size must be a positive int, got {v!r}")
        if self.world_size < 1:
            raise ValueError(f"parallel.world_size must be positive, got {self.world_size}")
        prod = math.prod(self.layout)
        if prod != self.world_size:
            raise ValueError(
                f"parallel: dp*cfg*ep*sp*cp*tp = {prod} does not equal world_size={self.world_size}")

    @property
    def layout(self) -> tuple[int, ...]:
        return tuple(getattr(self, f"{ax}_size") for ax in AXES)


@dataclass(frozen=True)
class RuntimeConfig:
    use_cuda_graph: bool = True
    flashinfer_workspace_bytes: int = 128 * 1024 * 1024
    flashinfer_prefill_backend: str | None = None
    force_linear_kernel: str | None = None
    debug_tensor_dump_dir: str | None = None
    debug_tensor_dump_filter: tuple[str, ...] | None = None
    debug_tensor_dump_filter_fn: str | None = None

    def __post_init__(self) -> None:
        if self.flashinfer_workspace_bytes <= 0:
            raise ValueError("runtime.flashinfer_workspace_bytes must be positive")
        if self.flashinfer_prefill_backend not in PREFILL_BACKENDS:
            raise ValueError(
                f"runtime.flashinfer_prefill_backend={self.flashinfer_prefill_backend!r} not in {PREFILL_BACKENDS}")
        if self.debug_tensor_dump_filter is not None and self.debug_tensor_dump_filter_fn is not None:
            raise ValueError("runtime: debug_tensor_dump_filter and debug_tensor_dump_filter_fn are mutually exclusive")
        if self.debug_tensor_dump_filter is not None:
            object.__setattr__(self, "debug_tensor_dump_filter", tuple(self.debug_tensor_dump_filter))


@dataclass(frozen=True)
class EngineConfig:
    backends: BackendConfig = field(default_factory=BackendConfig)
    device: DeviceConfig = field(default_factory=DeviceConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)

    # ------------------------------------------------------------ constructors
    @classmethod
    def auto(cls) -> "EngineConfig":
        """Defaults for this machine: CUDA + bf16 when a GPU is visible, else CPU + fp32."""
        if torch.cuda.is_available():
            return cls()
        return cls(device=DeviceConfig(target="cpu", params_dtype=torch.float32),
                   runtime=RuntimeConfig(use_cuda_graph=False))

    @classmethod
    def from_env(cls, base: "EngineConfig | None" = None, *, explicit: "EngineConfig | None" = None) -> "EngineConfig":
        """Overlay ``PHYAI_*`` variables on ``base``.

        Fields of ``explicit`` that differ from the dataclass defaults are treated as
        set by the caller and win over the environment.
        """
        cfg = base if base is not None else cls.auto()
        pinned = _non_default_fields(explicit) if explicit is not None else set()

        def pick(section: str, name: str, envf, current):
            if (section, name) in pinned or not envf.is_set():
                return current
            return envf.get()

        b, d, p, r = cfg.backends, cfg.device, cfg.parallel, cfg.runtime
        backends = BackendConfig(
            attn=pick("backends", "attn", envs.PHYAI_ATTN_BACKEND, b.attn),
            norm=pick("backends", "norm", envs.PHYAI_NORM_BACKEND, b.norm),
            linear=pick("backends", "linear", envs.PHYAI_LINEAR_BACKEND, b.linear),
            vgpu=pick("backends", "vgpu", envs.PHYAI_VGPU_BACKEND, b.vgpu),
        )
        device = DeviceConfig(
            target=pick("device", "target", envs.PHYAI_DEVICE, d.target),
            params_dtype=pick("device", "params_dtype", envs.PHYAI_PARAMS_DTYPE, d.params_dtype),
        )
        sizes = {f"{ax}_size": pick("parallel", f"{ax}_size", getattr(envs, f"PHYAI_{ax.upper()}_SIZE"),
                                    getattr(p, f"{ax}_size")) for ax in AXES}
        ws = pick("parallel", "world_size", envs.PHYAI_WORLD_SIZE, p.world_size)
        if not envs.PHYAI_WORLD_SIZE.is_set() and ("parallel", "world_size") not in pinned:
            ws = math.prod(sizes.values()) if any(
                getattr(envs, f"PHYAI_{ax.upper()}_SIZE").is_set() for ax in AXES) else ws
        parallel = ParallelConfig(world_size=ws, **sizes)
        runtime = RuntimeConfig(
            use_cuda_graph=pick("runtime", "use_cuda_graph", envs.PHYAI_USE_CUDA_GRAPH, r.use_cuda_graph),
            flashinfer_workspace_bytes=pick("runtime", "flashinfer_workspace_bytes",
                                            envs.PHYAI_FLASHINFER_WORKSPACE_BYTES, r.flashinfer_workspace_bytes),
            flashinfer_prefill_backend=pick("runtime", "flashinfer_prefill_backend",
                                            envs.PHYAI_FLASHINFER_PREFILL_BACKEND, r.flashinfer_prefill_backend),
            force_linear_kernel=pick("runtime", "force_linear_kernel", envs.PHYAI_FORCE_LINEAR_KERNEL,
                                     r.force_linear_kernel),
            debug_tensor_dump_dir=pick("runtime", "debug_tensor_dump_dir", envs.PHYAI_DEBUG_TENSOR_DUMP_DIR,
                                       r.debug_tensor_dump_dir),
            debug_tensor_dump_filter=pick("runtime", "debug_tensor_dump_filter",
                                          envs.PHYAI_DEBUG_TENSOR_DUMP_FILTER, r.debug_tensor_dump_filter),
            debug_tensor_dump_filter_fn=pick("runtime", "debug_tensor_dump_filter_fn",
                                             envs.PHYAI_DEBUG_TENSOR_DUMP_FILTER_FN, r.debug_tensor_dump_filter_fn),
        )
        return cls(backends=backends, device=device, parallel=parallel, runtime=runtime)

    def replace(self, **sections: Any) -> "EngineConfig":
        """``cfg.replace(runtime={"use_cuda_graph": False})`` or ``replace(runtime=RuntimeConfig(...))``."""
        new: dict[str, Any] = {}
        for name, val in sections.items():
            if name not in ("backends", "device", "parallel", "runtime"):
                raise TypeError(f"EngineConfig has no section {name!r}")
            cur = getattr(self, name)
            new[name] = dataclasses.replace(cur, **val) if isinstance(val, dict) else val
        return dataclasses.replace(self, **new)

    # ------------------------------------------------------- resolved choices
    def resolved_backend(self, kind: str) -> str:
        """'b200' or 'torch' for ``kind`` in attn / norm / linear after resolving ``auto``."""
        v = getattr(self.backends, kind)
        if v in (None, "auto"):
            return "b200" if str(self.device.target).startswith("cuda") else "torch"
        return v


def _non_default_fields(cfg: EngineConfig) -> set[tuple[str, str]]:
    out: set[tuple[str, str]] = set()
    default = EngineConfig()
    for sec in ("backends", "device", "parallel", "runtime"):
        a, b = getattr(cfg, sec), getattr(default, sec)
        for f in dataclasses.fields(a):
            if getattr(a, f.name) != getattr(b, f.name):
                out.add((sec, f.name))
    return out


# ------------------------------------------------------------------ singleton
_CURRENT: EngineConfig | None = None


def get_engine_config() -> EngineConfig:
    """The installed config; an auto default when the engine has not installed one."""
    global _CURRENT
    if _CURRENT is None:
        _CURRENT = EngineConfig.auto()
    return _CURRENT


def set_engine_config(cfg: EngineConfig) -> None:
    global _CURRENT
    if not isinstance(cfg, EngineConfig):
        raise TypeError(f"expected EngineConfig, got {type(cfg).__name__}")
    _CURRENT = cfg


def init_engine_config(cfg: EngineConfig | None = None) -> EngineConfig:
    """Install ``cfg`` (or env-resolved defaults) and return it."""
    resolved = cfg if cfg is not None else EngineConfig.from_env()
    set_engine_config(resolved)
    return resolved


def reset_engine_config() -> None:
    """Test hook: forget the installed config."""
    global _CURRENT
    _CURRENT = None


def resolve_engine_defaults(params_dtype: torch.dtype | None = None, attn_backend: str | None = None,
                            norm_backend: str | None = None) -> tuple[torch.dtype, str, str]:
    """Fill constructor arguments left at ``None`` from the installed config."""
    cfg = get_engine_config()
    return (
        params_dtype if params_dtype is not None else cfg.device.params_dtype,
        _canon(attn_backend) if attn_backend not in (None, "auto") else cfg.resolved_backend("attn"),
        _canon(norm_backend) if norm_backend not in (None, "auto") else cfg.resolved_backend("norm"),
    )


__all__ = [
    "AXES", "BackendConfig", "DeviceConfig", "ParallelConfig", "RuntimeConfig", "EngineConfig",
    "get_engine_config", "set_engine_config", "init_engine_config", "reset_engine_config",
    "resolve_engine_defaults",
]
