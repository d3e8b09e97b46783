"""Typed ``PHYAI_*`` environment variables.

One :class:`EnvField` per variable: name, parser, default. ``envs.X.get()`` parses
on every call (tests monkeypatch the environment), ``envs.X.is_set()`` tells an
unset variable from one set to its default. The names match the reference's
catalogue (phyai/src/phyai/env.py:137-188) so deployment scripts carry over.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Generic, TypeVar

import torch

T = TypeVar("T")

_TRUE = {"1", "true", "yes", "on", "y", "t"}
_FALSE = {"0", "false", "no", "off", "n", "f", ""}
_DTYPES = {
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
    "fp16": torch.float16, "float16": torch.float16, "half": torch.float16,
    "fp32": torch.float32, "float32": torch.float32, "float": torch.float32,
}


def parse_bool(s: str) -> bool:
    v = s.strip().lower()
    if v in _TRUE:
        return True
    if v in _FALSE:
        return False
    raise ValueError(f"cannot read {s!r} as a boolean")


def parse_dtype(s: str) -> torch.dtype:
    key = s.strip().lower().removeprefix("torch.")
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {s!r}; choose one of {sorted(_DTYPES)}")
    return _DTYPES[key]


def parse_regex_list(s: str) -> tuple[str, ...]:
    """A JSON array of regex strings, or one bare pattern."""
    text = s.strip()
    if not text.startswith("["):
        return (text,)
    items = json.loads(text)
    if not isinstance(items, list) or not all(isinstance(i, str) for i in items):
        raise ValueError(f"expected a JSON array of strings, got {s!r}")
    return tuple(items)


@dataclass(frozen=True)
class EnvField(Generic[T]):
    name: str
    default: Any
    parser: Callable[[str], T]

    def is_set(self) -> bool:
        return self.name in os.environ

    def raw(self) -> str | None:
        return os.environ.get(self.name)

    def get(self) -> T | Any:
        raw = os.environ.get(self.name)
        if raw is None:
            return self.default
        try:
            return self.parser(raw)
        except Exception as e:
            raise ValueError(f"environment variable {self.name}={raw!r}: {e}") from e


class envs:
    """Every ``PHYAI_*`` variable the engine reads."""

    # backend / kernel selection
    PHYAI_ATTN_BACKEND = EnvField("PHYAI_ATTN_BACKEND", None, str)
    PHYAI_NORM_BACKEND = EnvField("PHYAI_NORM_BACKEND", None, str)
    PHYAI_LINEAR_BACKEND = EnvField("PHYAI_LINEAR_BACKEND", None, str)
    PHYAI_VGPU_BACKEND = EnvField("PHYAI_VGPU_BACKEND", None, str)
    # device / dtype
    PHYAI_DEVICE = EnvField("PHYAI_DEVICE", None, str)
    PHYAI_PARAMS_DTYPE = EnvField("PHYAI_PARAMS_DTYPE", None, parse_dtype)
    # runtime
    PHYAI_USE_CUDA_GRAPH = EnvField("PHYAI_USE_CUDA_GRAPH", None, parse_bool)
    # parallel layout
    PHYAI_WORLD_SIZE = EnvField("PHYAI_WORLD_SIZE", None, int)
    PHYAI_DP_SIZE = EnvField("PHYAI_DP_SIZE", None, int)
    PHYAI_CFG_SIZE = EnvField("PHYAI_CFG_SIZE", None, int)
    PHYAI_EP_SIZE = EnvField("PHYAI_EP_SIZE", None, int)
    PHYAI_SP_SIZE = EnvField("PHYAI_SP_SIZE", None, int)
    PHYAI_CP_SIZE = EnvField("PHYAI_CP_SIZE", None, int)
    PHYAI_TP_SIZE = EnvField("PHYAI_TP_SIZE", None, int)
    # low-level tuning (the two workspace knobs are accepted for compatibility; the
    # attention kernels here need no workspace)
    PHYAI_FLASHINFER_WORKSPACE_BYTES = EnvField("PHYAI_FLASHINFER_WORKSPACE_BYTES", None, int)
    PHYAI_FLASHINFER_PREFILL_BACKEND = EnvField("PHYAI_FLASHINFER_PREFILL_BACKEND", None, str)
    PHYAI_FORCE_LINEAR_KERNEL = EnvField("PHYAI_FORCE_LINEAR_KERNEL", None, str)
    # collectives
    PHYAI_FORCE_BACKEND = EnvField("PHYAI_FORCE_BACKEND", None, str)
    PHYAI_NCCL_SO_PATH = EnvField("PHYAI_NCCL_SO_PATH", None, str)
    PHYAI_COMM_TIMEOUT_S = EnvField("PHYAI_COMM_TIMEOUT_S", 60.0, float)
    PHYAI_HEARTBEAT_S = EnvField("PHYAI_HEARTBEAT_S", 0.0, float)
    PHYAI_USE_PYNCCL = EnvField("PHYAI_USE_PYNCCL", False, parse_bool)   # register the ctypes NCCL backend ahead of torch's
    PHYAI_PEER_COMM = EnvField("PHYAI_PEER_COMM", True, parse_bool)    # fused peer-memory collectives (0: NCCL only)
    PHYAI_PEER_GUARD = EnvField("PHYAI_PEER_GUARD", False, parse_bool)  # 1: guard bands around every symmetric-heap allocation (PeerGroup.check_guards reads them back)
    PHYAI_PEER_HEAP_MB = EnvField("PHYAI_PEER_HEAP_MB", 0, int)          # symmetric heap size override
    # kernel routing (read by the native library itself on first use: listed here so they show up with the rest)
    PHYAI_GEMM_PERSIST = EnvField("PHYAI_GEMM_PERSIST", True, parse_bool)        # 0: one tile per CTA for large GEMMs too
    PHYAI_GEMM_PERSIST_COMM = EnvField("PHYAI_GEMM_PERSIST_COMM", True, parse_bool)  # 0: peer modes stay off the persistent kernel
    PHYAI_COMM_FUSED_TAIL = EnvField("PHYAI_COMM_FUSED_TAIL", True, parse_bool)  # 0: row-parallel products of few rows as two launches (push GEMM, reduce) instead of one
    PHYAI_GEMM_PERSIST_PUSH_WORLD = EnvField("PHYAI_GEMM_PERSIST_PUSH_WORLD", 2, int)  # largest group whose push / scatter GEMMs run persistent
    PHYAI_GEMM_2CTA = EnvField("PHYAI_GEMM_2CTA", None, parse_bool)             # CTA-pair (cta_group::2) GEMM: 1 every large plain problem, 0 never, unset: very wide / long-K shapes only
    PHYAI_NORM_TMA = EnvField("PHYAI_NORM_TMA", False, parse_bool)              # 1: many-row norms through bulk copies into shared memory
    PHYAI_ATTN_POLY = EnvField("PHYAI_ATTN_POLY", 0, int)                       # pipelined attention: 0..2 of every 4 exponentials on the FMA pipe
    PHYAI_PI05_EXPERT_SPLITS = EnvField("PHYAI_PI05_EXPERT_SPLITS", None, int)  # KV split of the expert's joint attention (default 8)
    PHYAI_PI05_PREFIX_SPLITS = EnvField("PHYAI_PI05_PREFIX_SPLITS", None, int)  # KV split of the prefix attention (default: 2 at batch 1, 1 above; the tensor-parallel plan takes 4 from 896 prefix rows)
    PHYAI_PI05_OVERLAP = EnvField("PHYAI_PI05_OVERLAP", True, parse_bool)       # 0: no second stream (first Euler step after the prefix)
    PHYAI_COSMOS3_FP8 = EnvField("PHYAI_COSMOS3_FP8", False, parse_bool)        # 1: Cosmos3 generation tower in block-scaled fp8
    PHYAI_COSMOS3_NVFP4 = EnvField("PHYAI_COSMOS3_NVFP4", False, parse_bool)    # 1: Cosmos3 generation tower in NVFP4 (one GPU; needs the _blockscaled module)
    PHYAI_COSMOS3_FUSED_SAMPLER = EnvField("PHYAI_COSMOS3_FUSED_SAMPLER", True, parse_bool)  # 0: UniPC update as host-issued tensor ops
    PHYAI_COSMOS3_GRAPH = EnvField("PHYAI_COSMOS3_GRAPH", True, parse_bool)    # 0: every launch of a Cosmos3 denoise step from the host (default: one CUDA graph per request on a single GPU)
    PHYAI_PI05_FP8 = EnvField("PHYAI_PI05_FP8", False, parse_bool)              # 1: Pi0.5 / Pi0 prefix decoder and action expert in block-scaled fp8
    PHYAI_PI05_TP_SCATTER_ROWS = EnvField("PHYAI_PI05_TP_SCATTER_ROWS", 512, int)  # prefix rows from which a 4+ rank Pi0.5 TP group reduce-scatters instead of pushing whole partials
    PHYAI_PI05_EXPERT_KERNEL = EnvField("PHYAI_PI05_EXPERT_KERNEL", False, parse_bool)  # 1: Euler loop as one persistent kernel (measured slower than launch by launch at batch 1)
    PHYAI_CHECK_KERNEL_STATUS = EnvField("PHYAI_CHECK_KERNEL_STATUS", False, parse_bool)  # 1: read the device status word after every Engine.step even without peer groups
    # debug / tensor dump
    PHYAI_DEBUG_TENSOR_DUMP_DIR = EnvField("PHYAI_DEBUG_TENSOR_DUMP_DIR", None, str)
    PHYAI_DEBUG_TENSOR_DUMP_FILTER = EnvField("PHYAI_DEBUG_TENSOR_DUMP_FILTER", None, parse_regex_list)
    PHYAI_DEBUG_TENSOR_DUMP_FILTER_FN = EnvField("PHYAI_DEBUG_TENSOR_DUMP_FILTER_FN", None, str)

    @classmethod
    def fields(cls) -> dict[str, EnvField]:
        return {k: v for k, v in vars(cls).items() if isinstance(v, EnvField)}


__all__ = ["EnvField", "envs", "parse_bool", "parse_dtype", "parse_regex_list"]
