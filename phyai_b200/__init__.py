"""phyai_b200: a latency-first serving engine for Physical-AI models on NVIDIA B200.

``import phyai_b200`` stays cheap: public names resolve on first access (PEP 562).
"""

from __future__ import annotations

import importlib
from typing import Any

__version__ = "0.1.0"

_LAZY = {
    "Engine": "phyai_b200.engine", "EngineArgs": "phyai_b200.engine", "Entry": "phyai_b200.engine",
    "EntryArgs": "phyai_b200.engine",
    "EngineConfig": "phyai_b200.engine_config", "BackendConfig": "phyai_b200.engine_config",
    "DeviceConfig": "phyai_b200.engine_config", "ParallelConfig": "phyai_b200.engine_config",
    "RuntimeConfig": "phyai_b200.engine_config", "get_engine_config": "phyai_b200.engine_config",
    "set_engine_config": "phyai_b200.engine_config", "init_engine_config": "phyai_b200.engine_config",
    "envs": "phyai_b200.env",
}


def __getattr__(name: str) -> Any:
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'phyai_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(mod), name)
    globals()[name] = value
    return value


def __dir__() -> list[str]:
    return sorted(list(globals()) + list(_LAZY))


__all__ = list(_LAZY) + ["__version__"]
