"""Runner and scheduler base classes (reference: phyai/src/phyai/runtime/model_runner.py:47-88,
phyai/src/phyai/runtime/schedule/base.py:26-42)."""

from __future__ import annotations

import abc
from typing import Any


class ModelRunner(abc.ABC):
    """Owns one stage of a model: its static buffers, its kernels, its CUDA graphs."""

    @abc.abstractmethod
    def setup(self) -> None: ...

    def warmup(self) -> None:
        """Run the stage once eagerly (lazy initialisation) before any capture."""

    def plan_inference(self, meta: Any) -> None:
        """Stage the shape-dependent metadata of the next ``forward`` (no-op by default)."""

    @abc.abstractmethod
    def forward(self, batch: Any) -> Any: ...

    def close(self) -> None:
        pass


class Scheduler(abc.ABC):
    """Turns one request into runner calls and returns the result."""

    @abc.abstractmethod
    def setup(self) -> None: ...

    @abc.abstractmethod
    def step(self, request: Any) -> Any: ...

    def close(self) -> None:
        pass


__all__ = ["ModelRunner", "Scheduler"]
