"""Collective vocabulary and the backend protocol.

Reference: phyai/src/phyai/parallel/backend.py:20-75.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Protocol, runtime_checkable

import torch


class Op(enum.Enum):
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"
    ALL_TO_ALL = "all_to_all"
    BROADCAST = "broadcast"
    SEND = "send"
    RECV = "recv"
    BARRIER = "barrier"


class Mode(enum.Enum):
    EAGER = "eager"
    GRAPH_CAPTURING = "graph_capturing"


@dataclass(frozen=True)
class Topology:
    """What a backend may want to know about the ranks of one mesh axis."""

    world_size: int
    axis_size: int
    same_node: bool = True
    nvlink: bool = True


@dataclass(frozen=True)
class Call:
    """One collective request as seen by backends."""

    op: Op
    axis: str
    mesh: Any
    dtype: torch.dtype
    nbytes: int
    mode: Mode
    device_type: str
    extra: tuple = ()


@runtime_checkable
class Backend(Protocol):
    name: str

    def can_handle(self, call: Call) -> bool: ...

    def supports_capture(self) -> bool: ...

    def execute(self, call: Call, *tensors: torch.Tensor, **kw: Any) -> torch.Tensor | None: ...


__all__ = ["Op", "Mode", "Topology", "Call", "Backend"]
