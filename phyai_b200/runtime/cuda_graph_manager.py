"""Static-shape CUDA graphs.

``CudaGraph.capture(fn, example_inputs)`` copies the example inputs into static
buffers, runs ``fn`` a few times on a side stream (lazy initialisation, tensor-map
caches, communicator warm-up all happen here), then records one more run inside
``torch.cuda.graph`` with the communication layer in capture mode. ``replay(inputs)``
copies new values into the static buffers and launches the graph; the returned
tensors alias static memory. Reference: phyai/src/phyai/runtime/cuda_graph_manager.py:53-324.
"""

from __future__ import annotations

import contextlib
from typing import Any, Callable, Mapping

import torch

from ..parallel import state as pstate

_CAPTURE_STREAM: "torch.cuda.Stream | None" = None


@contextlib.contextmanager
def capture_on_stream(stream: "torch.cuda.Stream"):
    """Captures started inside the block record on ``stream`` (e.g. an SM-partition stream)."""
    global _CAPTURE_STREAM
    prev, _CAPTURE_STREAM = _CAPTURE_STREAM, stream
    try:
        yield
    finally:
        _CAPTURE_STREAM = prev


class CudaGraphError(RuntimeError):
    """Misuse of a graph object: captured twice, replayed before capture, an input of another shape."""


class CudaGraph:
    def __init__(self, name: str = "graph", warmup_iters: int = 3, *, num_warmup_iters: int | None = None, mempool=None) -> None:
        self.name, self.warmup_iters = name, (warmup_iters if num_warmup_iters is None else int(num_warmup_iters))
        self.mempool = mempool                  # memory pool captures use unless ``capture(pool=...)`` names another
        self.graph: torch.cuda.CUDAGraph | None = None
        self.static_inputs: dict[str, torch.Tensor] = {}
        self.static_output: Any = None
        self.replays = 0

    @property
    def captured(self) -> bool:
        return self.graph is not None

    def capture(self, fn: Callable[..., Any], example_inputs: Mapping[str, torch.Tensor], *, pool=None) -> Any:
        if self.captured:
            raise CudaGraphError(f"CudaGraph {self.name!r} is already captured")
        self.static_inputs = {k: v.clone() for k, v in example_inputs.items()}
        side = _CAPTURE_STREAM or torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(self.warmup_iters):
                fn(**self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.no_grad(), pstate.graph_capture(), torch.cuda.graph(g, pool=pool if pool is not None else self.mempool, stream=_CAPTURE_STREAM):
            self.static_output = fn(**self.static_inputs)
        self.graph = g
        return self.static_output

    def replay(self, inputs: Mapping[str, torch.Tensor] | None = None) -> Any:
        if self.graph is None:
            raise CudaGraphError(f"CudaGraph {self.name!r} replayed before capture")
        if inputs:
            for k, v in inputs.items():
                dst = self.static_inputs[k]
                if v.shape != dst.shape:
                    raise ValueError(f"graph {self.name!r}: input {k!r} has shape {tuple(v.shape)}, captured {tuple(dst.shape)}")
                if v.data_ptr() != dst.data_ptr():
                    dst.copy_(v, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_output

    def input_buffer(self, name: str) -> torch.Tensor:
        """The static tensor the captured graph reads input ``name`` from."""
        if name not in self.static_inputs:
            raise KeyError(f"graph {self.name!r} has no input {name!r}; inputs: {sorted(self.static_inputs)}")
        return self.static_inputs[name]

    @property
    def input_buffers(self) -> dict[str, torch.Tensor]:
        return dict(self.static_inputs)

    def reset(self) -> None:
        self.graph = None
        self.static_inputs = {}
        self.static_output = None


class CudaGraphRegistry:
    """Named graphs of one runner (e.g. one per prefix-length bucket)."""

    def __init__(self) -> None:
        self._graphs: dict[Any, CudaGraph] = {}

    def get_or_create(self, key: Any, **kw) -> CudaGraph:
        if key not in self._graphs:
            self._graphs[key] = CudaGraph(name=str(key), **kw)
        return self._graphs[key]

    def register(self, key: Any, graph: CudaGraph) -> CudaGraph:
        if key in self._graphs and self._graphs[key] is not graph:
            raise CudaGraphError(f"a graph is already registered under {key!r}")
        self._graphs[key] = graph
        return graph

    def deregister(self, key: Any) -> CudaGraph | None:
        g = self._graphs.pop(key, None)
        if g is not None:
            g.reset()
        return g

    def get(self, key: Any, default: CudaGraph | None = None) -> CudaGraph | None:
        return self._graphs.get(key, default)

    def has(self, key: Any) -> bool:
        return key in self._graphs

    def __contains__(self, key: Any) -> bool:
        return key in self._graphs

    def __getitem__(self, key: Any) -> CudaGraph:
        return self._graphs[key]

    def keys(self):
        return self._graphs.keys()

    def total_replays(self) -> int:
        return sum(g.replays for g in self._graphs.values())

    def clear(self) -> None:
        for g in self._graphs.values():
            g.reset()
        self._graphs.clear()


__all__ = ["CudaGraph", "CudaGraphRegistry", "capture_on_stream"]
