from .base import ModelRunner, Scheduler
from .cuda_graph_manager import CudaGraph, CudaGraphRegistry, capture_on_stream

__all__ = ["ModelRunner", "Scheduler", "CudaGraph", "CudaGraphRegistry", "capture_on_stream"]
