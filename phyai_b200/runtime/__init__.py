from .base import ModelRunner, Scheduler
from .cuda_graph_manager import CudaGraph, CudaGraphError, CudaGraphRegistry, capture_on_stream
from .ipc_buffer import CudaIpcBuffer, CudaIpcHandle, HostShmBuffer, HostShmHandle
from .tensor_dump import TensorDumper, load_filter_fn, load_pass, register_tensor_dumper

__all__ = ["ModelRunner", "Scheduler", "CudaGraph", "CudaGraphRegistry", "capture_on_stream", "CudaIpcBuffer", "CudaIpcHandle",
           "HostShmBuffer", "HostShmHandle", "TensorDumper", "load_pass", "CudaGraphError", "load_filter_fn", "register_tensor_dumper"]
