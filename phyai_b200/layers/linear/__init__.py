from .kernels import (B200Kernel, Dispatcher, KernelProbe, LinearKernel, Registry, TorchKernel,
                      get_linear_dispatcher, init)
from .layers import (ColumnParallelLinear, LinearBase, MergedColumnParallelLinear, QKVParallelLinear,
                     ReplicatedLinear, RowParallelLinear)

__all__ = ["B200Kernel", "Dispatcher", "KernelProbe", "LinearKernel", "Registry", "TorchKernel",
           "get_linear_dispatcher", "init", "ColumnParallelLinear", "LinearBase", "MergedColumnParallelLinear",
           "QKVParallelLinear", "ReplicatedLinear", "RowParallelLinear"]
