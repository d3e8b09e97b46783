from ..quant.scheme import Granularity
from ..quant.specs import (ActivationView, AllocationRequest, Bf16Spec, Fp8Spec, LinearActivationQuant, Nvfp4Spec, WeightSpec)
from .kernels import (B200Kernel, DefaultPolicy, Dispatcher, ForcedPolicy, KernelDispatcher, KernelProbe, LinearKernel,
                      LinearKernelRegistry, Policy, Registry, TorchKernel, get_linear_dispatcher, init,
                      list_registered_linear_kernels, register_linear_kernel, supported_specs_for_sm)
from .layers import (ColumnParallelLinear, LinearBase, MergedColumnParallelLinear, QKVParallelLinear,
                     ReplicatedLinear, RowParallelLinear)

__all__ = ["ActivationView", "AllocationRequest", "Bf16Spec", "Fp8Spec", "LinearActivationQuant", "Nvfp4Spec", "WeightSpec", "Granularity",
           "DefaultPolicy", "ForcedPolicy", "Policy", "KernelDispatcher", "LinearKernelRegistry", "register_linear_kernel",
           "list_registered_linear_kernels", "supported_specs_for_sm", "B200Kernel", "Dispatcher", "KernelProbe", "LinearKernel", "Registry", "TorchKernel",
           "get_linear_dispatcher", "init", "ColumnParallelLinear", "LinearBase", "MergedColumnParallelLinear",
           "QKVParallelLinear", "ReplicatedLinear", "RowParallelLinear"]
