from .importers import import_plan, register_importer
from .scheme import (FP8_BLOCK_128, FP8_PER_CHANNEL, FP8_PER_TENSOR, NVFP4_BLOCK_16, Granularity, Matcher, QDType,
                     QuantPlan, QuantScheme, Rule, TensorQuant, get_active_plan, load_quant_plan, use_quant_plan)
from .specs import (ActivationView, AllocationRequest, Bf16Spec, Fp8Spec, LinearActivationQuant, Nvfp4Spec, WeightSpec,
                    materialize)

__all__ = ["import_plan", "register_importer", "FP8_BLOCK_128", "FP8_PER_CHANNEL", "FP8_PER_TENSOR", "NVFP4_BLOCK_16",
           "Granularity", "Matcher", "QDType", "QuantPlan", "QuantScheme", "Rule", "TensorQuant", "get_active_plan",
           "load_quant_plan", "use_quant_plan", "AllocationRequest", "Bf16Spec", "Fp8Spec", "Nvfp4Spec", "materialize",
           "ActivationView", "WeightSpec", "LinearActivationQuant"]
