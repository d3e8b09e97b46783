from .configuration_qwen3_5 import Qwen3_5Config, Qwen3_5TextConfig, Qwen3_5VisionConfig, tiny_qwen3_5_config
from .modeling_qwen3_5 import Qwen3_5ForConditionalGeneration, Qwen3_5Model, Qwen3_5TextModel, qwen3_5_weight_remap

__all__ = ["Qwen3_5Config", "Qwen3_5TextConfig", "Qwen3_5VisionConfig", "tiny_qwen3_5_config", "Qwen3_5ForConditionalGeneration",
           "Qwen3_5Model", "Qwen3_5TextModel", "qwen3_5_weight_remap"]
