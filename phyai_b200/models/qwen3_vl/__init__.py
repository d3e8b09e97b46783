from .configuration_qwen3_vl import Qwen3VLConfig, Qwen3VLTextConfig, Qwen3VLVisionConfig, tiny_qwen3_vl_config
from .modeling_qwen3_vl import Qwen3VLForConditionalGeneration, Qwen3VLModel, Qwen3VLTextModel, Qwen3VLVisionModel

__all__ = ["Qwen3VLConfig", "Qwen3VLTextConfig", "Qwen3VLVisionConfig", "tiny_qwen3_vl_config", "Qwen3VLForConditionalGeneration",
           "Qwen3VLModel", "Qwen3VLTextModel", "Qwen3VLVisionModel"]
