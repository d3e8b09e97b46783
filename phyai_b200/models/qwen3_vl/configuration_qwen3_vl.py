"""Qwen3-VL configuration (vision tower with DeepStack taps + mRoPE text decoder).

Reference: phyai/src/phyai/models/qwen3_vl/configuration_qwen3_vl.py:1-159.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..configuration import PretrainedConfig


@dataclass(frozen=True)
class Qwen3VLVisionConfig(PretrainedConfig):
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple[int, ...] = (8, 16, 24)
    hidden_act: str = "gelu_pytorch_tanh"

    def __post_init__(self) -> None:
        object.__setattr__(self, "deepstack_visual_indexes", tuple(self.deepstack_visual_indexes))


@dataclass(frozen=True)
class Qwen3VLTextConfig(PretrainedConfig):
    nested_sources = {"mrope_section": "rope_scaling.mrope_section"}

    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 5e6
    mrope_section: tuple[int, ...] = (24, 20, 20)
    hidden_act: str = "silu"

    def __post_init__(self) -> None:
        object.__setattr__(self, "mrope_section", tuple(self.mrope_section))


@dataclass(frozen=True)
class Qwen3VLConfig(PretrainedConfig):
    vision_config: Qwen3VLVisionConfig = field(default_factory=Qwen3VLVisionConfig)
    text_config: Qwen3VLTextConfig = field(default_factory=Qwen3VLTextConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652


def tiny_qwen3_vl_config() -> Qwen3VLConfig:
    return Qwen3VLConfig(
        vision_config=Qwen3VLVisionConfig(depth=3, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, out_hidden_size=48,
                                          num_position_embeddings=16, deepstack_visual_indexes=(0, 1)),
        text_config=Qwen3VLTextConfig(vocab_size=128, hidden_size=48, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                                      num_key_value_heads=2, head_dim=12, mrope_section=(2, 2, 2)),
        image_token_id=120, video_token_id=121, vision_start_token_id=119)


__all__ = ["Qwen3VLVisionConfig", "Qwen3VLTextConfig", "Qwen3VLConfig", "tiny_qwen3_vl_config"]
