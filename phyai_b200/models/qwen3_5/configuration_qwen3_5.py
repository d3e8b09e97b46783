"""Qwen3.5 configuration: hybrid decoder (three gated-delta-net layers per full-attention layer), partial mRoPE.

Reference: phyai/src/phyai/models/qwen3_5/configuration_qwen3_5.py:11-168.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..configuration import PretrainedConfig


@dataclass(frozen=True)
class Qwen3_5VisionConfig(PretrainedConfig):
    depth: int = 12
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_heads: int = 12
    in_channels: int = 3
    patch_size: int = 16
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    out_hidden_size: int = 1024
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple[int, ...] = ()
    hidden_act: str = "gelu_pytorch_tanh"


@dataclass(frozen=True)
class Qwen3_5TextConfig(PretrainedConfig):
    nested_sources = {"mrope_section": "rope_parameters.mrope_section", "partial_rotary_factor": "rope_parameters.partial_rotary_factor",
                      "rope_theta": "rope_parameters.rope_theta"}

    vocab_size: int = 248320
    hidden_size: int = 1024
    intermediate_size: int = 3584
    num_hidden_layers: int = 24
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 256
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    mrope_section: tuple[int, ...] = (11, 11, 10)
    attn_output_gate: bool = True
    tie_word_embeddings: bool = True
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 16
    layer_types: tuple[str, ...] = ("linear_attention", "linear_attention", "linear_attention", "full_attention") * 6

    def __post_init__(self) -> None:
        object.__setattr__(self, "mrope_section", tuple(self.mrope_section))
        object.__setattr__(self, "layer_types", tuple(self.layer_types))
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError(f"{len(self.layer_types)} layer types for {self.num_hidden_layers} layers")
        if not set(self.layer_types) <= {"linear_attention", "full_attention"}:
            raise ValueError(f"layer_types may hold 'linear_attention' and 'full_attention' only, got {self.layer_types}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        rot = int(self.head_dim * self.partial_rotary_factor)
        if rot <= 0 or rot % 2 or sum(self.mrope_section) != rot // 2:
            raise ValueError(f"mrope_section {self.mrope_section} must sum to rotary_dim/2 = {rot // 2}")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)


@dataclass(frozen=True)
class Qwen3_5Config(PretrainedConfig):
    vision_config: Qwen3_5VisionConfig = field(default_factory=Qwen3_5VisionConfig)
    text_config: Qwen3_5TextConfig = field(default_factory=Qwen3_5TextConfig)
    image_token_id: int = 248056
    video_token_id: int = 248057


def tiny_qwen3_5_config() -> Qwen3_5Config:
    return Qwen3_5Config(
        vision_config=Qwen3_5VisionConfig(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, out_hidden_size=48,
                                          num_position_embeddings=16),
        text_config=Qwen3_5TextConfig(vocab_size=128, hidden_size=48, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4,
                                      num_key_value_heads=2, head_dim=16, partial_rotary_factor=0.5, mrope_section=(2, 1, 1),
                                      linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4,
                                      layer_types=("linear_attention", "linear_attention", "linear_attention", "full_attention")),
        image_token_id=120, video_token_id=121)


__all__ = ["Qwen3_5VisionConfig", "Qwen3_5TextConfig", "Qwen3_5Config", "tiny_qwen3_5_config"]
