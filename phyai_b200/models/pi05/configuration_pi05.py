"""Pi0.5 configuration: SigLIP vision tower, PaliGemma (Gemma-2B) prefix LM, Gemma-300M
action expert with AdaRMS conditioning, and the flow-matching sampler knobs.

Defaults are the public ``pi05_base`` geometry (reference:
phyai/src/phyai/models/pi05/configuration_pi05.py:28-272). ``config.json`` files
written for the reference load here unchanged.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..configuration import PretrainedConfig


@dataclass(frozen=True)
class SiglipVisionConfig(PretrainedConfig):
    hidden_size: int = 1152
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    intermediate_size: int = 4304
    image_size: int = 224
    patch_size: int = 14
    num_channels: int = 3
    layer_norm_eps: float = 1e-6
    projection_dim: int = 2048

    def __post_init__(self) -> None:
        if self.image_size % self.patch_size:
            raise ValueError(f"image_size={self.image_size} is not a multiple of patch_size={self.patch_size}")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError(f"hidden_size={self.hidden_size} is not a multiple of num_attention_heads={self.num_attention_heads}")

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def _check_heads(c) -> None:
    if c.num_attention_heads % c.num_key_value_heads:
        raise ValueError(f"num_attention_heads={c.num_attention_heads} is not a multiple of "
                         f"num_key_value_heads={c.num_key_value_heads}")
    if c.head_dim <= 0 or c.head_dim % 2:
        raise ValueError(f"head_dim={c.head_dim} must be a positive even number")


@dataclass(frozen=True)
class PaliGemmaTextConfig(PretrainedConfig):
    hidden_size: int = 2048
    num_hidden_layers: int = 18
    num_attention_heads: int = 8
    num_key_value_heads: int = 1
    head_dim: int = 256
    intermediate_size: int = 16384
    vocab_size: int = 257152
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 8192

    def __post_init__(self) -> None:
        _check_heads(self)

    @property
    def joint_attention_dim(self) -> int:
        return self.num_attention_heads * self.head_dim


@dataclass(frozen=True)
class GemmaExpertConfig(PretrainedConfig):
    hidden_size: int = 1024
    num_hidden_layers: int = 18
    num_attention_heads: int = 8
    num_key_value_heads: int = 1
    head_dim: int = 256
    intermediate_size: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 8192
    use_adarms: bool = True
    adarms_cond_dim: int = 1024

    def __post_init__(self) -> None:
        _check_heads(self)
        if self.use_adarms and self.adarms_cond_dim != self.hidden_size:
            raise ValueError(f"adarms_cond_dim={self.adarms_cond_dim} must equal hidden_size={self.hidden_size}: "
                             "the time MLP output is the AdaRMS condition")

    @property
    def joint_attention_dim(self) -> int:
        return self.num_attention_heads * self.head_dim


@dataclass(frozen=True)
class PI05RecommendedEngineConfig(PretrainedConfig):
    """Engine knobs the model was tuned with. The two fields exist for config-file
    compatibility; this engine's attention kernels need neither a backend choice nor a workspace."""

    flashinfer_prefill_backend: str | None = "fa2"
    flashinfer_workspace_bytes: int = 256 * 1024 * 1024


@dataclass(frozen=True)
class PI05Config(PretrainedConfig):
    vision: SiglipVisionConfig = field(default_factory=SiglipVisionConfig)
    text: PaliGemmaTextConfig = field(default_factory=PaliGemmaTextConfig)
    expert: GemmaExpertConfig = field(default_factory=GemmaExpertConfig)
    chunk_size: int = 50
    max_action_dim: int = 32
    num_inference_steps: int = 10
    min_period: float = 4e-3
    max_period: float = 4.0
    tokenizer_max_length: int = 200
    recommended_engine: PI05RecommendedEngineConfig = field(default_factory=PI05RecommendedEngineConfig)

    def __post_init__(self) -> None:
        v, t, e = self.vision, self.text, self.expert
        if v.projection_dim != t.hidden_size:
            raise ValueError(f"vision.projection_dim={v.projection_dim} must equal text.hidden_size={t.hidden_size}")
        if t.joint_attention_dim != e.joint_attention_dim or t.head_dim != e.head_dim:
            raise ValueError("text and expert must agree on head_dim and heads*head_dim (joint attention)")
        if t.num_key_value_heads != e.num_key_value_heads:
            raise ValueError("text and expert must agree on num_key_value_heads (shared KV layout)")
        if t.num_hidden_layers != e.num_hidden_layers:
            raise ValueError("text and expert must have the same depth (layers are paired)")
        if self.chunk_size <= 0 or self.num_inference_steps <= 0:
            raise ValueError("chunk_size and num_inference_steps must be positive")

    @property
    def num_layers(self) -> int:
        return self.text.num_hidden_layers


def tiny_pi05_config(**over) -> PI05Config:
    """A small geometry for CPU tests: 2 layers everywhere, widths 64/128/64."""
    base = dict(
        vision=SiglipVisionConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=256,
                                  image_size=56, patch_size=14, projection_dim=128),
        text=PaliGemmaTextConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                                 head_dim=32, intermediate_size=512, vocab_size=1024),
        expert=GemmaExpertConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                                 head_dim=32, intermediate_size=256, adarms_cond_dim=64),
        chunk_size=10, max_action_dim=8, num_inference_steps=5, tokenizer_max_length=16)
    base.update(over)
    return PI05Config(**base)


__all__ = ["SiglipVisionConfig", "PaliGemmaTextConfig", "GemmaExpertConfig", "PI05RecommendedEngineConfig",
           "PI05Config", "tiny_pi05_config"]
