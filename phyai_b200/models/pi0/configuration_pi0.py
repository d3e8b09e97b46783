"""Pi0 configuration (reference: phyai/src/phyai/models/pi0/configuration_pi0.py:24-231).

Same towers as Pi0.5; the action expert uses plain Gemma RMSNorm (no AdaRMS), the robot
state enters as one extra suffix token, and the prompt budget is 48 tokens.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..configuration import PretrainedConfig
from ..pi05.configuration_pi05 import GemmaExpertConfig, PaliGemmaTextConfig, SiglipVisionConfig


def _pi0_expert() -> GemmaExpertConfig:
    return GemmaExpertConfig(use_adarms=False)


@dataclass(frozen=True)
class PI0Config(PretrainedConfig):
    vision: SiglipVisionConfig = field(default_factory=SiglipVisionConfig)
    text: PaliGemmaTextConfig = field(default_factory=PaliGemmaTextConfig)
    expert: GemmaExpertConfig = field(default_factory=_pi0_expert)
    chunk_size: int = 50
    max_state_dim: int = 32
    max_action_dim: int = 32
    num_inference_steps: int = 10
    min_period: float = 4e-3
    max_period: float = 4.0
    tokenizer_max_length: int = 48
    empty_cameras: int = 0

    def __post_init__(self) -> None:
        v, t, e = self.vision, self.text, self.expert
        if v.projection_dim != t.hidden_size:
            raise ValueError("vision.projection_dim must equal text.hidden_size")
        if (t.joint_attention_dim != e.joint_attention_dim or t.head_dim != e.head_dim
                or t.num_key_value_heads != e.num_key_value_heads or t.num_hidden_layers != e.num_hidden_layers):
            raise ValueError("text and expert must agree on heads, head_dim, kv heads and depth")
        if e.use_adarms:
            raise ValueError("the Pi0 expert uses plain RMSNorm (use_adarms must be False)")
        if self.chunk_size <= 0 or self.num_inference_steps <= 0:
            raise ValueError("chunk_size and num_inference_steps must be positive")

    @property
    def num_layers(self) -> int:
        return self.text.num_hidden_layers

    @property
    def suffix_len(self) -> int:
        return 1 + self.chunk_size


def tiny_pi0_config(**over) -> PI0Config:
    """The small CPU geometry: ViT 2 layers width 64, Gemma-style prefix 2 layers hidden 128
    (4 q heads / 1 kv head, head_dim 32, MLP 512, vocab 1024), expert 2 layers width 64,
    state 8, horizon 10 x action 8, 5 Euler steps, 16 prompt tokens, 56x56 images."""
    base = dict(
        vision=SiglipVisionConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=256,
                                  image_size=56, patch_size=14, projection_dim=128),
        text=PaliGemmaTextConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                                 head_dim=32, intermediate_size=512, vocab_size=1024),
        expert=GemmaExpertConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                                 head_dim=32, intermediate_size=256, use_adarms=False, adarms_cond_dim=64),
        chunk_size=10, max_state_dim=8, max_action_dim=8, num_inference_steps=5, tokenizer_max_length=16)
    base.update(over)
    return PI0Config(**base)


__all__ = ["PI0Config", "tiny_pi0_config"]
