"""Cosmos3: mixture-of-transformers world model (video / sound generation and action inference)."""

from .configuration_cosmos3 import (Cosmos3AVAESoundConfig, Cosmos3Config, Cosmos3WanVAEConfig, cosmos3_super_config,
                                    tiny_cosmos3_config)
from .sampler_unipc import UniPCMultistepSampler, resolve_use_karras_sigmas
from .scheduler_cosmos3 import (ACTION_MODES, Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3T2VRequest,
                                Cosmos3T2VScheduler, pixel_to_latent_shape)
from .transformer_cosmos3 import Cosmos3Transformer, cosmos3_weight_remap

__all__ = ["Cosmos3Config", "Cosmos3WanVAEConfig", "Cosmos3AVAESoundConfig", "cosmos3_super_config", "tiny_cosmos3_config",
           "UniPCMultistepSampler", "resolve_use_karras_sigmas", "Cosmos3T2VRequest", "Cosmos3ActionRequest",
           "Cosmos3T2VScheduler", "Cosmos3PolicyScheduler", "ACTION_MODES", "pixel_to_latent_shape", "Cosmos3Transformer",
           "cosmos3_weight_remap"]
