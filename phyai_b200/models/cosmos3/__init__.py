"""Cosmos3: mixture-of-transformers world model (video / sound generation and action inference)."""

from .configuration_cosmos3 import (Cosmos3AVAESoundConfig, Cosmos3Config, Cosmos3WanVAEConfig, cosmos3_super_config,
                                    tiny_cosmos3_config)
from .sampler_unipc import UniPCMultistepSampler, resolve_use_karras_sigmas
from .avae_sound import Cosmos3AVAESoundDecoder, cosmos3_avae_weight_remap
from .modeling_cosmos3 import Cosmos3Condition
from .scheduler_cosmos3 import (ACTION_MODES, Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3PolicyWNScheduler, Cosmos3Runner,
                                Cosmos3T2VRequest, Cosmos3T2VScheduler, Cosmos3T2VWNScheduler, pixel_to_latent_shape)
from .transformer_cosmos3 import Cosmos3Transformer, cosmos3_weight_remap
from .vae_wan import Cosmos3WanVAE, cosmos3_vae_weight_remap

# one runner class serves the video and the action schedulers
Cosmos3T2VRunner = Cosmos3ActionRunner = Cosmos3Runner

__all__ = ["Cosmos3Config", "Cosmos3WanVAEConfig", "Cosmos3AVAESoundConfig", "cosmos3_super_config", "tiny_cosmos3_config",
           "UniPCMultistepSampler", "resolve_use_karras_sigmas", "Cosmos3T2VRequest", "Cosmos3ActionRequest",
           "Cosmos3T2VScheduler", "Cosmos3PolicyScheduler", "ACTION_MODES", "pixel_to_latent_shape", "Cosmos3Transformer",
           "cosmos3_weight_remap", "Cosmos3Condition", "Cosmos3Runner", "Cosmos3T2VRunner", "Cosmos3ActionRunner", "Cosmos3T2VWNScheduler", "Cosmos3PolicyWNScheduler",
           "Cosmos3WanVAE", "cosmos3_vae_weight_remap", "Cosmos3AVAESoundDecoder", "cosmos3_avae_weight_remap"]
