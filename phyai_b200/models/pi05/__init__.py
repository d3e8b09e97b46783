from .configuration_pi05 import (GemmaExpertConfig, PaliGemmaTextConfig, PI05Config, SiglipVisionConfig,
                                 tiny_pi05_config)

__all__ = ["GemmaExpertConfig", "PaliGemmaTextConfig", "PI05Config", "SiglipVisionConfig", "tiny_pi05_config"]
