"""Pi0: PaliGemma prefix + flow-matching action expert with a state token."""

from ..pi05.configuration_pi05 import GemmaExpertConfig, PaliGemmaTextConfig, SiglipVisionConfig
from .configuration_pi0 import PI0Config, tiny_pi0_config

_MODELING = ("PI0Model", "PI0ExpertStack", "PI0Heads")
# pieces Pi0 shares with Pi0.5 (same classes), under the names the reference's pi0 package exports
_SHARED = {"PaliGemmaLanguageModel": "PaliGemmaLanguageModel", "PaliGemmaDecoderLayer": "PaliGemmaDecoderLayer", "PI0VisionTower": "PI05VisionTower",
           "PI0ExpertLayer": "PaliGemmaDecoderLayer"}
_SCHEDULING = {"PI0Request": "scheduler_ws1_pi0", "PI0WS1Scheduler": "scheduler_ws1_pi0"}


def __getattr__(name: str):
    import importlib

    if name in _MODELING:
        return getattr(importlib.import_module(".modeling_pi0", __name__), name)
    if name == "ActionTimeHeads":
        return importlib.import_module(".modeling_pi0", __name__).PI0Heads
    if name in _SHARED:
        return getattr(importlib.import_module("..pi05.modeling_pi05", __name__), _SHARED[name])
    if name in _SCHEDULING:
        return getattr(importlib.import_module("." + _SCHEDULING[name], __name__), name)
    raise AttributeError(name)


__all__ = ["GemmaExpertConfig", "PaliGemmaTextConfig", "SiglipVisionConfig", "PI0Config", "tiny_pi0_config", *_MODELING, *_SCHEDULING, "ActionTimeHeads", *_SHARED]
