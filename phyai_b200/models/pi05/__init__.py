"""Pi0.5: PaliGemma prefix + flow-matching action expert with time-conditioned norms."""

from .configuration_pi05 import (GemmaExpertConfig, PaliGemmaTextConfig, PI05Config, SiglipVisionConfig,
                                 tiny_pi05_config)

_MODELING = ("PI05Model", "PI05VisionTower", "PaliGemmaLanguageModel", "PI05ExpertStack", "ActionTimeHeads", "PaliGemmaDecoderLayer",
             "PI05ExpertLayer", "GemmaMLP", "GemmaAttentionProj", "SiglipBlock", "dense_attention")
_SCHEDULING = {"PI05Request": "scheduler_ws1_pi05", "PI05WS1Scheduler": "scheduler_ws1_pi05", "PI05WNScheduler": "scheduler_wn_pi05",
               "PI05Plan": "plan_pi05", "PI05TPPlan": "plan_tp_pi05"}


def __getattr__(name: str):
    # the model and scheduler modules import the layer stack (and on a GPU box the CUDA extension): on first use only
    import importlib

    if name in _MODELING:
        return getattr(importlib.import_module(".modeling_pi05", __name__), name)
    if name in _SCHEDULING:
        return getattr(importlib.import_module("." + _SCHEDULING[name], __name__), name)
    raise AttributeError(name)


__all__ = ["GemmaExpertConfig", "PaliGemmaTextConfig", "PI05Config", "SiglipVisionConfig", "tiny_pi05_config", *_MODELING, *_SCHEDULING]
