from . import shards
from .shards import Loader, fused, replicated, sharded, vocab, weight_norm_fold
from .loader import LoadReport, build_index, load_pretrained, run_post_load
from .synthetic import synthetic_state_dict, write_checkpoint

WeightLoader = Loader

__all__ = ["Loader", "WeightLoader", "fused", "replicated", "sharded", "vocab", "weight_norm_fold", "shards", "LoadReport", "build_index", "load_pretrained", "run_post_load",
           "synthetic_state_dict", "write_checkpoint"]
