from . import shards
from .loader import LoadReport, build_index, load_pretrained, run_post_load
from .synthetic import synthetic_state_dict, write_checkpoint

__all__ = ["shards", "LoadReport", "build_index", "load_pretrained", "run_post_load",
           "synthetic_state_dict", "write_checkpoint"]
