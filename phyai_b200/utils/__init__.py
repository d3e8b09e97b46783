from .checkpoint import find_safetensors, load_config, resolve_checkpoint
from .cuda import init_cublas, init_cuda, print_distributed_topology, print_topology, sm_arch
from .logging import all_ranks_log, this_rank_log

__all__ = ["find_safetensors", "load_config", "resolve_checkpoint", "init_cublas", "init_cuda",
           "print_distributed_topology", "print_topology", "sm_arch", "all_ranks_log", "this_rank_log"]
