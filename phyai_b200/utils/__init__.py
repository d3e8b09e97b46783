from .checkpoint import find_safetensors, load_config, resolve_checkpoint
from .cuda import init_cublas, init_cuda, print_distributed_topology, print_topology, sm_arch
from .logging import all_ranks_log, this_rank_log
from .profile import (NoOpProfiler, NsysProfiler, NvtxProfiler, Profiler, make_profiler, set_profiler, ProfilerConfig, TimelineProfiler, TorchProfiler, add_profile_cli_args, event_scope,
                      get_profiler, install_profiler, mark_instant, profile_config_from_args)

__all__ = ["find_safetensors", "load_config", "resolve_checkpoint", "init_cublas", "init_cuda",
           "print_distributed_topology", "print_topology", "sm_arch", "all_ranks_log", "this_rank_log", "NoOpProfiler", "NvtxProfiler", "NsysProfiler", "Profiler", "make_profiler", "set_profiler",
           "ProfilerConfig", "TimelineProfiler", "TorchProfiler", "add_profile_cli_args", "event_scope", "get_profiler",
           "install_profiler", "mark_instant", "profile_config_from_args"]
