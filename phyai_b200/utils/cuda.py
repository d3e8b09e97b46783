"""Device helpers (reference: phyai/src/phyai/utils/cuda.py:26-211)."""

from __future__ import annotations

import logging
import os
from functools import lru_cache

import torch

from .logging import this_rank_log

logger = logging.getLogger(__name__)


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))


@lru_cache(maxsize=None)
def _sm_arch_of(index: int) -> int:
    major, minor = torch.cuda.get_device_capability(index)
    return major * 10 + minor


def sm_arch(device: torch.device | str | int | None = None) -> int:
    """Compute capability as an int (100 for B200); 0 when no GPU is visible."""
    if not torch.cuda.is_available():
        return 0
    if device is None:
        idx = torch.cuda.current_device()
    elif isinstance(device, int):
        idx = device
    else:
        d = torch.device(device)
        idx = d.index if d.index is not None else torch.cuda.current_device()
    return _sm_arch_of(idx)


def init_cuda(target: str, params_dtype: torch.dtype) -> torch.device:
    """Bind this process to its device (``cuda`` without an index means LOCAL_RANK)."""
    dev = torch.device(target)
    if dev.type == "cuda":
        if not torch.cuda.is_available():
            raise RuntimeError(f"device.target={target!r} but no CUDA device is visible")
        idx = dev.index if dev.index is not None else local_rank() % max(torch.cuda.device_count(), 1)
        torch.cuda.set_device(idx)
        dev = torch.device("cuda", idx)
    # Parameters are always created with an explicit dtype, so the process-wide
    # default dtype is left alone (user code keeps float32 arithmetic).
    return dev


def init_cublas() -> None:
    """Kept for API parity: the GEMMs here are this repository's own kernels."""


def topology_lines() -> list[str]:
    lines: list[str] = []
    if not torch.cuda.is_available():
        return ["no CUDA device visible"]
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        lines.append(f"cuda:{i} {p.name} sm_{p.major}{p.minor} {p.multi_processor_count} SMs "
                     f"{p.total_memory / 2**30:.0f} GiB")
    n = torch.cuda.device_count()
    for i in range(n):
        row = []
        for j in range(n):
            row.append("self" if i == j else ("p2p" if torch.cuda.can_device_access_peer(i, j) else "----"))
        lines.append(f"  peer access cuda:{i}: " + " ".join(row))
    return lines


def print_topology() -> None:
    for line in topology_lines():
        this_rank_log(logger, logging.INFO, "%s", line)


def print_distributed_topology() -> None:
    """Gather (rank, host, device) from every rank and print the table on rank 0."""
    import socket

    import torch.distributed as dist

    me = {"rank": dist.get_rank() if dist.is_initialized() else 0, "host": socket.gethostname(),
          "device": torch.cuda.current_device() if torch.cuda.is_available() else -1}
    rows = [me]
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        rows = [None] * dist.get_world_size()
        dist.all_gather_object(rows, me)
    for r in sorted(rows, key=lambda x: x["rank"]):
        this_rank_log(logger, logging.INFO, "rank %d on %s cuda:%d", r["rank"], r["host"], r["device"])


__all__ = ["sm_arch", "init_cuda", "init_cublas", "print_topology", "print_distributed_topology",
           "topology_lines", "local_rank"]
