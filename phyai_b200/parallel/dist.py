"""Process-group bootstrap (reference: phyai/src/phyai/parallel/dist.py:26-89)."""

from __future__ import annotations

import datetime
import os

import torch

from ..env import envs


def init_dist(world_size: int, device_type: str, *, timeout_s: float | None = None) -> bool:
    """Make sure a default process group of ``world_size`` ranks exists.

    Returns True when this call created the group (the caller then owns its
    teardown). ``world_size == 1`` needs no group. Rendezvous values come from the
    torchrun variables, defaulting to a single-host setup on 127.0.0.1.
    """
    import torch.distributed as dist

    if world_size <= 1:
        return False
    if dist.is_initialized():
        if dist.get_world_size() != world_size:
            raise RuntimeError(f"process group has {dist.get_world_size()} ranks, config wants {world_size}")
        return False
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    rank = int(os.environ.get("RANK", "0"))
    backend = "nccl" if device_type == "cuda" else "gloo"
    if backend == "nccl":
        backend = "cuda:nccl,cpu:gloo"  # host-side object exchange and heartbeats ride on gloo
    t = timeout_s if timeout_s is not None else envs.PHYAI_COMM_TIMEOUT_S.get()
    kwargs = {}
    if device_type == "cuda" and torch.cuda.is_available():
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, rank=rank, world_size=world_size,
                            timeout=datetime.timedelta(seconds=t), **kwargs)
    return True


def destroy_dist() -> None:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


__all__ = ["init_dist", "destroy_dist"]
