"""Rank-aware logging helpers (reference: phyai/src/phyai/utils/logging.py:25-71)."""

from __future__ import annotations

import logging
import os


def _rank_world() -> tuple[int, int]:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except Exception:
        pass
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def rank_prefix() -> str:
    r, w = _rank_world()
    return f"[rank {r}/{w}] "


def all_ranks_log(logger: logging.Logger, level: int, msg: str, *args) -> None:
    """Every rank emits the record, prefixed with ``[rank R/W]``."""
    if logger.isEnabledFor(level):
        logger.log(level, rank_prefix() + msg, *args)


def this_rank_log(logger: logging.Logger, level: int, msg: str, *args, rank: int = 0) -> None:
    """Only ``rank`` (default 0) emits the record."""
    r, _ = _rank_world()
    if r == rank:
        all_ranks_log(logger, level, msg, *args)


__all__ = ["all_ranks_log", "this_rank_log", "rank_prefix"]
