"""Plugins ``cosmos3_policy`` / ``cosmos3_policy_wn``: action inference (policy, forward and
inverse dynamics) with the Cosmos3 transformer.

Reference: phyai/src/phyai/models/cosmos3/main_cosmos3_policy.py:36-157.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from pathlib import Path
from typing import ClassVar

from ...engine import Engine, Entry, EntryArgs
from ...engine_config import get_engine_config
from ...utils.logging import this_rank_log
from .configuration_cosmos3 import Cosmos3Config, Cosmos3WanVAEConfig
from .main_cosmos3 import build_transformer, build_vae
from .sampler_unipc import resolve_use_karras_sigmas
from .scheduler_cosmos3 import Cosmos3ActionRequest, Cosmos3PolicyScheduler
from .transformer_cosmos3 import Cosmos3Transformer
from .vae_wan import Cosmos3WanVAE

logger = logging.getLogger(__name__)


@dataclass
class Cosmos3PolicyArgs(EntryArgs):
    checkpoint_dir: str | Path | None = None
    config: Cosmos3Config | None = None
    flow_shift: float = 10.0
    use_karras_sigmas: bool | None = None   # None: scheduler/scheduler_config.json, else Karras
    decode_video: bool = False
    vae_config: Cosmos3WanVAEConfig | None = None
    weight_strict: bool = False
    random_init_seed: int = 0


@Engine.register
class Cosmos3PolicyEntry(Entry):
    name: ClassVar[str] = "cosmos3_policy"
    args_cls: ClassVar[type[EntryArgs]] = Cosmos3PolicyArgs

    def __init__(self) -> None:
        self.transformer: Cosmos3Transformer | None = None
        self.vae: Cosmos3WanVAE | None = None
        self.scheduler: Cosmos3PolicyScheduler | None = None
        self.decode_video = False

    def setup(self, args: Cosmos3PolicyArgs) -> None:  # type: ignore[override]
        eng = get_engine_config()
        device, dtype = eng.device.target, eng.device.params_dtype
        ckpt = Path(args.checkpoint_dir) if args.checkpoint_dir is not None else None
        self.decode_video = bool(args.decode_video)
        self.transformer = build_transformer(args, ckpt, device, dtype)
        if self.decode_video:
            self.vae = build_vae(args, ckpt, device, dtype)
        karras = resolve_use_karras_sigmas(args.use_karras_sigmas, ckpt)
        self.scheduler = Cosmos3PolicyScheduler(self.transformer, vae=self.vae, device=device, flow_shift=args.flow_shift,
                                                use_karras_sigmas=karras)
        self.scheduler.setup()
        this_rank_log(logger, logging.INFO, "%s ready (cfg=%d, decode_video=%s, flow_shift=%s, karras=%s)", self.name,
                      self.scheduler.cfg_size, self.decode_video, args.flow_shift, karras)

    def step(self, request: Cosmos3ActionRequest):  # type: ignore[override]
        """The action (B, chunk, raw_action_dim); the dict ``action / video / pixels`` when built with ``decode_video``."""
        if self.scheduler is None:
            raise RuntimeError(f"{type(self).__name__}.step before setup")
        out = self.scheduler.step(request, decode_video=self.decode_video)
        return out if self.decode_video else out["action"]

    def close(self) -> None:
        if self.scheduler is not None:
            self.scheduler.close()
        self.scheduler = self.transformer = self.vae = None

    def dump_targets(self):
        return {} if self.transformer is None else {"transformer": self.transformer}


__all__ = ["Cosmos3PolicyArgs", "Cosmos3PolicyEntry"]
