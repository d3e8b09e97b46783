"""Plugin ``pi0`` (reference: phyai/src/phyai/models/pi0/main_pi0.py:27-145)."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable, ClassVar

import torch

from ...engine import Engine, Entry, EntryArgs
from ...engine_config import get_engine_config
from ...layers.quant import load_quant_plan, use_quant_plan
from ...utils.checkpoint import load_config
from ...weights import load_pretrained
from ..pi05.main_pi05 import resolve_num_images
from .configuration_pi0 import PI0Config
from .modeling_pi0 import PI0Model
from .scheduler_ws1_pi0 import PI0Request, PI0WS1Scheduler

PI0_DROP_KEYS = frozenset({"paligemma_with_expert.gemma_expert.lm_head.weight"})


def pi0_default_remap(key: str) -> str | None:
    """Upstream compatibility: strip a leading ``model.``, drop the unused expert lm_head, and map the
    older ``time_mlp_*`` names onto ``action_time_mlp_*``."""
    if key.startswith("model."):
        key = key[len("model."):]
    if key in PI0_DROP_KEYS:
        return None
    for old, new in (("time_mlp_in.", "action_time_mlp_in."), ("time_mlp_out.", "action_time_mlp_out.")):
        if key.startswith(old):
            return new + key[len(old):]
    return key


def compose_remap(user):
    if user is not None and not callable(user) and not isinstance(user, dict):
        raise TypeError(f"weight_remap must be callable, dict or None, got {type(user).__name__}")

    def remap(key: str):
        key = pi0_default_remap(key)
        if key is None or user is None:
            return key
        if callable(user):
            return user(key)
        for src, dst in user.items():
            if src in key:
                key = key.replace(src, dst)
        return key

    return remap


@dataclass
class PI0Args(EntryArgs):
    checkpoint_dir: str | Path | None = None
    config: PI0Config | None = None
    max_batch_size: int = 1
    weight_remap: Callable[[str], str | None] | dict[str, str] | None = None
    weight_strict: bool = True
    vision_params_dtype: torch.dtype | None = None
    inputs_image_shape: list[list[int]] | None = None
    random_init_seed: int | None = 0


@Engine.register
class PI0Entry(Entry):
    name: ClassVar[str] = "pi0"
    args_cls: ClassVar[type[EntryArgs]] = PI0Args

    def __init__(self) -> None:
        self.model: PI0Model | None = None
        self.scheduler: PI0WS1Scheduler | None = None

    def build_local(self, args: PI0Args, max_batch_size: int) -> PI0WS1Scheduler:
        eng = get_engine_config()
        config = args.config or (load_config(args.checkpoint_dir, PI0Config) if args.checkpoint_dir else PI0Config())
        with use_quant_plan(load_quant_plan(args.checkpoint_dir)):
            self.model = PI0Model(config, vision_params_dtype=args.vision_params_dtype, device=eng.device.target)
        if args.checkpoint_dir is not None:
            load_pretrained(self.model, args.checkpoint_dir, remap=compose_remap(args.weight_remap), strict=args.weight_strict)
        elif args.random_init_seed is not None:
            self.model.init_random(args.random_init_seed)
        n_img = resolve_num_images(args.inputs_image_shape, config.vision.num_channels)
        return PI0WS1Scheduler(self.model, max_batch_size=max_batch_size, num_images=n_img,
                               device=eng.device.target, use_cuda_graph=eng.runtime.use_cuda_graph)

    def setup(self, args: PI0Args) -> None:  # type: ignore[override]
        self.scheduler = self.build_local(args, args.max_batch_size)
        self.scheduler.setup()

    def step(self, request: PI0Request) -> torch.Tensor:  # type: ignore[override]
        if self.scheduler is None:
            raise RuntimeError("PI0Entry.step before setup")
        return self.scheduler.step(request)

    def close(self) -> None:
        if self.scheduler is not None:
            self.scheduler.close()
        self.scheduler, self.model = None, None

    def dump_targets(self):
        return {} if self.model is None else {"model": self.model}


__all__ = ["PI0Args", "PI0Entry", "pi0_default_remap", "compose_remap"]
