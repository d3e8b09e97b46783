"""Plugin ``pi05``: single-GPU Pi0.5 serving entry.

Reference: phyai/src/phyai/models/pi05/main_pi05.py:101-326 (argument bundle, config
resolution order, dropped checkpoint keys, camera-count validation).
"""

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
from .configuration_pi05 import PI05Config
from .modeling_pi05 import PI05Model
from .scheduler_ws1_pi05 import PI05Request, PI05WS1Scheduler

# present in upstream checkpoints, never consumed at inference (the expert emits vectors, not tokens)
PI05_DROP_KEYS = frozenset({"paligemma_with_expert.gemma_expert.lm_head.weight"})


def compose_remap(user):
    """Drop-set first, then the caller's callable / substring-replacement dict."""
    if user is not None and not callable(user) and not isinstance(user, dict):
        raise TypeError(f"weight_remap must be callable, dict or None, got {type(user).__name__}")

    def remap(key: str):
        if key in PI05_DROP_KEYS:
            return None
        if user is None:
            return key
        if callable(user):
            return user(key)
        for src, dst in user.items():
            if src in key:
                key = key.replace(src, dst)
        return key

    return remap


@dataclass
class PI05Args(EntryArgs):
    checkpoint_dir: str | Path | None = None      # None: default geometry, random weights
    config: PI05Config | None = None               # overrides checkpoint_dir/config.json
    max_batch_size: int = 1
    weight_remap: Callable[[str], str | None] | dict[str, str] | None = None
    weight_strict: bool = True
    vision_params_dtype: torch.dtype | None = None  # torch.float32 = vision tower parity path
    inputs_image_shape: list[list[int]] | None = None  # one [H, W, C] per camera; None = 3 cameras
    random_init_seed: int | None = 0               # used only when checkpoint_dir is None
    quantization: str | None = None                # "fp8_block": serve prefix decoder + expert in block-scaled fp8


def resolve_num_images(inputs_image_shape, num_channels: int) -> int:
    if inputs_image_shape is None:
        return 3
    if len(inputs_image_shape) == 0:
        raise ValueError("inputs_image_shape must list at least one image")
    for i, shape in enumerate(inputs_image_shape):
        if len(shape) != 3:
            raise ValueError(f"inputs_image_shape[{i}]={shape} must be [H, W, C]")
        h, w, c = shape
        if h <= 0 or w <= 0:
            raise ValueError(f"inputs_image_shape[{i}]: H and W must be positive, got [{h}, {w}]")
        if c != num_channels:
            raise ValueError(f"inputs_image_shape[{i}]: {c} channels, the vision tower takes {num_channels}")
    return len(inputs_image_shape)


@Engine.register
class PI05Entry(Entry):
    name: ClassVar[str] = "pi05"
    args_cls: ClassVar[type[EntryArgs]] = PI05Args
    #: mesh axis the vision encoder blocks are sharded over (``None``: whole tower on every rank)
    vision_axis: ClassVar[str | None] = "tp"

    def expert_axis_for(self, args) -> str | None:
        """Mesh axis the action expert is sharded over (``None``: whole on every rank)."""
        return "tp"

    def __init__(self) -> None:
        self.model: PI05Model | None = None
        self.scheduler: PI05WS1Scheduler | None = None

    def build_model(self, args: PI05Args) -> PI05Model:
        eng = get_engine_config()
        if args.config is not None:
            config = args.config
        elif args.checkpoint_dir is not None:
            config = load_config(args.checkpoint_dir, PI05Config)
        else:
            config = PI05Config()
        with use_quant_plan(load_quant_plan(args.checkpoint_dir)):
            model = PI05Model(config, vision_params_dtype=args.vision_params_dtype, device=eng.device.target,
                              vision_axis=self.vision_axis, expert_axis=self.expert_axis_for(args))
        if args.checkpoint_dir is not None:
            load_pretrained(model, args.checkpoint_dir, remap=compose_remap(args.weight_remap), strict=args.weight_strict)
        elif args.random_init_seed is not None:
            model.init_random(args.random_init_seed)
        return model

    def setup(self, args: PI05Args) -> None:  # type: ignore[override]
        eng = get_engine_config()
        self.model = self.build_model(args)
        n_img = resolve_num_images(args.inputs_image_shape, self.model.config.vision.num_channels)
        self.scheduler = PI05WS1Scheduler(self.model, max_batch_size=args.max_batch_size, num_images=n_img,
                                          device=eng.device.target, use_cuda_graph=eng.runtime.use_cuda_graph,
                                          quantization=args.quantization)
        self.scheduler.setup()

    def step(self, request: PI05Request) -> torch.Tensor:  # type: ignore[override]
        if self.scheduler is None:
            raise RuntimeError("PI05Entry.step before setup")
        return self.scheduler.step(request)

    def close(self) -> None:
        if self.scheduler is not None:
            self.scheduler.close()
        self.scheduler, self.model = None, None

    def dump_targets(self):
        return {} if self.model is None else {"model": self.model}


__all__ = ["PI05Args", "PI05Entry", "PI05_DROP_KEYS", "compose_remap", "resolve_num_images"]
