"""Plugin ``pi05_tp``: tensor-parallel Pi0.5 (every rank holds a slice of each projection).

All ranks of the ``tp`` axis take the same request and return the same action chunk. The attention
heads and MLP columns are sharded by the parallel linear layers (the single KV head of the Gemma
stacks is replicated); the row-parallel products are summed with ``parallel.all_reduce``, which on
CUDA goes to the peer-memory backend for these small messages (one push kernel + one reduce kernel,
no NCCL launch). The model runs its eager path here: the single-GPU plugin's captured plan assumes
whole weights, and one B200 already serves the batch-1 case faster than a TP group can (about 17 ms;
a TP step adds 2 x 36 reductions per denoise step), so this entry exists for checkpoints that do
not fit one GPU and for parity with TP-capable layers.

The reference has TP-capable Pi0.5 layers and no scheduler that drives them
(phyai/src/phyai/models/pi05/modeling_pi05.py:388-1008; its schedulers are scheduler_ws1_pi05.py and scheduler_wn_pi05.py, single GPU and data parallel).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from ... import parallel as P
from ...engine import Engine, EntryArgs
from ...engine_config import get_engine_config
from ...runtime import Scheduler
from .main_pi05 import PI05Args, PI05Entry, resolve_num_images
from .modeling_pi05 import PI05Model
from .scheduler_ws1_pi05 import PI05Request


class PI05TPScheduler(Scheduler):
    def __init__(self, model: PI05Model, *, max_batch_size: int, num_images: int, device) -> None:
        self.model, self.max_batch_size, self.num_images = model, max_batch_size, num_images
        self.device = torch.device(device)
        mesh = P.default_mesh()
        self.tp_size = mesh.axis_size("tp") if mesh is not None else 1
        self.tp_rank = mesh.axis_local_rank("tp") if mesh is not None else 0

    def setup(self) -> None:
        if self.tp_size > 1:
            P.warmup(("tp",))

    @torch.no_grad()
    def step(self, request: PI05Request) -> torch.Tensor:
        B = request.pixel_values.shape[0]
        if B > self.max_batch_size:
            raise ValueError(f"batch of {B} exceeds max_batch_size={self.max_batch_size}")
        if request.pixel_values.shape[1] != self.num_images:
            raise ValueError(f"{request.pixel_values.shape[1]} cameras, the plugin was set up for {self.num_images}")
        cfg = self.model.config
        noise = request.noise
        if noise is None:
            g = torch.Generator(device="cpu").manual_seed(0)     # identical on every rank
            noise = torch.randn(B, cfg.chunk_size, cfg.max_action_dim, generator=g)
        dt = next(self.model.parameters()).dtype
        return self.model.sample_actions(request.pixel_values.to(self.device, dt), request.input_ids.to(self.device),
                                         request.lang_lens.to(self.device), noise.to(self.device, dt))

    def close(self) -> None:
        return None


@dataclass
class PI05TPArgs(PI05Args):
    pass


@Engine.register
class PI05TPEntry(PI05Entry):
    name: ClassVar[str] = "pi05_tp"
    args_cls: ClassVar[type[EntryArgs]] = PI05TPArgs

    def setup(self, args: PI05TPArgs) -> None:  # type: ignore[override]
        eng = get_engine_config()
        self.model = self.build_model(args)
        n_img = resolve_num_images(args.inputs_image_shape, self.model.config.vision.num_channels)
        self.scheduler = PI05TPScheduler(self.model, max_batch_size=args.max_batch_size, num_images=n_img, device=eng.device.target)
        self.scheduler.setup()


__all__ = ["PI05TPArgs", "PI05TPEntry", "PI05TPScheduler"]
