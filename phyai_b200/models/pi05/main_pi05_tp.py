"""Plugin ``pi05_tp``: tensor-parallel Pi0.5 (every rank holds a slice of each projection).

All ranks of the ``tp`` axis take the same request and return the same action chunk. On CUDA bf16 the
request runs through :class:`PI05TPPlan`, captured as one CUDA graph per prompt bucket: q heads and
MLP columns of the prefix decoder are sharded (the single KV head of the Gemma stacks is replicated), every
row-parallel product leaves its GEMM through the epilogue into the peers' memory and is summed by the kernel
that also applies the residual and the next RMS norm, the cameras (not the vision weights) are split over the
ranks, and the action expert stays whole on every rank unless ``shard_expert`` asks otherwise. Elsewhere (CPU, fp32, a single rank) the eager model path runs, with the
row-parallel products summed by ``parallel.all_reduce``.

The reference has TP-capable Pi0.5 layers and no scheduler that drives them
(phyai/src/phyai/models/pi05/modeling_pi05.py:388-1008; its schedulers are scheduler_ws1_pi05.py and scheduler_wn_pi05.py, single GPU and data parallel).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import ClassVar

import torch

from ... import parallel as P
from ...engine import Engine, EntryArgs
from ...engine_config import get_engine_config
from .main_pi05 import PI05Args, PI05Entry, resolve_num_images
from .modeling_pi05 import PI05Model
from .plan_pi05 import PI05Plan
from .scheduler_ws1_pi05 import PI05Request, PI05WS1Scheduler


class PI05TPScheduler(PI05WS1Scheduler):
    """The single-GPU scheduler with the tensor-parallel plan behind it. Noise that the request does not
    carry is drawn on the host from a generator every rank seeds alike, so the ranks stay identical."""

    def __init__(self, model: PI05Model, *, max_batch_size: int, num_images: int, device, use_cuda_graph: bool = True,
                 axis: str = "tp") -> None:
        super().__init__(model, max_batch_size=max_batch_size, num_images=num_images, device=device,
                         use_cuda_graph=use_cuda_graph)
        self.axis = axis
        mesh = P.default_mesh()
        self.tp_size = mesh.axis_size(axis) if mesh is not None else 1
        self.tp_rank = mesh.axis_local_rank(axis) if mesh is not None else 0
        self._noise_gen = torch.Generator(device="cpu").manual_seed(0)
        # the plan splits the cameras over the ranks and needs the whole vision tower on each of them
        if self.tp_size > 1 and model.vision.blocks[0].out.tp_size > 1:
            self.use_plan = self.use_cuda_graph = False

    def setup(self) -> None:
        super().setup()
        if self.tp_size > 1 and not self.use_plan:
            P.warmup((self.axis,))

    def _make_plan(self) -> PI05Plan:
        if self.tp_size == 1:
            return super()._make_plan()
        from .plan_tp_pi05 import PI05TPPlan

        return PI05TPPlan(self.model, max_batch_size=self.max_batch_size, num_images=self.num_images, device=self.device,
                          axis=self.axis)

    def _before_capture(self, bucket: int) -> None:
        # the warm-up runs execute the peer kernels for real, and their waits on peers are bounded: start together
        if self.tp_size > 1:
            self.plan.pg.sync()

    def _captured(self, bucket: int) -> None:
        # capture time differs between ranks; the first replay's bounded waits start together
        if self.tp_size > 1:
            self.plan.pg.sync()

    def close(self) -> None:
        """Drops the graphs, then (collectively) the peer mappings: a later engine of the same process gets a fresh group."""
        pg = getattr(self.plan, "pg", None)
        super().close()
        if pg is not None:
            torch.cuda.synchronize()
            pg.close()

    @torch.no_grad()
    def step(self, request: PI05Request) -> torch.Tensor:
        if request.noise is None:
            cfg = self.cfg
            B = request.pixel_values.shape[0]
            noise = torch.randn(B, cfg.chunk_size, cfg.max_action_dim, generator=self._noise_gen)
            request = dataclasses.replace(request, noise=noise)
        return super().step(request)


@dataclass
class PI05TPArgs(PI05Args):
    #: shard the action expert too. Off by default: at 0.6 GB it is kept whole on every rank, which lets the Euler
    #: loop run without communication (the latency-bound part of a request); on, its blocks reduce over peer memory
    shard_expert: bool = False


@Engine.register
class PI05TPEntry(PI05Entry):
    name: ClassVar[str] = "pi05_tp"
    args_cls: ClassVar[type[EntryArgs]] = PI05TPArgs
    #: the encoder blocks of the vision tower stay whole on every rank (see PI05TPPlan)
    vision_axis: ClassVar[str | None] = None

    def expert_axis_for(self, args) -> str | None:
        return "tp" if getattr(args, "shard_expert", False) else None

    def setup(self, args: PI05TPArgs) -> None:  # type: ignore[override]
        eng = get_engine_config()
        self.model = self.build_model(args)
        n_img = resolve_num_images(args.inputs_image_shape, self.model.config.vision.num_channels)
        self.scheduler = PI05TPScheduler(self.model, max_batch_size=args.max_batch_size, num_images=n_img, device=eng.device.target,
                                         use_cuda_graph=eng.runtime.use_cuda_graph)
        self.scheduler.setup()


__all__ = ["PI05TPArgs", "PI05TPEntry", "PI05TPScheduler"]
