"""Single-GPU Pi0.5 scheduler: request -> action chunk.

On CUDA bf16 the request runs through :class:`PI05Plan` as ONE CUDA graph per
prompt-length bucket (vision + prefix + Euler loop); the per-shape metadata lives in
static device buffers that are rewritten only when ``(batch, lang_lens)`` changes, so a
steady stream of same-shape requests does no host-side planning at all. Anywhere else
(CPU, fp32 parity, tensor dumps) the eager model path runs.

Reference behaviour: phyai/src/phyai/models/pi05/scheduler_ws1_pi05.py:163-779
(request fields, prompt buckets {16, 48, 112, max}, padding of short batches).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ...runtime import CudaGraphRegistry, Scheduler
from ...utils.profile import event_scope
from .modeling_pi05 import PI05Model
from .plan_pi05 import PI05Layout, PI05Plan


@dataclass
class PI05Request:
    """One inference call for up to ``max_batch_size`` robots.

    pixel_values  (B, n_img, C, H, W) in [-1, 1], already at the tower resolution
    input_ids     (B, tokenizer_max_length) int64, right-padded
    lang_lens     (B,) int64 number of real prompt tokens per robot
    noise         optional (B, chunk, action_dim) starting noise; drawn N(0,1) when absent
    """

    pixel_values: torch.Tensor
    input_ids: torch.Tensor
    lang_lens: torch.Tensor
    noise: torch.Tensor | None = None


class PI05WS1Scheduler(Scheduler):
    def __init__(self, model: PI05Model, *, max_batch_size: int = 1, num_images: int = 3,
                 device: torch.device | str | None = None, use_cuda_graph: bool = True,
                 quantization: str | None = None) -> None:
        if max_batch_size <= 0 or num_images <= 0:
            raise ValueError("max_batch_size and num_images must be positive")
        self.model, self.cfg = model, model.config
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.max_batch_size, self.num_images = max_batch_size, num_images
        self.params_dtype = model.params_dtype
        tok_max = self.cfg.tokenizer_max_length
        self.lang_buckets = sorted({b for b in (16, 48, 112) if 0 < b < tok_max} | {tok_max})
        self.use_plan = (self.device.type == "cuda" and self.params_dtype == torch.bfloat16
                         and model.vision.compute_dtype == torch.bfloat16)
        self.use_cuda_graph = bool(use_cuda_graph) and self.use_plan
        self.plan: PI05Plan | None = None
        self.quantization = quantization          # None | "bf16" | "fp8_block" (see PI05Plan)
        self.graphs = CudaGraphRegistry()
        self.generator: torch.Generator | None = None

    def setup(self) -> None:
        if not self.use_plan:
            return
        import os

        from ... import ops

        ops.set_pdl(os.environ.get("PHYAI_PDL", "1") not in ("0", "false", "off"))
        self.plan = self._make_plan()
        self.plan.build_modulation_tables()

    def _make_plan(self) -> PI05Plan:
        return PI05Plan(self.model, max_batch_size=self.max_batch_size, num_images=self.num_images,
                        device=self.device, quantization=self.quantization)

    def _before_capture(self, bucket: int) -> None:
        """Called before the warm-up runs and the capture of a bucket's graph."""

    def _captured(self, bucket: int) -> None:
        """Called once after a bucket's graph has been captured, before its first replay."""

    def bucket_for(self, max_lang: int) -> int:
        for b in self.lang_buckets:
            if max_lang <= b:
                return b
        raise ValueError(f"prompt of {max_lang} tokens exceeds tokenizer_max_length={self.cfg.tokenizer_max_length}")

    def _validate(self, r: PI05Request) -> int:
        cfg = self.cfg
        B = r.pixel_values.shape[0]
        if not 1 <= B <= self.max_batch_size:
            raise ValueError(f"batch {B} outside [1, max_batch_size={self.max_batch_size}]")
        want = (B, self.num_images, cfg.vision.num_channels, cfg.vision.image_size, cfg.vision.image_size)
        if tuple(r.pixel_values.shape) != want:
            raise ValueError(f"pixel_values {tuple(r.pixel_values.shape)} != {want}")
        if tuple(r.input_ids.shape) != (B, cfg.tokenizer_max_length):
            raise ValueError(f"input_ids {tuple(r.input_ids.shape)} != {(B, cfg.tokenizer_max_length)}")
        if tuple(r.lang_lens.shape) != (B,):
            raise ValueError(f"lang_lens {tuple(r.lang_lens.shape)} != {(B,)}")
        if r.noise is not None and tuple(r.noise.shape) != (B, cfg.chunk_size, cfg.max_action_dim):
            raise ValueError(f"noise {tuple(r.noise.shape)} != {(B, cfg.chunk_size, cfg.max_action_dim)}")
        return B

    @torch.no_grad()
    def step(self, request: PI05Request) -> torch.Tensor:
        B = self._validate(request)
        cfg = self.cfg
        lens = tuple(int(v) for v in request.lang_lens.tolist())   # one tiny D2H read: the layout key
        if min(lens) < 0 or max(lens) > cfg.tokenizer_max_length:
            raise ValueError(f"lang_lens {lens} outside [0, {cfg.tokenizer_max_length}]")
        if not self.use_plan:
            return self._step_eager(request, lens)
        plan = self.plan
        if plan is None:
            raise RuntimeError("PI05WS1Scheduler.step called before setup()")
        bucket = self.bucket_for(max(lens))
        with event_scope("pi05.stage_inputs"):
            plan.set_layout(PI05Layout(B, lens, bucket))
            n = B * self.num_images
            plan.pixels[:n].copy_(request.pixel_values.reshape(n, *request.pixel_values.shape[2:]), non_blocking=True)
            plan.input_ids[:B].copy_(request.input_ids, non_blocking=True)
            if request.noise is None:
                plan.noise.normal_(generator=self.generator)
            else:
                plan.noise[:B].copy_(request.noise, non_blocking=True)
        with event_scope("pi05.forward"):
            if self.use_cuda_graph:
                g = self.graphs.get_or_create(bucket)
                if not g.captured:
                    self._before_capture(bucket)
                    g.capture(lambda: plan.run(bucket), {})
                    self._captured(bucket)
                g.replay()
            else:
                plan.run(bucket)
        return plan.out[:B].clone()

    def _step_eager(self, r: PI05Request, lens: tuple[int, ...]) -> torch.Tensor:
        dev, dt = self.device, self.params_dtype
        B = r.pixel_values.shape[0]
        noise = r.noise if r.noise is not None else torch.randn(B, self.cfg.chunk_size, self.cfg.max_action_dim,
                                                                 generator=self.generator)
        out = self.model.sample_actions(r.pixel_values.to(dev, dt), r.input_ids.to(dev), torch.tensor(lens),
                                        noise.to(dev, dt))
        return out.to(dt)

    def close(self) -> None:
        self.graphs.clear()
        self.plan = None


__all__ = ["PI05Request", "PI05WS1Scheduler"]
