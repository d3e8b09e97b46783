"""Single-GPU Pi0 scheduler (reference: phyai/src/phyai/models/pi0/scheduler_ws1_pi0.py:39-578).

Same structure as the Pi0.5 scheduler: one CUDA graph per prompt-length bucket covering
vision, prefix and the whole Euler loop; metadata rewritten only when the request shape
changes. The reference rebuilds its metadata (with host syncs) every step and replays ten
per-step graphs from Python.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ...utils.profile import event_scope
from ..pi05.plan_pi05 import PI05Layout
from ..pi05.scheduler_ws1_pi05 import PI05WS1Scheduler
from .modeling_pi0 import PI0Model
from .plan_pi0 import PI0Plan


@dataclass
class PI0Request:
    pixel_values: torch.Tensor        # (B, n_img, C, H, W)
    input_ids: torch.Tensor           # (B, tokenizer_max_length) int64
    lang_lens: torch.Tensor           # (B,) int64
    state: torch.Tensor               # (B, max_state_dim)
    noise: torch.Tensor | None = None  # (B, chunk, action_dim)


class PI0WS1Scheduler(PI05WS1Scheduler):
    def setup(self) -> None:
        if not self.use_plan:
            return
        import os

        from ... import ops

        ops.set_pdl(os.environ.get("PHYAI_PDL", "1") not in ("0", "false", "off"))
        self.plan = PI0Plan(self.model, max_batch_size=self.max_batch_size, num_images=self.num_images,
                            device=self.device, quantization=getattr(self, "quantization", None))
        self.plan.build_modulation_tables()

    def _validate(self, r: PI0Request) -> int:  # type: ignore[override]
        B = super()._validate(r)
        if tuple(r.state.shape) != (B, self.cfg.max_state_dim):
            raise ValueError(f"state {tuple(r.state.shape)} != {(B, self.cfg.max_state_dim)}")
        return B

    @torch.no_grad()
    def step(self, request: PI0Request) -> torch.Tensor:  # type: ignore[override]
        if self.use_plan and self.plan is not None:
            B = request.pixel_values.shape[0]
            self.plan.state[:B].copy_(request.state, non_blocking=True)
        return super().step(request)

    def _step_eager(self, r: PI0Request, lens) -> torch.Tensor:  # type: ignore[override]
        dev, dt = self.device, self.params_dtype
        B = r.pixel_values.shape[0]
        noise = r.noise if r.noise is not None else torch.randn(B, self.cfg.chunk_size, self.cfg.max_action_dim,
                                                                 generator=self.generator)
        out = self.model.sample_actions(r.pixel_values.to(dev, dt), r.input_ids.to(dev), torch.tensor(lens),
                                        r.state.to(dev, dt), noise.to(dev, dt))
        return out.to(dt)


__all__ = ["PI0Request", "PI0WS1Scheduler"]
