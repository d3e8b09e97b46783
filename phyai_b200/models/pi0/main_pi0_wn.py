"""Plugin ``pi0_wn``: data-parallel Pi0 (one replica per GPU, rank 0 routes the batch).

Same routing as the Pi0.5 data-parallel plugin (no header exchange, one grouped point-to-point launch
per step that rank 0 does not wait for, gather of the action chunks); a Pi0 request carries one more tensor, the state vector.
The reference ships data parallelism for Pi0.5 only (phyai/src/phyai/models/pi05/main_pi05_wn.py:42-138);
its Pi0 batch sweep runs on one GPU (benchmark/bench_n_batch_ws1_pi0.py).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from ...engine import Engine, EntryArgs
from ...engine_config import get_engine_config
from ..pi05.scheduler_wn_pi05 import PI05WNScheduler
from .main_pi0 import PI0Args, PI0Entry
from .scheduler_ws1_pi0 import PI0Request


class PI0WNScheduler(PI05WNScheduler):
    def _shapes(self):
        px, ids, lens, nz = super()._shapes()
        return [px, ids, lens, ((self.per_rank_B, self.cfg.max_state_dim), None), nz]

    def _pack(self, request: PI0Request, real_B: int):
        px, ids, lens, nz = super()._pack(request, real_B)
        return [px, ids, lens, request.state.to(self.device, self.dtype), nz]

    def _unpack(self, tensors):
        return PI0Request(*tensors)


@dataclass
class PI0WNArgs(PI0Args):
    pass


@Engine.register
class PI0WNEntry(PI0Entry):
    name: ClassVar[str] = "pi0_wn"
    args_cls: ClassVar[type[EntryArgs]] = PI0WNArgs

    def setup(self, args: PI0WNArgs) -> None:  # type: ignore[override]
        dp = get_engine_config().parallel.dp_size
        local = self.build_local(args, -(-args.max_batch_size // dp))
        self.scheduler = PI0WNScheduler(local, device=get_engine_config().device.target)
        self.scheduler.setup()

    def step(self, request: PI0Request | None) -> torch.Tensor:  # type: ignore[override]
        if self.scheduler is None:
            raise RuntimeError("PI0WNEntry.step before setup")
        return self.scheduler.step(request)


__all__ = ["PI0WNArgs", "PI0WNEntry", "PI0WNScheduler"]
