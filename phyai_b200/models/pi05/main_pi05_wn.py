"""Plugin ``pi05_wn``: data-parallel Pi0.5 (one replica per GPU).

``max_batch_size`` is the total over all ranks; each rank serves
``ceil(max_batch_size / dp)`` robots (reference: phyai/src/phyai/models/pi05/main_pi05_wn.py:42-138).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from ...engine import Engine, EntryArgs
from ...engine_config import get_engine_config
from .main_pi05 import PI05Args, PI05Entry, resolve_num_images
from .scheduler_wn_pi05 import PI05WNScheduler
from .scheduler_ws1_pi05 import PI05Request, PI05WS1Scheduler


@dataclass
class PI05WNArgs(PI05Args):
    pass


@Engine.register
class PI05WNEntry(PI05Entry):
    name: ClassVar[str] = "pi05_wn"
    args_cls: ClassVar[type[EntryArgs]] = PI05WNArgs

    def setup(self, args: PI05WNArgs) -> None:  # type: ignore[override]
        eng = get_engine_config()
        dp = eng.parallel.dp_size
        per_rank = -(-args.max_batch_size // dp)
        self.model = self.build_model(args)
        n_img = resolve_num_images(args.inputs_image_shape, self.model.config.vision.num_channels)
        local = PI05WS1Scheduler(self.model, max_batch_size=per_rank, num_images=n_img, device=eng.device.target,
                                 use_cuda_graph=eng.runtime.use_cuda_graph, quantization=args.quantization)
        self.scheduler = PI05WNScheduler(local, device=eng.device.target)
        self.scheduler.setup()

    def step(self, request: PI05Request | None) -> torch.Tensor:  # type: ignore[override]
        if self.scheduler is None:
            raise RuntimeError("PI05WNEntry.step before setup")
        return self.scheduler.step(request)


__all__ = ["PI05WNArgs", "PI05WNEntry"]
