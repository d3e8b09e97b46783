"""Data-parallel Pi0: one replica per GPU, rank 0 scatters the batch (pixels, prompt ids, state, noise) and gathers the actions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 examples/pi0/run_pi0_wn.py
"""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig  # noqa: E402
from phyai_b200.models.pi0.main_pi0_wn import PI0WNArgs  # noqa: E402
from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request  # noqa: E402


def main() -> None:
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    cfg = EngineConfig(device=DeviceConfig(dev, torch.bfloat16), parallel=ParallelConfig(world_size=world, dp_size=world))
    engine = Engine(EngineArgs("pi0_wn", PI0WNArgs(checkpoint_dir=None, max_batch_size=world, inputs_image_shape=[[224, 224, 3]] * 3), cfg))
    req = None
    if rank == 0:   # only the router rank holds the request; the others receive their share
        req = PI0Request(pixel_values=torch.rand(world, 3, 3, 224, 224, device=dev) * 2 - 1,
                         input_ids=torch.randint(0, 1000, (world, 48), device=dev), lang_lens=torch.full((world,), 48, device=dev),
                         state=torch.randn(world, 32, device=dev, dtype=torch.bfloat16),
                         noise=torch.randn(world, 50, 32, device=dev, dtype=torch.bfloat16))
    for _ in range(5):
        out = engine.step(req)
    if rank == 0:
        print("actions for", out.shape[0], "robots:", tuple(out.shape))
    engine.close()


if __name__ == "__main__":
    main()
