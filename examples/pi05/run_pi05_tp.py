"""Tensor-parallel Pi0.5: every rank holds a shard of each decoder projection and receives the same request. On CUDA
bf16 the request runs as one captured graph whose row-parallel GEMMs store into the peers' memory (``PI05TPPlan``); the
single-GPU plan stays the low-latency default at batch 1, this plugin is for checkpoints that should not be replicated.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/pi05/run_pi05_tp.py
"""

import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig  # noqa: E402
from phyai_b200.models.pi05.main_pi05_tp import PI05TPArgs  # noqa: E402
from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request  # noqa: E402


def main() -> None:
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    cfg = EngineConfig(device=DeviceConfig(dev, torch.bfloat16), parallel=ParallelConfig(world_size=world, tp_size=world))
    engine = Engine(EngineArgs("pi05_tp", PI05TPArgs(checkpoint_dir=None, max_batch_size=1, inputs_image_shape=[[224, 224, 3]] * 3,
                                                     shard_expert=os.environ.get("PI05_TP_SHARD_EXPERT", "0") == "1"), cfg))
    g = torch.Generator().manual_seed(0)                     # the same request on every rank
    req = PI05Request(pixel_values=(torch.rand(1, 3, 3, 224, 224, generator=g) * 2 - 1).to(dev, torch.bfloat16),
                      input_ids=torch.randint(0, 1000, (1, 200), generator=g).to(dev), lang_lens=torch.tensor([200], device=dev),
                      noise=torch.randn(1, 50, 32, generator=g).to(dev, torch.bfloat16))
    import json
    import statistics

    import torch.distributed as dist

    out = engine.step(req)
    for _ in range(2):
        engine.step(req)
    ms = []
    for _ in range(int(os.environ.get("PI05_TP_TIMED_STEPS", "8"))):
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step(req)
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ms)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)       # the slowest rank defines the latency
    if rank == 0:
        print(json.dumps({"plugin": "pi05_tp", "tp": world, "p50_ms_max_over_ranks": round(float(t), 3), "steps": len(ms),
                          "action_chunk": list(out.shape), "finite": bool(torch.isfinite(out.float()).all()),
                          "path": type(engine.entry.scheduler.plan).__name__,
                          "expert": "whole on every rank" if getattr(engine.entry.scheduler.plan, "expert_replicated", True) else "sharded"}))
    engine.close()


if __name__ == "__main__":
    main()
