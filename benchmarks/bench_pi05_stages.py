"""Where a Pi0.5 action chunk spends its time: vision tower, prefix prefill, action expert.

Each stage of :class:`phyai_b200.models.pi05.plan_pi05.PI05Plan` is captured in a CUDA graph of
its own and replayed between CUDA events; the whole request (one graph, as the scheduler runs it)
is timed the same way. An L2 flush (a write larger than the cache) runs before every timed replay.
Prints one JSON line. Synthetic pixels / ids / noise, random-init weights, bf16.

    python benchmarks/bench_pi05_stages.py --batch 1 --steps 20 --warmup 3
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def measure_stages(batch: int = 1, steps: int = 20, warmup: int = 3, lang_len: int = 48, model: str = "base") -> dict:
    """Median milliseconds of each stage (and of the whole request) for one batch size; see the module docstring."""
    a = argparse.Namespace(batch=batch, steps=steps, warmup=warmup, lang_len=lang_len, model=model)
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi05.configuration_pi05 import PI05Config, tiny_pi05_config
    from phyai_b200.models.pi05.main_pi05 import PI05Args
    from phyai_b200.models.pi05.plan_pi05 import PI05Layout
    from phyai_b200.runtime.cuda_graph_manager import CudaGraph

    dev = torch.device("cuda:0")
    cfg = PI05Config() if a.model == "base" else tiny_pi05_config()
    side = cfg.vision.image_size
    ec = EngineConfig(device=DeviceConfig("cuda:0", torch.bfloat16), runtime=RuntimeConfig(use_cuda_graph=True))
    eng = Engine(EngineArgs("pi05", PI05Args(config=cfg, max_batch_size=a.batch, random_init_seed=0,
                                             inputs_image_shape=[[side, side, 3]] * 3), ec))
    sched = eng.entry.scheduler
    plan = sched.plan
    B = a.batch
    bucket = sched.bucket_for(a.lang_len)
    plan.set_layout(PI05Layout(B, (a.lang_len,) * B, bucket))
    plan.pixels.uniform_(-1, 1)
    plan.input_ids.random_(0, cfg.text.vocab_size)
    plan.noise.normal_()

    stages = {"vision": plan.vision, "prefix": lambda: plan.prefix(bucket), "expert": plan.expert,
              "request": lambda: plan.run(bucket)}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out: dict[str, float] = {}
    for name, fn in stages.items():
        g = CudaGraph()
        g.capture(fn, {})
        for _ in range(a.warmup):
            g.replay()
        ts = []
        for _ in range(a.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        out[name] = round(statistics.median(ts), 4)
    eng.close()
    return {"bench": "pi05_stages", "batch": B, "lang_bucket": bucket, "model": a.model, "median_ms": out, "steps": a.steps,
            "warmup": a.warmup, "l2": "flushed before every replay", "dtype": "bf16", "data": "synthetic"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lang-len", type=int, default=48)
    ap.add_argument("--model", default="base", choices=["base", "tiny"])
    a = ap.parse_args()
    print(json.dumps(measure_stages(a.batch, a.steps, a.warmup, a.lang_len, a.model)))


if __name__ == "__main__":
    main()
