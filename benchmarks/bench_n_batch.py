"""Latency / throughput of a policy plugin versus batch size.

    python benchmarks/bench_n_batch.py --model pi05 --batch-sizes 1 2 4 8 --n-warmup 5 --n-timed 30 [--jsonl out.jsonl]

For each batch size the engine is rebuilt (static buffers and CUDA graphs are sized by
``max_batch_size``), ``--n-warmup`` untimed steps run, then ``--n-timed`` steps are timed with one
CUDA-event pair each. Reported per batch size: mean / median / p50 / p90 / p99 / stdev / min / max
latency in ms and samples per second; one JSON line per batch size is appended to ``--jsonl``.
Inputs are synthetic (uniform pixels, a one-token or full-length prompt), weights random-init.

Reference: benchmark/bench_n_batch.py:84-441, bench_n_batch_ws1_pi0.py, bench_n_batch_ws1_pi05.py.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import statistics
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


@dataclasses.dataclass
class BenchResult:
    model: str
    batch_size: int
    n_timed: int
    mean_ms: float
    median_ms: float
    p50_ms: float
    p90_ms: float
    p99_ms: float
    stdev_ms: float
    min_ms: float
    max_ms: float
    samples_per_s: float

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self))


def percentile(xs, q):
    s = sorted(xs)
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


def summarize(model: str, bs: int, lat: list[float]) -> BenchResult:
    return BenchResult(model, bs, len(lat), statistics.fmean(lat), statistics.median(lat), percentile(lat, 0.5), percentile(lat, 0.9),
                       percentile(lat, 0.99), statistics.pstdev(lat) if len(lat) > 1 else 0.0, min(lat), max(lat),
                       bs / (statistics.median(lat) * 1e-3))


class NBatchBenchRunner:
    def __init__(self, model: str, *, device: str = "cuda:0", lang_len: int = 1, use_cuda_graph: bool = True,
                 impl: str = "ours") -> None:
        self.model, self.device, self.lang_len, self.use_cuda_graph = model, device, lang_len, use_cuda_graph
        self.impl = impl

    def build_reference(self, bs: int):
        """The unmodified reference package (installed under ``baseline/_ref``) through its own Engine and plugins,
        bf16 everywhere (its Pi0 plugin defaults the vision tower to fp32; both arms are timed in bf16)."""
        import os

        import torch

        # the reference's own knob: its default 128 MiB FlashInfer workspace overflows from batch 8 (Pi0.5) / batch 1 (Pi0)
        os.environ.setdefault("PHYAI_FLASHINFER_WORKSPACE_BYTES", str(1 << 30))
        sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "baseline" / "_ref"))
        from phyai.engine import Engine, EngineArgs
        from phyai.engine_config import DeviceConfig, EngineConfig, RuntimeConfig

        cfg = EngineConfig(device=DeviceConfig(target=self.device, params_dtype=torch.bfloat16),
                           runtime=RuntimeConfig(use_cuda_graph=self.use_cuda_graph))
        px = (torch.rand(bs, 3, 3, 224, 224, device=self.device) * 2 - 1).to(torch.bfloat16)
        noise = torch.randn(bs, 50, 32, device=self.device, dtype=torch.bfloat16)
        if self.model == "pi05":
            from phyai.models.pi05.main_pi05 import PI05Args
            from phyai.models.pi05.scheduler_ws1_pi05 import PI05Request

            eng = Engine(EngineArgs("pi05", PI05Args(checkpoint_dir=None, max_batch_size=bs, inputs_image_shape=[[224, 224, 3]] * 3), cfg))
            ids = torch.zeros(bs, 200, dtype=torch.long, device=self.device)
            ids[:, 0] = 2
            return eng, PI05Request(pixel_values=px, input_ids=ids, lang_lens=torch.full((bs,), self.lang_len, device=self.device), noise=noise)
        from phyai.models.pi0.main_pi0 import PI0Args
        from phyai.models.pi0.scheduler_ws1_pi0 import PI0Request

        eng = Engine(EngineArgs("pi0", PI0Args(checkpoint_dir=None, max_batch_size=bs, vision_params_dtype=torch.bfloat16), cfg))
        ids = torch.zeros(bs, 48, dtype=torch.long, device=self.device)
        ids[:, 0] = 2
        return eng, PI0Request(pixel_values=px, input_ids=ids, lang_lens=torch.full((bs,), min(self.lang_len, 48), device=self.device),
                               state=torch.randn(bs, 32, device=self.device, dtype=torch.bfloat16), noise=noise)

    def build(self, bs: int):
        import torch

        if self.impl == "reference":
            return self.build_reference(bs)
        from phyai_b200.engine import Engine, EngineArgs
        from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig

        cfg = EngineConfig(device=DeviceConfig(self.device, torch.bfloat16), runtime=RuntimeConfig(use_cuda_graph=self.use_cuda_graph))
        shape = [[224, 224, 3]] * 3
        if self.model == "pi05":
            from phyai_b200.models.pi05.main_pi05 import PI05Args
            from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request

            eng = Engine(EngineArgs("pi05", PI05Args(checkpoint_dir=None, max_batch_size=bs, inputs_image_shape=shape), cfg))
            ids = torch.zeros(bs, 200, dtype=torch.long, device=self.device)
            ids[:, 0] = 2
            req = PI05Request(pixel_values=torch.rand(bs, 3, 3, 224, 224, device=self.device) * 2 - 1, input_ids=ids,
                              lang_lens=torch.full((bs,), self.lang_len, device=self.device), noise=torch.randn(bs, 50, 32, device=self.device))
        elif self.model == "pi0":
            from phyai_b200.models.pi0.main_pi0 import PI0Args
            from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request

            eng = Engine(EngineArgs("pi0", PI0Args(checkpoint_dir=None, max_batch_size=bs, inputs_image_shape=shape), cfg))
            ids = torch.zeros(bs, 48, dtype=torch.long, device=self.device)
            ids[:, 0] = 2
            req = PI0Request(torch.rand(bs, 3, 3, 224, 224, device=self.device) * 2 - 1, ids, torch.full((bs,), min(self.lang_len, 48), device=self.device),
                             torch.randn(bs, 32, device=self.device), torch.randn(bs, 50, 32, device=self.device))
        else:
            raise SystemExit(f"unknown model {self.model!r}")
        return eng, req

    def run(self, bs: int, n_warmup: int, n_timed: int) -> BenchResult:
        import torch

        eng, req = self.build(bs)
        for _ in range(n_warmup):
            eng.step(req)
        torch.cuda.synchronize()
        lat = []
        for _ in range(n_timed):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step(req)
            e1.record()
            e1.synchronize()
            lat.append(e0.elapsed_time(e1))
        eng.close()
        return summarize(self.model if self.impl == "ours" else f"{self.model} (reference)", bs, lat)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", choices=("pi05", "pi0"), default="pi05")
    ap.add_argument("--batch-sizes", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--n-warmup", type=int, default=5)
    ap.add_argument("--n-timed", type=int, default=30)
    ap.add_argument("--lang-len", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--jsonl", type=str, default=None)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    a = ap.parse_args()
    runner = NBatchBenchRunner(a.model, lang_len=a.lang_len, use_cuda_graph=not a.no_graph, impl=a.impl)
    for bs in a.batch_sizes:
        t0 = time.time()
        r = runner.run(bs, a.n_warmup, a.n_timed)
        print(r.to_json(), f"# built+ran in {time.time() - t0:.1f}s", flush=True)
        if a.jsonl:
            with open(a.jsonl, "a") as f:
                f.write(r.to_json() + "\n")


if __name__ == "__main__":
    main()
