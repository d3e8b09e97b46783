"""Headline benchmark: Pi0.5 action-chunk latency (p50 / p99) at batch 1 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 serves one robot on one B200 through ``Engine(plugin="pi05")``. N > 1 (launched
under torchrun, one rank per GPU) serves N robots data-parallel through
``Engine(plugin="pi05_wn")``: per-GPU work is fixed (weak scaling) and the metric is
the latency of the whole N-robot step, max over ranks. Inputs are synthetic (uniform
pixels, uniform prompt ids of the full 200-token budget, N(0,1) noise) and weights are
random-init with the pi05_base geometry. The model runs in bf16.

Two measurements per run:
* ``value`` / ``ms_per_step``: device time of ``engine.step`` on device-resident
  inputs, one CUDA-event pair per step, L2 flushed (256 MiB write) between steps;
* ``e2e``: the same call fed from pinned host memory, including the host->device
  copies of that step's inputs and the device->host read of the action chunk.

A second block, ``cosmos3``, rides on the same JSON line: one guided denoise step of the
Cosmos3-Super geometry (7040 video + 512 text tokens, 40 blocks, guidance 7.0) over the N GPUs
of the run as a CFG x TP mesh (1: cfg1 x tp1, 2: cfg1 x tp2, 4: cfg1 x tp4, 8: cfg2 x tp4), i.e.
strong scaling of a fixed request, timed on the device between consecutive sampler updates,
max over ranks (``benchmarks/bench_cosmos3.py`` holds the measurement). ``--no-cosmos3`` skips it.

For N > 1 a third block, ``pi05_tp``, serves the headline request (one robot) with all N GPUs as one tensor-parallel
group (``Engine(plugin="pi05_tp")``): strong scaling of the batch-1 latency. The reference has no such scheduler.

``--impl reference`` runs the unmodified reference package installed under
``baseline/_ref`` through its own ``Engine`` / schedulers with the same requests.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
BASELINE_P50_MS = None  # the reference publishes no number for this metric


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--lang-len", type=int, default=200, help="real prompt tokens per robot")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--dtype", choices=("bf16", "fp8_block"), default="bf16",
                    help="fp8_block: prefix decoder and action expert in block-scaled fp8 (ours arm; not the headline dtype)")
    ap.add_argument("--no-cosmos3", action="store_true", help="skip the Cosmos3 TP / CFG block")
    ap.add_argument("--no-pi05-tp", action="store_true", help="skip the tensor-parallel Pi0.5 block (N > 1)")
    ap.add_argument("--cosmos3-model", default="super", help="geometry of the Cosmos3 block (super | nano | small)")
    ap.add_argument("--cosmos3-steps", type=int, default=6)
    ap.add_argument("--cosmos3-warmup", type=int, default=3)
    return ap.parse_args()


COSMOS3_LAYOUT = {1: (1, 1), 2: (1, 2), 4: (1, 4), 8: (2, 4)}   # n_gpus -> (cfg, tp)


def cosmos3_block(args: argparse.Namespace) -> dict:
    """The Cosmos3 denoise step of this run's arm over all N GPUs; a failure is reported, not raised."""
    import argparse as _ap

    if args.gpus not in COSMOS3_LAYOUT:
        return {"skipped": f"no CFG x TP layout for {args.gpus} GPUs (have {sorted(COSMOS3_LAYOUT)})"}
    try:
        from benchmarks.bench_cosmos3 import run_block

        cfg, tp = COSMOS3_LAYOUT[args.gpus]
        ns = _ap.Namespace(model=args.cosmos3_model, tp=tp, cfg=cfg, steps=args.cosmos3_steps, warmup=max(args.cosmos3_warmup, 3),
                           impl=args.impl, policy=False, batch=1, layers=0)
        rec = run_block(ns, keep_process_group=True)
        rec["scaling"] = "strong"
        return rec
    except Exception as e:  # noqa: BLE001 - the headline line must still be printed
        return {"error": f"{type(e).__name__}: {e}".replace("\n", " ")[:300]}


def pi05_tp_block(args: argparse.Namespace, device: str) -> dict:
    """The headline request (one robot, batch 1) served by ALL N GPUs as one tensor-parallel group: strong scaling of
    the latency, through ``Engine(plugin="pi05_tp")``. Device time per step, L2 flushed, p50, max over ranks."""
    import torch
    import torch.distributed as dist

    N = args.gpus
    if N == 1:
        return {"skipped": "one GPU: the headline value is this request"}
    if args.impl == "reference":
        return {"unavailable": "the reference ships no tensor-parallel Pi0.5 scheduler (single-GPU and data-parallel only)"}
    if args.dtype != "bf16":
        return {"skipped": "the tensor-parallel plan serves bf16"}
    try:
        from phyai_b200.engine import Engine, EngineArgs
        from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig, RuntimeConfig
        from phyai_b200.models.pi05.main_pi05_tp import PI05TPArgs
        from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request

        cfg = EngineConfig(device=DeviceConfig(target=device, params_dtype=torch.bfloat16),
                           parallel=ParallelConfig(world_size=N, tp_size=N), runtime=RuntimeConfig(use_cuda_graph=not args.no_graph))
        engine = Engine(EngineArgs("pi05_tp", PI05TPArgs(checkpoint_dir=None, max_batch_size=1, inputs_image_shape=[[224, 224, 3]] * 3), cfg))
        host = make_request_tensors(torch, 1, args.lang_len)            # the same request on every rank
        t = [x.to(device) for x in host]
        req = PI05Request(pixel_values=t[0], input_ids=t[1], lang_lens=t[2], noise=t[3])
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)
        for _ in range(max(args.warmup, 3)):
            out = engine.step(req)
        ms = []
        for _ in range(args.steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            e0.record()
            out = engine.step(req)
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        st = torch.tensor([percentile(ms, 0.5), percentile(ms, 0.99)], device=device, dtype=torch.float64)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        plan = engine.entry.scheduler.plan
        rec = {"metric": "pi05_action_chunk_latency_p50_ms", "value": round(float(st[0]), 4), "p99_ms": round(float(st[1]), 4), "unit": "ms",
               "parallelism": f"tp{N}", "scaling": "strong", "global_batch": 1, "steps": args.steps,
               "plan": type(plan).__name__, "expert": "whole on every rank" if getattr(plan, "expert_replicated", True) else "sharded",
               "finite": bool(torch.isfinite(out.float()).all().item()), "abs_mean": round(float(out.float().abs().mean().item()), 6)}
        engine.close()
        del engine, flush
        torch.cuda.empty_cache()
        return rec
    except Exception as e:  # noqa: BLE001 - the headline line must still be printed
        return {"error": f"{type(e).__name__}: {e}".replace("\n", " ")[:300]}


def percentile(xs: list[float], q: float) -> float:
    s = sorted(xs)
    if not s:
        return float("nan")
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.path = index, None, None

    def start(self) -> None:
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in Path(self.path).read_text().strip().splitlines() if r.strip()]
            sm = [float(r[0]) for r in rows if len(r) >= 7]
            if sm:
                out["sm_mhz"] = statistics.median(sm)
                out["sm_max_mhz"] = float(rows[0][1])
                out["power_w_max"] = max(float(r[2]) for r in rows if len(r) >= 7)
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for i, n in enumerate(names):
                    if any(r[3 + i].strip().lower().startswith("active") for r in rows if len(r) >= 7):
                        out["reasons"].append(n)
                out["samples"] = len(sm)
            os.unlink(self.path)
        except Exception:
            pass
        return out


def make_request_tensors(torch, n_robots: int, lang_len: int, seed: int = 0):
    """Pinned-host synthetic inputs of the pi05_base shapes."""
    g = torch.Generator().manual_seed(seed)
    pix = (torch.rand(n_robots, 3, 3, 224, 224, generator=g) * 2 - 1).to(torch.bfloat16)
    ids = torch.zeros(n_robots, 200, dtype=torch.int64)
    ids[:, :lang_len] = torch.randint(1, 257152, (n_robots, lang_len), generator=g)
    lens = torch.full((n_robots,), lang_len, dtype=torch.int64)
    noise = torch.randn(n_robots, 50, 32, generator=g).to(torch.bfloat16)
    return [t.pin_memory() for t in (pix, ids, lens, noise)]


def run(args: argparse.Namespace) -> dict:
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    N = args.gpus
    if N > 1 and not dist.is_initialized():
        # one process group for the whole run: the engines and the Cosmos3 block find it initialised and leave it alone
        if args.impl == "reference":
            dist.init_process_group("nccl", device_id=torch.device(device))
        else:
            from phyai_b200.parallel.dist import init_dist

            init_dist(N, "cuda")

    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        from phyai.engine import Engine, EngineArgs
        from phyai.engine_config import DeviceConfig, EngineConfig, ParallelConfig, RuntimeConfig
        from phyai.models.pi05.main_pi05 import PI05Args
        from phyai.models.pi05.main_pi05_wn import PI05WNArgs
        from phyai.models.pi05.scheduler_ws1_pi05 import PI05Request
        launch_count = lambda: 0  # noqa: E731
    else:
        from phyai_b200 import ops
        from phyai_b200.engine import Engine, EngineArgs
        from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig, RuntimeConfig
        from phyai_b200.models.pi05.main_pi05 import PI05Args
        from phyai_b200.models.pi05.main_pi05_wn import PI05WNArgs
        from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request
        launch_count = ops.launch_counter

    cfg = EngineConfig(device=DeviceConfig(target=device, params_dtype=torch.bfloat16),
                       parallel=ParallelConfig(world_size=N, dp_size=N),
                       runtime=RuntimeConfig(use_cuda_graph=not args.no_graph))
    shape = [[224, 224, 3]] * 3
    qkw = {}
    if args.dtype == "fp8_block":
        if args.impl == "reference":
            # the reference reads its quantisation from a checkpoint's config; this benchmark builds random weights in memory
            raise RuntimeError("the reference arm serves fp8 only from an fp8 checkpoint on disk; none is generated here")
        qkw = {"quantization": "fp8_block"}
    if N == 1:
        engine = Engine(EngineArgs("pi05", PI05Args(checkpoint_dir=None, max_batch_size=1, inputs_image_shape=shape, **qkw), cfg))
    else:
        engine = Engine(EngineArgs("pi05_wn", PI05WNArgs(checkpoint_dir=None, max_batch_size=N,
                                                         inputs_image_shape=shape, **qkw), cfg))

    host = make_request_tensors(torch, N, args.lang_len)
    dev_in = [t.to(device) for t in host]
    req_dev = PI05Request(pixel_values=dev_in[0], input_ids=dev_in[1], lang_lens=dev_in[2], noise=dev_in[3])
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_dev():
        return engine.step(req_dev)

    def step_e2e():
        moved = [t.to(device, non_blocking=True) for t in host]
        out = engine.step(PI05Request(pixel_values=moved[0], input_ids=moved[1], lang_lens=moved[2], noise=moved[3]))
        return out.to("cpu")  # device -> host read of the action chunk (synchronises)

    for _ in range(max(args.warmup, 3)):
        step_dev()
    barrier()
    # kernels per step: count one eager pass of the same request (graph replays do not tick the host counter)
    per_step_launches = 0
    if args.impl == "ours":
        sched = engine.entry.scheduler
        local = getattr(sched, "local", sched)
        if local.plan is not None:
            c0 = launch_count()
            local.plan.run(local.bucket_for(args.lang_len))
            torch.cuda.synchronize()
            per_step_launches = launch_count() - c0
    barrier()

    sampler = ClockSampler(local_rank)
    sampler.start()
    lat_ms: list[float] = []
    barrier()
    t_region0 = time.perf_counter()
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if N > 1:
            dist.barrier()
        e0.record()
        step_dev()
        e1.record()
        e1.synchronize()
        lat_ms.append(e0.elapsed_time(e1))
    barrier()
    region_s = time.perf_counter() - t_region0
    clocks = sampler.stop()

    e2e_ms: list[float] = []
    for _ in range(2):
        step_e2e()
    barrier()
    for _ in range(args.steps):
        flush.zero_()
        barrier()
        t0 = time.perf_counter()
        step_e2e()
        e2e_ms.append((time.perf_counter() - t0) * 1e3)
    barrier()

    stats = torch.tensor([percentile(lat_ms, 0.5), percentile(lat_ms, 0.99), statistics.fmean(lat_ms),
                          percentile(e2e_ms, 0.5), percentile(e2e_ms, 0.99)], device=device, dtype=torch.float64)
    if N > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    p50, p99, mean, e50, e99 = (float(v) for v in stats.tolist())
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = N * 50 * 32 * 2
    last = step_dev().float()
    finite = bool(torch.isfinite(last).all().item())
    checksum = float(last.abs().mean().item())
    if not finite:
        raise RuntimeError("the action chunk holds non-finite values")
    result = {
        "metric": "pi05_action_chunk_latency_p50_ms", "value": round(p50, 4), "unit": "ms", "n_gpus": N,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(mean, 4),
        "higher_is_better": False, "scaling": "weak",
        "vs_baseline": (p50 / BASELINE_P50_MS) if BASELINE_P50_MS else None,
        "dtype": args.dtype, "data": "synthetic (uniform pixels, uniform prompt ids, N(0,1) noise; random-init weights)",
        "impl": args.impl, "p99_ms": round(p99, 4), "samples_per_s": round(N / (p50 * 1e-3), 2),
        "config": {"model": "pi05_base geometry (SigLIP-So400m + Gemma-2B prefix + Gemma-300M expert)",
                   "global_batch": N, "per_gpu_batch": 1, "seq_len": 768 + args.lang_len, "prompt_tokens": args.lang_len,
                   "cameras": 3, "denoise_steps": 10, "action_chunk": [50, 32],
                   "parallelism": "single" if N == 1 else f"dp{N}", "cuda_graph": not args.no_graph,
                   "l2": "flushed between timed steps (256 MiB write)"},
        "clocks": clocks,
        "e2e": {"value": round(e50, 4), "unit": "ms", "p99_ms": round(e99, 4), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": int(per_step_launches * args.steps),
        "gpu_launches_per_step": int(per_step_launches),
        "timed_region_s": round(region_s, 3),
        "output": {"finite": finite, "abs_mean": round(checksum, 6)},
    }
    engine.close()
    del engine, req_dev, dev_in, flush
    torch.cuda.empty_cache()
    if not args.no_pi05_tp:
        result["pi05_tp"] = pi05_tp_block(args, device)
    if not args.no_cosmos3:
        result["cosmos3"] = cosmos3_block(args)
    if N > 1 and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


def main() -> None:
    args = parse_args()
    if args.impl == "reference" and not (ROOT / "baseline" / "_ref" / "phyai").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    try:
        res = run(args)
    except SystemExit:
        raise
    except Exception as e:  # noqa: BLE001
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                msg = f"{type(e).__name__}: {e}".replace("\n", " ")[:300]
                print(json.dumps({"impl": "reference", "unavailable": msg}))
            return
        raise
    if res:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
