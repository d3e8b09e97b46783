"""Cosmos3 policy request: per-phase latency against the roofline, over a batch sweep.

    python -m benchmarks.roofline.profile_cosmos3_policy --model nano --batches 1 2 4 8 --out-dir out/roofline_c3

Each batch size runs ``benchmarks/bench_cosmos3.py --policy`` in a child process (so every size starts from a clean
allocator) and reads its JSON line: the median denoise step (CUDA events) and the whole request. The request splits into
``denoise = steps x step`` and ``conditioning + text prefill + decode = request - denoise``; the denoise step is put
against the FLOP / traffic model of the generation tower. ``--impl reference`` profiles the unmodified reference the
same way. Reference counterpart: benchmark/cosmos3_policy/profile_cosmos3_policy.py (driver run.sh:49-62).
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from benchmarks.roofline import flops, hw_probe  # noqa: E402


def run_one(model: str, batch: int, steps: int, warmup: int, impl: str) -> dict:
    cmd = [sys.executable, str(ROOT / "benchmarks" / "bench_cosmos3.py"), "--model", model, "--policy", "--batch", str(batch),
           "--steps", str(steps), "--warmup", str(warmup), "--impl", impl]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1800)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{") and '"metric"' in ln]
    if r.returncode != 0 or not lines:
        raise RuntimeError(f"{' '.join(cmd)} failed:\n{(r.stdout + r.stderr)[-2000:]}")
    return json.loads(lines[-1])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="nano")
    ap.add_argument("--batches", type=int, nargs="+", default=[1])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--out-dir", default=None)
    a = ap.parse_args()

    from benchmarks.bench_cosmos3 import GEOMETRY
    from phyai_b200.models.cosmos3.configuration_cosmos3 import Cosmos3Config

    peaks = hw_probe.load_peaks()
    results, md = [], []
    for b in a.batches:
        m = run_one(a.model, b, a.steps, a.warmup, a.impl)
        geo = dict(GEOMETRY[a.model]["cfg"])
        if m.get("layers"):
            geo["num_hidden_layers"] = m["layers"]
        cfg = Cosmos3Config(**geo)
        stage = flops.cosmos3_step_stages(cfg, m["tokens"], m.get("text_tokens", 0), b, guided=m.get("guidance", 0) not in (0, 1.0))
        rows = flops.report(stage, {"gen_tower_step": m["value"]}, peaks)
        n_steps = m["steps"] + m["warmup"]            # denoise steps of the one request the benchmark runs
        other = None if not m.get("request_ms") else round(m["request_ms"] - n_steps * m.get("mean_ms", m["value"]), 2)
        results.append({"batch": b, "impl": a.impl, "step_ms": m["value"], "request_ms": m.get("request_ms"),
                        "outside_denoise_ms": other, "rows": rows, "denoise_steps": n_steps})
        md.append(f"### {a.model} policy, batch {b}, {a.impl} (request {m.get('request_ms')} ms)\n\n" + flops.to_markdown(rows))
        if a.out_dir:
            Path(a.out_dir).mkdir(parents=True, exist_ok=True)
            (Path(a.out_dir) / f"cosmos3_policy_b{b}_{a.impl}.svg").write_text(
                flops.to_svg(rows, f"Cosmos3 {a.model} policy batch {b} ({a.impl}): denoise step vs roofline"))
    text = "\n\n".join(md)
    print(text)
    if a.out_dir:
        (Path(a.out_dir) / f"cosmos3_policy_{a.impl}.json").write_text(json.dumps({"peaks": peaks, "results": results}, indent=1))
        (Path(a.out_dir) / f"cosmos3_policy_{a.impl}.md").write_text(text + "\n")


if __name__ == "__main__":
    main()
