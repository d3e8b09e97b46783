"""Pi0.5 per-stage latency against the roofline, over a batch sweep.

    python -m benchmarks.roofline.profile_pi05 --batches 1 2 4 8 --out-dir out/roofline_pi05

For every batch size: vision / prefix / expert / whole-request medians (``benchmarks/bench_pi05_stages.py``:
one CUDA graph per stage, CUDA events, L2 flushed before every replay) joined with the FLOP and traffic model of
``benchmarks/roofline/flops.py`` and the measured peaks (``MEASURED_PEAKS.json`` or ``hw_probe``). Writes
``pi05_roofline.json``, ``pi05_roofline.md`` and one SVG bar chart per batch size; prints the markdown.
Reference counterpart: benchmark/pi05/profile_pi05.py and plot_pi05.py (driver: benchmark/pi05/run.sh).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from benchmarks.roofline import flops, hw_probe  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batches", type=int, nargs="+", default=[1])
    ap.add_argument("--lang-len", type=int, default=48)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="base", choices=["base", "tiny"])
    ap.add_argument("--probe", action="store_true", help="measure the peaks on this GPU instead of reading the recorded ones")
    ap.add_argument("--out-dir", default=None)
    a = ap.parse_args()

    from benchmarks.bench_pi05_stages import measure_stages
    from phyai_b200.models.pi05.configuration_pi05 import PI05Config, tiny_pi05_config

    peaks = hw_probe.probe() if a.probe else hw_probe.load_peaks()
    cfg = PI05Config() if a.model == "base" else tiny_pi05_config()
    results, md = [], []
    for b in a.batches:
        m = measure_stages(b, a.steps, a.warmup, a.lang_len, a.model)
        stages = flops.pi05_stages(cfg, b, 3, m["lang_bucket"])
        rows = flops.report(stages, m["median_ms"], peaks)
        total = sum(s.roofline_ms(peaks) for s in stages)
        rows.append({"stage": "request", "gflop": round(sum(s.flops for s in stages) / 1e9, 2),
                     "weights_mb": round(sum(s.weight_bytes for s in stages) / 1e6, 1),
                     "traffic_mb": round(sum(s.bytes for s in stages) / 1e6, 1), "bound": "sum of stages", "roofline_ms": round(total, 4),
                     "measured_ms": m["median_ms"]["request"], "frac_of_roofline": round(total / m["median_ms"]["request"], 3),
                     "tflops": None, "gbs": None})
        results.append({"batch": b, "lang_bucket": m["lang_bucket"], "rows": rows})
        md.append(f"### batch {b} (peaks: {peaks['source']})\n\n" + flops.to_markdown(rows))
        if a.out_dir:
            Path(a.out_dir).mkdir(parents=True, exist_ok=True)
            (Path(a.out_dir) / f"pi05_roofline_b{b}.svg").write_text(flops.to_svg(rows, f"Pi0.5 batch {b}: measured vs roofline"))
    text = "\n\n".join(md)
    print(text)
    if a.out_dir:
        (Path(a.out_dir) / "pi05_roofline.json").write_text(json.dumps({"peaks": peaks, "results": results}, indent=1))
        (Path(a.out_dir) / "pi05_roofline.md").write_text(text + "\n")


if __name__ == "__main__":
    main()
