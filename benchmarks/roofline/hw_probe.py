"""Measure the two roofline denominators on the visible GPU: copy bandwidth and bf16 GEMM throughput.

    python -m benchmarks.roofline.hw_probe [--out peaks.json]

The copy is a STREAM-style device-to-device ``copy_`` of 1 GiB (read + write counted); the GEMM is an
8192^3 bf16 cuBLAS matmul, timed as a burst (10 calls) and as a 2-second loop (the figure a kernel inside a
long step competes with: the 1 kW power cap lowers the clock). CUDA events after warm-up. If a
``MEASURED_PEAKS.json`` sits at the repository root its figures are returned by :func:`load_peaks`
instead, so every report of one build divides by the same numbers.
Reference counterpart: benchmark/pi05/hardware_probe.py:34-132.
"""

from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_peaks(path: str | Path | None = None) -> dict:
    """Measured peaks of this pool if the file exists, else the documented fallback figures."""
    p = Path(path) if path else ROOT / "MEASURED_PEAKS.json"
    peaks = dict(FALLBACK)
    if p.is_file():
        data = json.loads(p.read_text())
        peaks.update({k: v for k, v in data.items() if isinstance(v, (int, float))})
        peaks["source"] = str(p.name)
    return peaks


def _time(fn, n: int) -> float:
    import torch

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / n


def probe(device: str = "cuda:0", gemm_dim: int = 8192, copy_bytes: int = 1 << 30, sustained_s: float = 2.0) -> dict:
    import torch

    torch.cuda.set_device(device)
    src = torch.empty(copy_bytes, dtype=torch.uint8, device=device)
    dst = torch.empty_like(src)
    for _ in range(3):
        dst.copy_(src)
    copy_ms = _time(lambda: dst.copy_(src), 10)
    del src, dst
    a = torch.randn(gemm_dim, gemm_dim, device=device, dtype=torch.bfloat16)
    b = torch.randn(gemm_dim, gemm_dim, device=device, dtype=torch.bfloat16)
    for _ in range(3):
        a @ b
    burst_ms = _time(lambda: a @ b, 10)
    flop = 2.0 * gemm_dim ** 3
    n_loop = max(10, int(sustained_s * 1e3 / burst_ms))
    t0 = time.perf_counter()
    sustained_ms = _time(lambda: a @ b, n_loop)
    props = torch.cuda.get_device_properties(device)
    return {"device": props.name, "sms": props.multi_processor_count, "hbm_gbs": round(2 * copy_bytes / copy_ms / 1e6, 1),
            "bf16_tflops": round(flop / burst_ms / 1e9, 1), "bf16_tflops_sustained": round(flop / sustained_ms / 1e9, 1),
            "sustained_loop_s": round(time.perf_counter() - t0, 2), "source": "hw_probe"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args()
    res = probe(a.device)
    print(json.dumps(res))
    if a.out:
        Path(a.out).write_text(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
