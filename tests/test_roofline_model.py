"""FLOP / traffic models behind the roofline reports (pure Python, no GPU)."""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from benchmarks.roofline import flops, hw_probe  # noqa: E402


def test_stage_arithmetic():
    s = flops.Stage("s").gemm(10, 20, 30, count=2).attn(4, 8, 2, 16, count=3, kv_heads=1)
    assert s.flops == 2 * 2 * 10 * 20 * 30 + 3 * 4 * 4 * 8 * 2 * 16
    assert s.weight_bytes == 2 * 20 * 30 * 2
    assert s.bytes == s.weight_bytes + 2 * (10 * 30 + 10 * 20) * 2 + 3 * 2 * 8 * 1 * 16 * 2
    peaks = {"hbm_gbs": 1.0, "bf16_tflops": 1e-3}
    assert s.bound(peaks) in ("compute", "memory") and s.roofline_ms(peaks) > 0


def test_pi05_model_matches_known_sizes():
    from phyai_b200.models.pi05.configuration_pi05 import PI05Config

    vision, prefix, expert = flops.pi05_stages(PI05Config(), batch=1, num_images=3, lang_tokens=48)
    # SigLIP-So400m blocks: about 0.4 G parameters; Gemma-2B decoder blocks: about 1.9 G; Gemma-300M expert read 10 times
    assert 0.39e9 < vision.weight_bytes / 2 < 0.43e9
    assert 1.8e9 < prefix.weight_bytes / 2 < 2.0e9
    assert 3.0e9 < expert.weight_bytes / 2 < 3.2e9
    peaks = hw_probe.load_peaks()
    assert vision.bound(peaks) == "compute" and expert.bound(peaks) == "memory"
    twice = flops.pi05_stages(PI05Config(), batch=2, num_images=3, lang_tokens=48)
    assert abs(twice[1].flops / prefix.flops - 2.0) < 1e-6           # products and attention both scale with the batch


def test_report_and_renderers():
    from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config

    stages = flops.pi05_stages(tiny_pi05_config(), 1, 2, 16)
    rows = flops.report(stages, {"vision": 0.01, "prefix": 0.02}, {"hbm_gbs": 6000.0, "bf16_tflops": 1500.0})
    assert [r["stage"] for r in rows] == ["vision", "prefix", "expert"] and rows[2]["measured_ms"] is None
    assert 0 < rows[0]["frac_of_roofline"] < 1
    md = flops.to_markdown(rows)
    assert md.count("\n") == len(rows) + 1 and "–" in md
    svg = flops.to_svg(rows, "title")
    assert svg.startswith("<svg") and svg.count("<rect") == 4
