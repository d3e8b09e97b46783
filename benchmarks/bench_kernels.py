"""Micro-benchmarks of this repository's kernels against library baselines, with roofline fractions.

    python benchmarks/bench_kernels.py [--set gemm|attention|norm|fp8|nvfp4|all] [--peaks MEASURED_PEAKS.json]

GEMMs are compared with ``torch.matmul`` (cuBLAS), attention with ``scaled_dot_product_attention``
and, when importable, FlashInfer / flash-attn; norms with an eager PyTorch expression. Each timing is
the mean over 10 launches after 3 warm-up launches, CUDA events on the launching stream; operands are
larger than L2 for the big shapes. Fractions are of the measured peaks in the json (copy bandwidth
and cuBLAS bf16), not of nominal figures.

Reference: phyai-kernel/benchmark/bench_rmsnorm.py, bench_adarmsnorm.py.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def bench(fn, n=10, warm=3):
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / n


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--set", default="all", choices=("gemm", "attention", "norm", "fp8", "nvfp4", "all"))
    ap.add_argument("--only", default=None, help="run a single named shape (for profiler captures)")
    ap.add_argument("--no-baselines", action="store_true", help="skip the library kernels (keeps a profiler capture small)")
    ap.add_argument("--gemm-2cta", action="store_true", help="also time the CTA-pair (cta_group::2) GEMM kernel")
    ap.add_argument("--peaks", default=str(Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"))
    a = ap.parse_args()
    import torch

    from phyai_b200 import ops

    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    if Path(a.peaks).is_file():
        peaks.update({k: v for k, v in json.loads(Path(a.peaks).read_text()).items() if isinstance(v, (int, float))})
    dev, bf = "cuda", torch.bfloat16
    rows = []
    if a.set in ("gemm", "all"):
        shapes = {"pi05.prefix.qkv": (968, 2048, 2560), "pi05.prefix.gate_up": (968, 2048, 32768), "pi05.prefix.down": (968, 16384, 2048),
                  "pi05.expert.qkv": (50, 1024, 2560), "pi05.expert.gate_up": (50, 1024, 8192), "cosmos3.qkv": (7040, 5120, 7168),
                  "cosmos3.gate_up": (7040, 5120, 27648), "cosmos3.down": (7040, 13824, 5120)}
        for name, (M, K, N) in shapes.items():
            if a.only and name != a.only:
                continue
            x, w = torch.randn(M, K, device=dev, dtype=bf) * 0.1, torch.randn(N, K, device=dev, dtype=bf) * 0.1
            out = torch.empty(M, N, device=dev, dtype=bf)
            t_o = bench(lambda: ops.gemm(x, w, out))
            t_c = float("nan") if a.no_baselines else bench(lambda: torch.matmul(x, w.t()))
            tf = 2 * M * N * K / t_o / 1e9
            rows.append(dict(kernel="gemm", shape=name, ours_ms=round(t_o, 4), cublas_ms=round(t_c, 4), tflops=round(tf, 1),
                             frac_of_measured_bf16=round(tf / peaks["bf16_tflops"], 3)))
            if a.gemm_2cta and M >= 512:
                ops.set_gemm_2cta(True)
                t_2 = bench(lambda: ops.gemm(x, w, out))
                ops.set_gemm_2cta(None)
                rows[-1].update(cta_pair_ms=round(t_2, 4), cta_pair_tflops=round(2 * M * N * K / t_2 / 1e9, 1))
    if a.set in ("fp8", "all"):
        # block-scaled fp8 (1x128 activation blocks, 128x128 weight blocks) against FlashInfer's groupwise kernel, the
        # library path the reference serves block-fp8 checkpoints with (layers/linear/backends/flashinfer.py:132-157)
        from phyai_b200.ops import fp8_block

        fp8_shapes = {"fp8.pi05.prefix.gate_up": (968, 2048, 32768), "fp8.pi05.expert.gate_up": (52, 1024, 8192),
                      "fp8.cosmos3.qkv": (7040, 5120, 7168), "fp8.cosmos3.gate_up": (7040, 5120, 27648), "fp8.cosmos3.down": (7040, 13824, 5120)}
        for name, (M, K, N) in fp8_shapes.items():
            if a.only and name != a.only:
                continue
            x, w = torch.randn(M, K, device=dev) * 0.5, torch.randn(N, K, device=dev) * 0.05
            xb = x.reshape(M, K // 128, 128)
            xs = xb.abs().amax(-1).clamp_min(1e-12) / 448.0
            x8 = (xb / xs[..., None]).clamp(-448, 448).reshape(M, K).to(torch.float8_e4m3fn)
            w8, ws = fp8_block.quantize_weight_block(w)
            out = torch.empty(M, N, device=dev, dtype=bf)
            t_o = bench(lambda: fp8_block.gemm_fp8_block(x8, xs, w8, ws, out))
            row = dict(kernel="gemm_fp8_block", shape=name, ours_ms=round(t_o, 4), tflops=round(2 * M * N * K / t_o / 1e9, 1),
                       kernel_status=ops.kernel_status())
            print(json.dumps(row), flush=True)          # before the library call: its first use may compile for minutes
            if not a.no_baselines:
                t_f, note = float("nan"), ""
                try:
                    import flashinfer.gemm as fg

                    xs_mn = xs.t().contiguous()                      # MN-major: (K/128, M)
                    ws_mn = ws.t().contiguous()                      # (K/128, N/128)
                    t_f = bench(lambda: fg.gemm_fp8_nt_groupwise(x8, w8, xs_mn, ws_mn, scale_granularity_mnk=(1, 128, 128),
                                                                 scale_major_mode="MN", out_dtype=bf))
                except Exception as e:  # noqa: BLE001 - a missing or unsupported library path is a result, not a failure
                    note = f"{type(e).__name__}: {str(e)[:120]}"
                print(json.dumps(dict(kernel="flashinfer.gemm_fp8_nt_groupwise", shape=name, flashinfer_ms=round(t_f, 4), note=note)), flush=True)
    if a.set in ("nvfp4", "all"):
        # NVFP4 (e2m1 operands, ue4m3 scale per 16, fp32 global scales) against FlashInfer's mm_fp4, the call the reference
        # serves NVFP4 checkpoints with (layers/linear/backends/flashinfer.py:163-200); both include nothing but the GEMM,
        # the activation quantiser is timed on its own
        from phyai_b200.layers.quant.specs import Nvfp4Spec
        from phyai_b200.ops import nvfp4

        if not nvfp4.available():
            print(json.dumps(dict(kernel="gemm_nvfp4", skipped="phyai_b200/_blockscaled is not built")), flush=True)
        else:
            for name, (M, K, N) in {"nvfp4.pi05.prefix.gate_up": (968, 2048, 32768), "nvfp4.pi05.expert.gate_up": (52, 1024, 8192),
                                    "nvfp4.cosmos3.qkv": (7040, 5120, 7168), "nvfp4.cosmos3.gate_up": (7040, 5120, 27648)}.items():
                if a.only and name != a.only:
                    continue
                x = (torch.randn(M, K, device=dev) * 0.5).to(bf)
                w = torch.randn(N, K, device=dev) * 0.05
                w4, wsf, wg = Nvfp4Spec.quantize(w)
                sfw = nvfp4.swizzle_scales(wsf, K)
                t_q = bench(lambda: nvfp4.quantize_activation(x, 1.0))
                x4, sfx = nvfp4.quantize_activation(x, 1.0)
                out = torch.empty(M, N, device=dev, dtype=bf)
                alpha = float(wg)
                t_o = bench(lambda: nvfp4.gemm_nvfp4(x4, sfx, w4, sfw, alpha, out=out))
                row = dict(kernel="gemm_nvfp4", shape=name, ours_ms=round(t_o, 4), tflops=round(2 * M * N * K / t_o / 1e9, 1),
                           quantize_act_ms=round(t_q, 4))
                print(json.dumps(row), flush=True)
                if not a.no_baselines:
                    t_f, note = float("nan"), ""
                    try:
                        import flashinfer

                        one = torch.ones(1, device=dev)
                        fa, fsa = flashinfer.nvfp4_quantize(x, one)
                        fb, fsb = flashinfer.nvfp4_quantize(w.to(bf), one)
                        al = torch.tensor([1.0], device=dev)
                        t_f = bench(lambda: flashinfer.mm_fp4(fa, fb.t(), fsa, fsb.t(), al, bf))
                    except Exception as e:  # noqa: BLE001 - a missing or unsupported library path is a result, not a failure
                        note = f"{type(e).__name__}: {str(e)[:160]}"
                    print(json.dumps(dict(kernel="flashinfer.mm_fp4", shape=name, flashinfer_ms=round(t_f, 4), note=note)), flush=True)
    if a.set in ("attention", "all"):
        for name, (S, T, hq, hkv, D) in {"cosmos3.gen": (7040, 512, 40, 8, 128), "cosmos3.gen.tp4": (7040, 512, 10, 2, 128)}.items():
            if a.only and name != a.only:
                continue
            q = torch.randn(S, hq, D, device=dev, dtype=bf)
            k, v = torch.randn(S + T, hkv, D, device=dev, dtype=bf), torch.randn(S + T, hkv, D, device=dev, dtype=bf)
            o, z = torch.empty_like(q), torch.zeros(1, dtype=torch.int32, device=dev)
            ql, kl = torch.full((1,), S, dtype=torch.int32, device=dev), torch.full((1,), S + T, dtype=torch.int32, device=dev)
            t_o = bench(lambda: ops.attention(q, k, v, o, z, ql, z, kl, max_q_len=S))
            qq, kk, vv = (t.transpose(0, 1)[None] for t in (q, k, v))
            t_s = float("nan") if a.no_baselines else bench(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, enable_gqa=True))
            tf = 4 * S * (S + T) * D * hq / t_o / 1e9
            rows.append(dict(kernel="attention", shape=name, ours_ms=round(t_o, 4), sdpa_ms=round(t_s, 4), tflops=round(tf, 1),
                             frac_of_measured_bf16=round(tf / peaks["bf16_tflops"], 3)))
        # the action expert's joint attention: 50 query tokens x 8 heads on one KV head of 256, 968 + 50 KV rows,
        # KV split over a cluster of 8 (the latency kernel, attention_tc.cu)
        if not a.only or a.only == "pi05.expert.joint":
            S, T, hq, hkv, D = 50, 1018, 8, 1, 256
            q = torch.randn(S, hq, D, device=dev, dtype=bf)
            k, v = torch.randn(T, hkv, D, device=dev, dtype=bf), torch.randn(T, hkv, D, device=dev, dtype=bf)
            o, z = torch.empty_like(q), torch.zeros(1, dtype=torch.int32, device=dev)
            ql, kl = torch.full((1,), S, dtype=torch.int32, device=dev), torch.full((1,), T, dtype=torch.int32, device=dev)
            t_o = bench(lambda: ops.attention(q, k, v, o, z, ql, z, kl, max_q_len=S, splits=8, sm_scale=D ** -0.5))
            qq, kk, vv = (t.transpose(0, 1)[None] for t in (q, k, v))
            t_s = float("nan") if a.no_baselines else bench(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, enable_gqa=True))
            rows.append(dict(kernel="attention", shape="pi05.expert.joint", ours_ms=round(t_o, 4), sdpa_ms=round(t_s, 4),
                             kv_bytes=2 * T * D * 2, gbs=round(2 * T * D * 2 / t_o / 1e6, 1)))
    if a.set in ("norm", "all"):
        for name, (R, D) in {"rms.7040x5120": (7040, 5120), "rms.65536x4096": (65536, 4096)}.items():
            if a.only and name != a.only:
                continue
            x, w = torch.randn(R, D, device=dev, dtype=bf), torch.ones(D, device=dev, dtype=bf)
            y = torch.empty_like(x)
            t_o = bench(lambda: ops.norm(x, "rms", weight=w, out=y))
            t_e = float("nan") if a.no_baselines else bench(lambda: (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(bf) * w)
            gbs = 2 * R * D * 2 / t_o / 1e6
            rows.append(dict(kernel="rms_norm", shape=name, ours_ms=round(t_o, 4), eager_ms=round(t_e, 4), gbs=round(gbs, 1),
                             frac_of_measured_hbm=round(gbs / peaks["hbm_gbs"], 3)))
        # AdaRMS (scale | shift | gate rows shared by a group of tokens) at the action-expert and Cosmos-sized shapes,
        # against the eager fp32 formula (counterpart of phyai-kernel/benchmark/bench_adarmsnorm.py)
        for name, (R, D, G) in {"ada_rms.50x1024": (50, 1024, 50), "ada_rms.800x1024": (800, 1024, 50), "ada_rms.8192x4096": (8192, 4096, 1024)}.items():
            if a.only and name != a.only:
                continue
            from phyai_b200.ops import ref

            x = torch.randn(R, D, device=dev, dtype=bf)
            mod = (torch.randn(R // G, 3 * D, device=dev, dtype=bf) * 0.1).contiguous()
            y = torch.empty_like(x)
            t_o = bench(lambda: ops.norm(x, "ada_rms", mod=mod, group=G, out=y))
            t_e = float("nan") if a.no_baselines else bench(lambda: ref.ada_rms_norm(x, mod.repeat_interleave(G, 0)))
            gbs = 2 * R * D * 2 / t_o / 1e6
            rows.append(dict(kernel="ada_rms_norm", shape=name, ours_ms=round(t_o, 4), eager_ms=round(t_e, 4), gbs=round(gbs, 1),
                             frac_of_measured_hbm=round(gbs / peaks["hbm_gbs"], 3)))
    for r in rows:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
