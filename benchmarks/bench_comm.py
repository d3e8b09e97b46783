"""Fused compute + collective kernels over peer memory against their NCCL compositions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_comm.py

For each shape: the fused path (GEMM whose epilogue pushes / scatters its tiles + reduce-residual-norm
[+ gather] kernel [+ waiting GEMM]) and the baseline (the same GEMM into a local buffer, NCCL all-reduce,
residual-add + RMSNorm kernel). Timed on the device with CUDA events over 20 iterations after 5 warm-up
iterations, max over ranks. The roofline time of a fused call is the slower of FLOPs / measured bf16
peak and bytes that must cross NVLink per GPU / 770 GB/s (measured peer-copy bandwidth on this pool).
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

NVLINK_GBS = 770.0


def timed(fn, n=20, warm=5, graph=False):
    """Mean device time of ``fn``. ``graph=True`` captures it once and times replays, which is how the serving paths
    run these kernels (no Python or launch overhead between them)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                fn()
        torch.cuda.synchronize()
        dist.barrier()
        eager, fn = fn, g.replay
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    e1.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from phyai_b200 import ops
    from phyai_b200 import parallel as P
    from phyai_b200.parallel.symm import PeerGroup

    peaks = {"bf16_tflops": 1590.0}
    f = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if f.is_file():
        peaks.update({k: v for k, v in json.loads(f.read_text()).items() if isinstance(v, (int, float))})
    mesh = P.init((world,), ("tp",), device="cuda")
    ops.set_pdl(True)
    pg = PeerGroup.for_axis(mesh, "tp", heap_bytes=3 << 30)
    bf = torch.bfloat16
    rows_out = []
    # (name, M tokens, K per rank, N hidden, N2 width of the following column-parallel GEMM per rank)
    shapes = [("pi05.expert.o_proj", 50, 2048 // world, 1024, 2560 // world), ("pi05.prefix.down", 968, 16384 // world, 2048, 32768 // world),
              ("cosmos3.o_proj", 7040, 5120 // world, 5120, 7168 // world), ("cosmos3.down", 7040, 13824 // world, 5120, 27648 // world)]
    for name, M, K, N, N2 in shapes:
        scatter = M >= 1024
        per = -(-M // world) if scatter else M
        st = pg.stream(f"s.{name}", per, N, gather_rows=M, gather_cols=N)
        x, w = torch.randn(M, K, device=dev, dtype=bf) * 0.1, torch.randn(N, K, device=dev, dtype=bf) * 0.1
        w2 = torch.randn(N2, N, device=dev, dtype=bf) * 0.1
        h, wn = torch.randn(M, N, device=dev, dtype=bf), torch.ones(N, device=dev, dtype=bf)
        part, y, z = torch.empty(M, N, device=dev, dtype=bf), torch.empty(M, N, device=dev, dtype=bf), torch.empty(M, N2, device=dev, dtype=bf)

        def fused():
            t = st.linear_reduce(x, w, scatter=scatter, residual=h, norm="rms", weight=wn, gather=True)
            ops.gemm(t.y, w2, z, wait=t.wait)

        def single():
            # whole partial to every peer, reduce + residual + norm in the GEMM's own CTAs (few rows) or in one
            # reduce kernel, normalised rows local: what the Pi0.5 tensor-parallel plan issues
            st.linear_reduce(x, w, residual=h, y=y, norm="rms", weight=wn)
            ops.gemm(y, w2, z)

        def baseline():
            ops.gemm(x, w, part)
            dist.all_reduce(part)
            ops.norm(part, "rms", weight=wn, residual=h, out=y)
            ops.gemm(y, w2, z)

        def compute_only():
            ops.gemm(x, w, part)
            ops.norm(part, "rms", weight=wn, residual=h, out=y)
            ops.gemm(y, w2, z)

        t_f, t_b, t_c = timed(fused), timed(baseline), timed(compute_only)
        try:
            g_f, g_b = timed(fused, graph=True), timed(baseline, graph=True)
        except Exception as e:      # a collective that cannot be captured on this stack
            g_f = g_b = float("nan")
            if rank == 0:
                print(f"# graph timing unavailable for {name}: {type(e).__name__}: {e}", flush=True)
        one = {}
        if not scatter:
            before = st.single_launches
            one = {"local_y_ms": round(timed(single), 4), "graph_local_y_ms": round(timed(single, graph=True), 4)}
            one["single_launch"] = st.single_launches > before
        flops = 2.0 * M * N * K + 2.0 * M * N2 * N
        # per GPU over NVLink: scatter sends (w-1)/w of its partial and gathers (w-1)/w of the normed rows; one-shot sends w-1 partials
        link_bytes = (2.0 * (world - 1) / world * M * N * 2) if scatter else ((world - 1) * M * N * 2.0 + (world - 1) * M * N * 2.0)
        roof_ms = max(flops / (peaks["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        rows_out.append(dict(shape=name, world=world, mode="scatter+gather" if scatter else "one-shot", fused_ms=round(t_f, 4),
                             nccl_composition_ms=round(t_b, 4), compute_only_ms=round(t_c, 4), graph_fused_ms=round(g_f, 4),
                             graph_nccl_composition_ms=round(g_b, 4), roofline_ms=round(roof_ms, 4),
                             frac_of_roofline=round(roof_ms / min(t_f, g_f if g_f == g_f else t_f), 3),
                             speedup_vs_nccl=round(t_b / t_f, 3), graph_speedup_vs_nccl=round(g_b / g_f, 3) if g_f == g_f else None, **one))
    if world == 2:
        for name, n in (("cfg.cosmos3.super_latent", 16 * 8 * 44 * 80), ("cfg.cosmos3.720p_latent", 48 * 24 * 45 * 80)):
            v = torch.randn(n, device=dev, dtype=bf)

            def fused_cfg():
                pg.cfg_exchange(v, is_cond=rank == 0, g=7.0)

            def nccl_cfg():
                pair = torch.empty(2, n, device=dev, dtype=bf)
                dist.all_gather_into_tensor(pair, v)
                ops.cfg_combine(pair[0], pair[1], 7.0)

            t_f, t_b = timed(fused_cfg), timed(nccl_cfg)
            roof = n * 2 / (NVLINK_GBS * 1e6)
            rows_out.append(dict(shape=name, world=2, mode="cfg exchange + combine", fused_ms=round(t_f, 4), nccl_composition_ms=round(t_b, 4),
                                 roofline_ms=round(roof, 5), frac_of_roofline=round(roof / t_f, 3), speedup_vs_nccl=round(t_b / t_f, 3)))
    torch.cuda.synchronize()
    status = ops.kernel_status()
    if rank == 0:
        for r in rows_out:
            print(json.dumps(r), flush=True)
        print(json.dumps({"kernel_status": status}))
    pg.sync()
    P.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
