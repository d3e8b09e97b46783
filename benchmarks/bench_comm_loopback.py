"""The fused compute + collective kernels on ONE GPU, for counter captures.

    python benchmarks/bench_comm_loopback.py [--case linear|scatter|cfg|gather|all] [--iters 5]

A profiler may not wrap a multi-rank job, and kernels that wait on one another may not run as separate
launches, so this harness plays a peer group of two inside one process: both ranks' symmetric slabs live
in this GPU's memory, the "peer" pointers point at them, and the launches are issued in an order in which
every wait is already satisfied when its kernel starts (both ranks' producers first, then the consumers;
for the pair exchange the partner's half is written by hand before the launch). The kernels, their
parameters and their memory traffic are the ones of a real two-GPU run except that remote stores land in
local HBM instead of crossing NVLink; numerics are checked against an fp32 statement of each collective.

Shapes follow the Cosmos3-Super tensor-parallel layer at tp = 2 (o-projection 1024 rows of the 7552,
K = 2560 per rank, N = 5120) and the guided latent of the CFG pair (4.1 M bf16).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from phyai_b200 import ops  # noqa: E402

WORLD = 2
SIG_BYTES = 8192          # 256 channels x 32 bytes


class Loopback:
    """Two slabs in local memory laid out like ``PeerGroup`` slabs: signal words first, then buffers."""

    def __init__(self, heap_bytes: int) -> None:
        self.ext = ops.ext()
        self.slabs = [torch.zeros(SIG_BYTES + heap_bytes, dtype=torch.uint8, device="cuda") for _ in range(WORLD)]
        self.ptrs = [s.data_ptr() for s in self.slabs]
        self.top = SIG_BYTES

    def alloc(self, nbytes: int) -> int:
        off = self.top
        self.top = (off + nbytes + 255) // 256 * 256
        assert self.top <= self.slabs[0].numel()
        return off

    def sig(self, rank: int) -> torch.Tensor:
        return self.slabs[rank][:SIG_BYTES].view(torch.int32).view(-1, 8)   # [channel][arrive0, arrive1, epoch, done, pad x4]

    def view(self, rank: int, off: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
        return self.slabs[rank][off:off + n].view(dtype).view(*shape)


def timed(fn, iters: int) -> float:
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def case_linear(iters: int, scatter: bool) -> dict:
    """Row-parallel GEMM whose epilogue stores into both ranks' slots, then the reduce + residual + RMSNorm
    consumer of each rank (``scatter``: tiles only to the row owner, the owner's normalised rows to both)."""
    M, K, N = 1024, 2560, 5120
    g = torch.Generator().manual_seed(0)
    lb = Loopback(2 * WORLD * M * N * 2 + M * N * 2 + (1 << 20))
    ext = lb.ext
    per = M // WORLD if scatter else 0
    slot_stride = (per if scatter else M) * N
    slots_off = lb.alloc(2 * WORLD * slot_stride * 2)
    y_off = lb.alloc(M * N * 2) if scatter else -1
    xs = [(torch.randn(M, K, generator=g) * 0.5).bfloat16().cuda() for _ in range(WORLD)]
    ws = [(torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda() for _ in range(WORLD)]
    res0 = torch.randn(M, N, generator=g).bfloat16().cuda()
    wn = (torch.randn(N, generator=g) * 0.1 + 1).bfloat16().cuda()
    hs = [res0.clone() for _ in range(WORLD)]
    ys = [torch.empty(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]

    def run():
        expect = 0
        for r in range(WORLD):                       # both producers first: every arrival is in before a consumer starts
            expect = ext.gemm_push(xs[r], ws[r], lb.ptrs, r, slots_off // 2, slot_stride, N, 0, 0, per, 0, -1, 0)
        for r in range(WORLD):
            hs[r].copy_(res0)
            ext.reduce_norm(lb.ptrs, r, slots_off // 2, slot_stride, M, N, N, 0, 0, expect, hs[r], None, None, None,
                            None if scatter else ys[r], ops.NORM["rms"], wn, None, 1e-6, 592, per,
                            y_off // 2 if scatter else -1, N if scatter else 0, 1)
        if scatter:
            for r in range(WORLD):                   # close the gathered-rows call on each rank (both owners have stored)
                rows = [max(0, min(per, M - q * per)) for q in range(WORLD)]
                arrivals = sum(max(1, min(n, 592)) for n in rows)
                ext.gather_consume(lb.ptrs, r, 0, 0, M, N, N, None, 0, 1, arrivals)

    ms = timed(run, iters)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    want_h = res0.float() + sum((x.float() @ w.float().t()).bfloat16().float() for x, w in zip(xs, ws))
    want_y = want_h.bfloat16().float()
    want_y = want_y * torch.rsqrt(want_y.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
    got_y = lb.view(0, y_off, (M, N)) if scatter else ys[0]
    err = float((got_y.float() - want_y).abs().max() / want_y.abs().max())
    flops = 2.0 * M * K * N * WORLD
    wire = (M * N * 2 * (WORLD - 1) / WORLD if scatter else M * N * 2 * (WORLD - 1)) * WORLD   # bytes that would cross NVLink
    return {"case": "scatter" if scatter else "linear", "M": M, "K": K, "N": N, "ms_both_ranks": round(ms, 4),
            "rel_err": round(err, 5), "tflops_per_rank_if_parallel": round(flops / WORLD / (ms / WORLD * 1e-3) / 1e12, 1),
            "remote_bytes": int(wire)}


def case_cfg(iters: int) -> dict:
    n = 16 * 8 * 176 * 184 // 8 * 8            # ~4.1 M elements
    g = torch.Generator().manual_seed(1)
    lb = Loopback(2 * n * 2 + (1 << 20))
    ext = lb.ext
    inbox = lb.alloc(2 * n * 2)
    cond = torch.randn(n, generator=g).bfloat16().cuda()
    unc = torch.randn(n, generator=g).bfloat16().cuda()
    out = torch.empty_like(cond)
    grid = min(128, max(1, (n // 8 + 255) // 256))

    def run():
        # rank 0 is the conditional branch; the partner's half (its push and its arrivals) is put in place by hand
        sig = lb.sig(0)
        parity = int(sig[0, 2].item()) & 1
        lb.view(0, inbox, (2, n))[parity].copy_(unc)
        sig[0, parity] = grid
        ext.cfg_exchange(cond, lb.ptrs, 0, 1, inbox // 2, True, 7.0, out, None, 0.0, 0, 0)
        lb.sig(1)[0, :2] = 0                        # the partner never consumes: drop what rank 0 signalled

    ms = timed(run, iters)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    want = unc.float() + 7.0 * (cond.float() - unc.float())
    err = float((out.float() - want).abs().max() / want.abs().max())
    return {"case": "cfg", "elements": n, "ms_incl_host_arming": round(ms, 4), "rel_err": round(err, 5), "remote_bytes": n * 2}


def case_gather(iters: int) -> dict:
    rows, N = 512, 5120
    g = torch.Generator().manual_seed(2)
    lb = Loopback(2 * WORLD * rows * N * 2 + (1 << 20))
    ext = lb.ext
    slots_off = lb.alloc(2 * WORLD * rows * N * 2)
    xs = [torch.randn(rows, N, generator=g).bfloat16().cuda() for _ in range(WORLD)]
    outs = [torch.empty(WORLD * rows, N, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]

    def run():
        expect = 0
        for r in range(WORLD):
            expect = ext.push_partial(xs[r], lb.ptrs, r, slots_off // 2, rows * N, N, 0, 0)
        for r in range(WORLD):
            ext.gather_consume(lb.ptrs, r, slots_off // 2, rows * N, rows, N, N, outs[r], 0, 0, expect)

    ms = timed(run, iters)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0 and torch.equal(outs[1], torch.cat(xs))
    return {"case": "gather", "rows": rows, "N": N, "ms_both_ranks": round(ms, 4), "remote_bytes": rows * N * 2 * WORLD}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=("linear", "scatter", "cfg", "gather", "all"))
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    ops.set_pdl(False)
    cases = ("linear", "scatter", "cfg", "gather") if a.case == "all" else (a.case,)
    for c in cases:
        if c == "linear":
            rec = case_linear(a.iters, False)
        elif c == "scatter":
            rec = case_linear(a.iters, True)
        elif c == "cfg":
            rec = case_cfg(a.iters)
        else:
            rec = case_gather(a.iters)
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
