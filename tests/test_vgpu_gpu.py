"""SM partitions on a real GPU: disjoint green contexts, work confined to a partition, two partitions running
at the same time, per-partition memory pools. Mirrors the reference's concurrency and life-cycle checks
(phyai/tests/vgpu/test_vgpu_concurrency.py:33-98, test_vgpu_basic.py)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _busy(stream, iters, out):
    """Compute-bound work of this library on `stream`: a 2048^3 bf16 GEMM repeated `iters` times."""
    from phyai_b200 import ops

    x = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16) * 0.02
    torch.cuda.current_stream().synchronize()
    with torch.cuda.stream(stream):
        for _ in range(iters):
            ops.gemm(x, w, out)


@pytest.fixture
def vg():
    from phyai_b200 import vgpu

    vgpu._reset_for_tests()
    yield vgpu
    vgpu.close_all()
    vgpu._reset_for_tests()


def test_two_disjoint_partitions_run_concurrently(vg):
    try:
        vg.init(0)
        parts = vg.create_vgpus([64, 64])
    except (vg.VGPUDriverError, ImportError) as e:
        pytest.skip(f"green contexts unavailable here: {e}")
    total = torch.cuda.get_device_properties(0).multi_processor_count
    assert [p.sm_count for p in parts[:2]] == [64, 64] and sum(p.sm_count for p in parts) == total
    a, b = parts[0], parts[1]
    # the same amount of work on each partition, first one after the other, then together
    outs = [torch.empty(2048, 2048, device="cuda", dtype=torch.bfloat16) for _ in range(2)]

    def timed(run):
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        run()
        for p in (a, b):
            torch.cuda.current_stream().wait_stream(p.stream)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    def on(p, out):
        p.stream.wait_stream(torch.cuda.current_stream())
        _busy(p.stream, 40, out)

    for _ in range(2):
        timed(lambda: (on(a, outs[0]), on(b, outs[1])))      # warm up both
    t_a = timed(lambda: on(a, outs[0]))
    t_b = timed(lambda: on(b, outs[1]))
    t_both = timed(lambda: (on(a, outs[0]), on(b, outs[1])))
    # disjoint SM sets: together they take about as long as the slower one, not the sum
    assert t_both < 0.8 * (t_a + t_b), (t_a, t_b, t_both)
    assert torch.isfinite(outs[0].float()).all() and torch.isfinite(outs[1].float()).all()
    # allocations inside activate() come from the partition's own pool
    with a.activate():
        t = torch.empty(1 << 20, device="cuda")
    assert a.mem_pool is not None and b.mem_pool is not None and a.mem_pool.id != b.mem_pool.id
    del t
    for p in parts:
        p.close()
    assert torch.ones(4, device="cuda").sum().item() == 4


def test_torch_backend_gives_one_shard(vg):
    from torch.cuda import green_contexts as gc

    if not gc.SUPPORTED:
        pytest.skip("this PyTorch build has no green-context binding")
    vg.init(0, driver=vg.TorchGreenDriver())
    (p,) = vg.create_vgpus([32], include_remainder=False)
    assert p.sm_count == 32
    out = torch.empty(2048, 2048, device="cuda", dtype=torch.bfloat16)
    with p.activate():
        _busy(torch.cuda.current_stream(), 2, out)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    with pytest.raises(vg.VGPURuntimeError):
        vg.create_vgpus([32, 32])
    p.close()
