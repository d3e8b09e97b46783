"""Child of test_peer_gpu.py: one rank of a peer-memory test (launched with torch.distributed.run).

Every check compares against an fp32 reference built from NCCL collectives of the same inputs."""

import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from phyai_b200 import ops
    from phyai_b200 import parallel as P
    from phyai_b200.ops import ref
    from phyai_b200.parallel.symm import PeerGroup

    mesh = P.init((world,), ("tp",), device="cuda")
    pg = PeerGroup.for_axis(mesh, "tp", heap_bytes=512 << 20)
    g = torch.Generator(device="cpu").manual_seed(1234)
    fails: list[str] = []

    def rnd(*shape, scale=1.0, per_rank=True):
        """Same generator stream on every rank; ``per_rank`` picks this rank's slice of a world-sized draw."""
        t = torch.randn((world, *shape) if per_rank else shape, generator=g) * scale
        return (t[rank] if per_rank else t).to(dev, torch.bfloat16), t

    def nccl_sum(x):
        y = x.float().clone()
        dist.all_reduce(y)
        return y

    def check(name, got, want, tol):
        got, want = got.detach().float().cpu(), want.detach().float().cpu()
        err = (got - want).abs().max().item()
        ref_mag = want.abs().max().item() + 1e-6
        if not (err <= tol * max(1.0, ref_mag)):
            fails.append(f"{name}: err {err:.4g} vs magnitude {ref_mag:.4g}")

    # ---- 1. push + reduce all-reduce, several calls in a row (both parities), odd sizes
    st = pg.stream("ar", 300, 512)
    for it, (m, n) in enumerate([(50, 512), (300, 256), (1, 8), (77, 200)]):
        x, _ = rnd(m, n)
        check(f"all_reduce[{it}]", st.all_reduce(x), nccl_sum(x), 0.02)

    # ---- 2. one-shot fused linear: GEMM epilogue pushes, consumer adds residual, norms
    M, K, N = 50, 256, 1024
    stl = pg.stream("lin", 512, 2048, gather_rows=1024, gather_cols=2048)
    for it in range(3):
        x, _ = rnd(M, K, scale=0.5)
        w, _ = rnd(N, K, scale=0.1)
        res, _ = rnd(M, N, per_rank=False)
        gate, _ = rnd(N, per_rank=False)
        wn, _ = rnd(N, per_rank=False, scale=0.1)
        h = res.clone()
        y = torch.empty_like(h)
        stl.linear_reduce(x, w, residual=h, col_gate=gate, y=y, norm="gemma_rms", weight=wn, eps=1e-6)
        part = nccl_sum(x.float() @ w.float().t())
        h_ref = res.float() + part * gate.float()
        check(f"linear_reduce.h[{it}]", h, h_ref, 0.03)
        check(f"linear_reduce.y[{it}]", y, ref.rms_norm(h.float(), wn.float(), 1e-6, gemma=True), 0.03)
    if stl.single_launches != 3:
        fails.append(f"50-row linear_reduce ran as {stl.single_launches} single launches of 3 (the reduce tail did not engage)")
    # the same shape as two launches (push GEMM, reduce kernel), AdaRMS this time, and a many-row call that never takes the tail
    mod, _ = rnd(3 * N, per_rank=False, scale=0.2)
    for it, (rows, tail) in enumerate([(M, False), (300, True)]):
        x, _ = rnd(rows, K, scale=0.5)
        w, _ = rnd(N, K, scale=0.1)
        res, _ = rnd(rows, N, per_rank=False)
        h = res.clone()
        y = torch.empty_like(h)
        before = stl.single_launches
        stl.linear_reduce(x, w, residual=h, col_gate=mod[2 * N:], y=y, norm="ada_rms", mod=mod, eps=1e-6, allow_tail=tail)
        if stl.single_launches != before:
            fails.append(f"linear_reduce case {it} took the single-launch path")
        part = nccl_sum(x.float() @ w.float().t())
        h_ref = res.float() + part * mod[2 * N:].float()
        check(f"linear_reduce.two_launch.h[{it}]", h, h_ref, 0.03)
        hb = h.float()
        y_ref = hb * torch.rsqrt(hb.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + mod[:N].float()) + mod[N:2 * N].float()
        check(f"linear_reduce.two_launch.y[{it}]", y, y_ref, 0.03)

    # ---- 3. two-step: scatter to row owners, reduce + norm there, gather into every rank, GEMM waits
    M, K, N, N2 = 777, 512, 1024, 768
    for it in range(3):
        x, _ = rnd(M, K, scale=0.5)
        w, _ = rnd(N, K, scale=0.1)
        res, _ = rnd(M, N, per_rank=False)
        wn, _ = rnd(N, per_rank=False, scale=0.1)
        w2, _ = rnd(N2, N, per_rank=False, scale=0.1)
        h = res.clone()
        ticket = stl.linear_reduce(x, w, scatter=True, residual=h, norm="rms", weight=wn, eps=1e-6, gather=True)
        z = ops.gemm(ticket.y, w2, wait=ticket.wait)
        part = nccl_sum(x.float() @ w.float().t())
        h_ref = res.float() + part
        per = -(-M // world)
        mine = slice(rank * per, min(M, (rank + 1) * per))
        check(f"scatter.h[{it}]", h[mine], h_ref[mine], 0.03)
        hb = h_ref.to(torch.bfloat16).float()
        y_ref = hb * torch.rsqrt(hb.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()
        check(f"scatter.y[{it}]", ticket.y, y_ref, 0.05)
        check(f"scatter.gemm[{it}]", z, y_ref.to(torch.bfloat16).float() @ w2.float().t(), 0.05)

    # ---- 3b. the same chain at a size that takes the persistent GEMM (scatter epilogue and waiting loads inside it)
    M, K, N, N2 = 2304, 512, 4096, 4096
    stb = pg.stream("big", -(-M // world), N, gather_rows=M, gather_cols=N)
    for it in range(2):
        x, _ = rnd(M, K, scale=0.5)
        w, _ = rnd(N, K, scale=0.1)
        res, _ = rnd(M, N, per_rank=False)
        wn, _ = rnd(N, per_rank=False, scale=0.1)
        w2, _ = rnd(N2, N, per_rank=False, scale=0.05)
        h = res.clone()
        ticket = stb.linear_reduce(x, w, scatter=True, residual=h, norm="rms", weight=wn, eps=1e-6, gather=True)
        z = ops.gemm(ticket.y, w2, wait=ticket.wait, act="silu", glu=True)
        part = nccl_sum(x.float() @ w.float().t())
        hb = (res.float() + part).to(torch.bfloat16).float()
        y_ref = (hb * torch.rsqrt(hb.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()).to(torch.bfloat16).float()
        check(f"persist.y[{it}]", ticket.y, y_ref, 0.05)
        zz = y_ref @ w2.float().t()
        check(f"persist.gemm[{it}]", z, torch.nn.functional.silu(zz[:, 0::2]) * zz[:, 1::2], 0.06)
    # one-shot push through the persistent kernel as well
    x, _ = rnd(640, 512, scale=0.5)
    w, _ = rnd(4096, 512, scale=0.1)
    sto = pg.stream("big1", 640, 4096)
    out = torch.empty(640, 4096, device=dev, dtype=torch.bfloat16)
    sto.linear_reduce(x, w, h_out=out)
    check("persist.one_shot", out, nccl_sum(x.float() @ w.float().t()), 0.03)

    # ---- 4. gather of row shards
    x, full = rnd(33, 256)
    got = stl.all_gather_rows(x)
    check("all_gather_rows", got, full.reshape(world * 33, 256).to(torch.bfloat16), 1e-6)

    # ---- 5. dispatcher: small bf16 all-reduce goes through the peer backend
    x, _ = rnd(64, 128)
    out = P.all_reduce(x, "tp")
    check("P.all_reduce", out, nccl_sum(x), 0.02)
    d = P.get_dispatcher()
    if "peer" not in d.registry.names():
        fails.append("peer backend not registered")

    # ---- 6. CFG pair (first two ranks), with the fused Euler update
    if world == 2:
        v, both = rnd(4, 16, 40)
        xs = torch.zeros(4 * 16 * 40, device=dev)
        for it in range(3):
            out = pg.cfg_exchange(v.contiguous(), is_cond=rank == 0, g=3.0, x_fp32=xs, dt=-0.1)
            c, u = both[0].to(torch.bfloat16).float(), both[1].to(torch.bfloat16).float()
            check(f"cfg_exchange[{it}]", out.cpu(), u + 3.0 * (c - u), 0.02)
        check("cfg_exchange.euler", xs.cpu().view(4, 16, 40), -0.3 * (u + 3.0 * (c - u)), 0.03)

    # ---- 7. the same fused linear replayed from a CUDA graph (device-side parity keeps it valid)
    M, K, N = 50, 256, 1024
    x, _ = rnd(M, K, scale=0.5)
    w, _ = rnd(N, K, scale=0.1)
    hbuf = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
    pg.sync()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        stl.linear_reduce(x, w, h_out=hbuf)
        side.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            stl.linear_reduce(x, w, h_out=hbuf)
        for _ in range(5):
            gr.replay()
        side.synchronize()
    check("graph.linear_reduce", hbuf, nccl_sum(x.float() @ w.float().t()), 0.03)

    # ---- 8. Cosmos3 GEN tower, tensor parallel over peer memory, against the single-rank eager model
    import tempfile
    from pathlib import Path

    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.models.cosmos3 import Cosmos3Config, Cosmos3Transformer
    from phyai_b200.parallel.mesh import Mesh
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    init_engine_config(EngineConfig(device=DeviceConfig("cuda", torch.bfloat16)))
    from phyai_b200.layers import linear as L

    L.init()
    P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cuda"))
    kvh = max(2, world)                      # the towers shard their K/V heads: at least one per rank
    mc = Cosmos3Config(hidden_size=512, num_hidden_layers=2, num_attention_heads=2 * kvh, num_key_value_heads=kvh, head_dim=128,
                       intermediate_size=1024, vocab_size=512, mrope_section=(24, 20, 20), latent_channel=16,
                       latent_patch_size=2, patch_latent_dim=64)
    with P.use_mesh("single"):
        single = Cosmos3Transformer(mc, params_dtype=torch.bfloat16, device=dev).eval()
    tp_model = Cosmos3Transformer(mc, params_dtype=torch.bfloat16, device=dev).eval()
    ckpt = Path(tempfile.gettempdir()) / "phyai_b200_peer_worker_ckpt"
    if rank == 0:
        write_checkpoint(ckpt, synthetic_state_dict(single, seed=3, std=0.05))
    dist.barrier()
    load_pretrained(single, ckpt, strict=False)
    load_pretrained(tp_model, ckpt, strict=False)
    single.use_fused = False
    ids = torch.randint(0, 512, (1, 12), generator=g).to(dev)
    mask = torch.ones(1, 12, dtype=torch.long, device=dev)
    for vs in ((2, 16, 20), (4, 32, 40)):          # 160 tokens: one-step reduce; 1280 tokens: scatter + gather
        lat = torch.randn(1, 16, *vs, generator=g).to(dev, torch.bfloat16)
        tt = torch.tensor([420.0], device=dev)
        with P.use_mesh("single"):
            want = single(lat, tt, single.encode_condition(ids, mask, vs, 24.0))
        cond = tp_model.encode_condition(ids, mask, vs, 24.0)
        for it in range(2):
            got = tp_model(lat, tt, cond)
            check(f"cosmos3.tp{world}{vs}[{it}]", got, want, 0.06)

    # ---- the ctypes NCCL backend against the real library: eager, and replayed from a CUDA graph
    try:
        from phyai_b200.parallel.backend import Call, Mode, Op
        from phyai_b200.parallel.backends.pynccl import PyNcclBackend

        pn = PyNcclBackend(mesh, ["tp"])
    except Exception as e:  # noqa: BLE001 - e.g. no libnccl that ctypes can load
        pn = None
        if rank == 0:
            print(f"pynccl skipped: {type(e).__name__}: {e}", flush=True)
    if pn is not None:
        def call(op, x, extra=()):
            return Call(op=op, axis="tp", mesh=mesh, dtype=x.dtype, nbytes=x.numel() * x.element_size(), mode=Mode.EAGER,
                        device_type="cuda", extra=extra)

        x = (torch.arange(24, device=dev, dtype=torch.float32).reshape(4, 6) + rank)
        got = pn.execute(call(Op.ALL_REDUCE, x, ("sum",)), x, reduce="sum")
        check("pynccl.all_reduce", got, nccl_sum(x), 1e-6)
        got = pn.execute(call(Op.ALL_GATHER, x, (0,)), x, dim=0)
        want = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(want, x)
        check("pynccl.all_gather", got, torch.cat(want), 1e-6)
        got = pn.execute(call(Op.BROADCAST, x, (world - 1,)), x, src=world - 1)
        check("pynccl.broadcast", got, torch.arange(24, device=dev, dtype=torch.float32).reshape(4, 6) + world - 1, 1e-6)
        xb = torch.ones(64, 128, device=dev, dtype=torch.bfloat16) * (rank + 1)
        pn.execute(call(Op.ALL_REDUCE, xb, ("sum",)), xb, reduce="sum")        # warm the path before capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            yb = pn.execute(call(Op.ALL_REDUCE, xb, ("sum",)), xb, reduce="sum")
        for k in (1, 2):
            xb.fill_(float(k * (rank + 1)))
            graph.replay()
            torch.cuda.synchronize()
            check(f"pynccl.graph[{k}]", yb, torch.full((64, 128), float(k * world * (world + 1) // 2)), 1e-2)
        # NCCL counts a captured collective as a reference on its communicator: the graph goes first,
        # otherwise destroying the communicator waits for it forever
        graph.reset()
        del graph, yb
        torch.cuda.synchronize()
        dist.barrier()
        pn.close()

    torch.cuda.synchronize()
    status = ops.kernel_status()
    if status != 0:
        fails.append(f"kernel status {status}")
    pg.sync()
    # PHYAI_PEER_GUARD=1 (set by the test): no kernel of any rank stored outside its buffer of this rank's heap
    if not pg.guard_bytes:
        fails.append("the symmetric heap has no guard bands")
    for g in PeerGroup.open_groups():
        try:
            g.check_guards()
        except Exception as e:  # noqa: BLE001
            fails.append(str(e))
    ok = torch.tensor([0 if fails else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in fails:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print("PEER_OK" if ok.item() == 1 else "PEER_FAILED", flush=True)
    P.shutdown()
    dist.destroy_process_group()
    return 0 if ok.item() == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
