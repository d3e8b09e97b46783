"""Child of test_dist_cpu.py: one gloo rank. Checks the collective vocabulary, tensor-parallel Cosmos3
against a single-rank model with the same checkpoint, and CFG-parallel guidance against sequential."""

import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mode = sys.argv[1]
    dist.init_process_group("gloo")
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig, init_engine_config
    from phyai_b200.layers import linear as L
    from phyai_b200.parallel.mesh import Mesh

    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False)))
    fails: list[str] = []

    def check(name, got, want, tol=1e-5):
        err = (got.float() - want.float()).abs().max().item()
        if not err <= tol * max(1.0, want.float().abs().max().item()):
            fails.append(f"{name}: err {err:.3g}")

    if mode == "collectives":
        mesh = P.init((world,), ("tp",), device="cpu")
        x = torch.arange(6, dtype=torch.float32).reshape(2, 3) + rank
        check("all_reduce", P.all_reduce(x, "tp"), sum(torch.arange(6.).reshape(2, 3) + r for r in range(world)))
        check("all_reduce.max", P.all_reduce(x, "tp", reduce="max"), torch.arange(6.).reshape(2, 3) + world - 1)
        ag = P.all_gather(x, "tp", dim=1)
        check("all_gather", ag, torch.cat([torch.arange(6.).reshape(2, 3) + r for r in range(world)], 1))
        rs = P.reduce_scatter(torch.ones(2 * world, 3) * (rank + 1), "tp", dim=0)
        check("reduce_scatter", rs, torch.ones(2, 3) * sum(range(1, world + 1)))
        a2a = P.all_to_all(torch.arange(world * 2.).reshape(world * 2, 1) + 100 * rank, "tp", split_dim=0, concat_dim=0)
        want = torch.cat([torch.arange(2.).reshape(2, 1) + 2 * rank + 100 * r for r in range(world)])
        check("all_to_all", a2a, want)
        check("broadcast", P.broadcast(torch.full((3,), float(rank)), "tp", src=1), torch.full((3,), 1.0))
        if rank == 0:
            P.send(torch.tensor([7.0]), 1, "tp")
        elif rank == 1:
            check("recv", P.recv(torch.zeros(1), 0, "tp"), torch.tensor([7.0]))
        P.barrier("tp")
        assert mesh.axis_size("tp") == world and mesh.axis_size("dp") == 1
    elif mode == "cosmos3_tp":
        from phyai_b200.models.cosmos3 import Cosmos3Transformer, tiny_cosmos3_config
        from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

        P.init((world,), ("tp",), device="cpu")
        L.init()
        P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cpu"))
        mc = tiny_cosmos3_config(action_gen=True, num_key_value_heads=max(2, world))      # one KV head per rank at least
        with P.use_mesh("single"):
            single = Cosmos3Transformer(mc, params_dtype=torch.float32, device="cpu").eval()
        tp_model = Cosmos3Transformer(mc, params_dtype=torch.float32, device="cpu").eval()
        ckpt = Path(tempfile.gettempdir()) / f"phyai_b200_dist_worker_{os.environ['MASTER_PORT']}"
        if rank == 0:
            write_checkpoint(ckpt, synthetic_state_dict(single, seed=3, std=0.2))
        dist.barrier()
        load_pretrained(single, ckpt, strict=False)
        load_pretrained(tp_model, ckpt, strict=False)
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(0, 256, (2, 6), generator=g)
        mask = torch.ones(2, 6, dtype=torch.long)
        vs = (2, 4, 6)
        lat, act = torch.randn(2, 4, *vs, generator=g), torch.randn(2, 3, 8, generator=g)
        t = torch.tensor([300.0, 300.0])
        dom = torch.tensor([1, 2])
        with P.use_mesh("single"):
            want = single(lat, t, single.encode_condition(ids, mask, vs, 24.0, action_len=3), action_latents=act, action_domain_id=dom)
        got = tp_model(lat, t, tp_model.encode_condition(ids, mask, vs, 24.0, action_len=3), action_latents=act, action_domain_id=dom)
        check("video", got[0], want[0], 1e-4)
        check("action", got[1], want[1], 1e-4)
    elif mode == "cosmos3_cfg":
        from phyai_b200.models.cosmos3 import Cosmos3T2VRequest, Cosmos3T2VScheduler, Cosmos3Transformer, tiny_cosmos3_config

        mesh = P.init((world, 1), ("cfg", "tp"), device="cpu")
        L.init()
        tr = Cosmos3Transformer(tiny_cosmos3_config(), params_dtype=torch.float32, device="cpu").eval().init_random(1, std=0.2)
        g = torch.Generator().manual_seed(0)
        ids, nids = torch.randint(0, 256, (1, 6), generator=g), torch.randint(0, 256, (1, 6), generator=g)
        mask = torch.ones(1, 6, dtype=torch.long)
        req = Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(2, 4, 6), num_inference_steps=3, guidance_scale=4.0)
        par = Cosmos3T2VScheduler(tr, device="cpu")
        par.setup()
        assert par.cfg_size == world and par.cfg_rank == rank
        got = par.step(req)
        P.register_mesh("single", Mesh((1, 1), ("cfg", "tp"), rank=0, build_groups=False, device_type="cpu"))
        with P.use_mesh("single"):
            seq = Cosmos3T2VScheduler(tr, device="cpu")
            seq.setup()
            assert seq.cfg_size == 1
            want = seq.step(req)
        check("cfg-parallel", got, want, 1e-4)
    elif mode == "vae_tiles":
        # spatially tiled VAE decode over the ranks (halo + feathered blend) against the one-rank decode
        from phyai_b200.models.cosmos3 import Cosmos3WanVAEConfig
        from phyai_b200.models.cosmos3.vae_wan import Cosmos3WanVAE

        P.init((1, world), ("cfg", "tp"), device="cpu")
        vcfg = Cosmos3WanVAEConfig(z_dim=4, decoder_base_dim=8, base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
        torch.manual_seed(5)                      # same weights on every rank
        vae = Cosmos3WanVAE(vcfg, dtype=torch.float32, device="cpu").eval()
        with torch.no_grad():
            for prm in vae.parameters():
                prm.copy_(torch.randn(prm.shape) * 0.1)
        lat = torch.randn(1, 4, 2, 6, 8, generator=torch.Generator().manual_seed(2))
        whole = vae.decode(lat)
        tiled = vae.decode_parallel(lat, halo=2)
        if tuple(tiled.shape) != tuple(whole.shape):
            fails.append(f"tiled decode shape {tuple(tiled.shape)} != {tuple(whole.shape)}")
        else:
            # the tiles see a halo of two latent rows instead of the whole frame: the interior agrees, the seam is blended
            err = (tiled - whole).abs()
            if not (torch.isfinite(tiled).all() and err.mean().item() < 0.05):
                fails.append(f"tiled decode differs: mean {err.mean().item():.3g} max {err.max().item():.3g}")
            gathered = [torch.zeros_like(tiled) for _ in range(world)]
            dist.all_gather(gathered, tiled)
            check("every rank holds the same clip", gathered[0], gathered[-1], 1e-6)
    elif mode == "pi05_tp":
        from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
        from phyai_b200.models.pi05.main_pi05_tp import PI05TPScheduler
        from phyai_b200.models.pi05.modeling_pi05 import PI05Model
        from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request
        from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

        P.init((world,), ("tp",), device="cpu")
        L.init()
        P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cpu"))
        cfg = tiny_pi05_config()
        with P.use_mesh("single"):
            single = PI05Model(cfg, device="cpu").eval()
        tp_model = PI05Model(cfg, device="cpu").eval()
        ckpt = Path(tempfile.gettempdir()) / f"phyai_b200_dist_worker_{os.environ['MASTER_PORT']}"
        if rank == 0:
            write_checkpoint(ckpt, synthetic_state_dict(single, seed=7, std=0.1))
        dist.barrier()
        load_pretrained(single, ckpt, strict=False)
        load_pretrained(tp_model, ckpt, strict=False)
        g = torch.Generator().manual_seed(0)
        req = PI05Request(torch.rand(2, 2, 3, 56, 56, generator=g) * 2 - 1, torch.randint(0, 1024, (2, 16), generator=g),
                          torch.tensor([16, 9]), torch.randn(2, 10, 8, generator=g))
        with P.use_mesh("single"):
            want = single.sample_actions(req.pixel_values, req.input_ids, req.lang_lens, req.noise)
        sch = PI05TPScheduler(tp_model, max_batch_size=2, num_images=2, device="cpu")
        sch.setup()
        assert sch.tp_size == world
        check("pi05 tp", sch.step(req), want, 2e-4)
    elif mode in ("pi05_dp", "pi0_dp"):
        from phyai_b200.engine import Engine, EngineArgs
        from phyai_b200.engine_config import ParallelConfig

        ec = EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False),
                          parallel=ParallelConfig(world_size=world, dp_size=world))
        single_ec = EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False))
        g = torch.Generator().manual_seed(0)
        B = 2 * world - 1                                # last rank gets a padded row
        px, ids, lens = torch.rand(B, 2, 3, 56, 56, generator=g) * 2 - 1, torch.randint(0, 1024, (B, 16), generator=g), torch.randint(1, 17, (B,), generator=g)
        noise = torch.randn(B, 10, 8, generator=g)
        shape = [[56, 56, 3]] * 2
        if mode == "pi05_dp":
            from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
            from phyai_b200.models.pi05.main_pi05 import PI05Args
            from phyai_b200.models.pi05.main_pi05_wn import PI05WNArgs
            from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request

            kw = dict(config=tiny_pi05_config(), inputs_image_shape=shape, random_init_seed=3)
            req = PI05Request(px, ids, lens, noise)
            eng = Engine(EngineArgs("pi05_wn", PI05WNArgs(max_batch_size=2 * world, **kw), ec))
            ref_args = ("pi05", PI05Args(max_batch_size=B, **kw))
        else:
            from phyai_b200.models.pi0.configuration_pi0 import tiny_pi0_config
            from phyai_b200.models.pi0.main_pi0 import PI0Args
            from phyai_b200.models.pi0.main_pi0_wn import PI0WNArgs
            from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request

            kw = dict(config=tiny_pi0_config(), inputs_image_shape=shape, random_init_seed=3)
            req = PI0Request(px, ids, lens, torch.randn(B, 8, generator=g), noise)
            eng = Engine(EngineArgs("pi0_wn", PI0WNArgs(max_batch_size=2 * world, **kw), ec))
            ref_args = ("pi0", PI0Args(max_batch_size=B, **kw))
        out = eng.step(req if rank == 0 else None)
        if rank == 0:
            assert out.shape[0] == B
            # the same request through the single-process plugin (same seed -> same weights)
            P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cpu"))
            from phyai_b200.models.pi05.modeling_pi05 import PI05Model  # noqa: F401  (import side effects only)
            with P.use_mesh("single"):
                model = eng.entry.model
                if mode == "pi05_dp":
                    want = model.sample_actions(px, ids, lens, noise)
                else:
                    want = model.sample_actions(px, ids, lens, req.state, noise)
            check(mode, out, want, 2e-4)
        # an oversize batch must raise on every rank instead of leaving peers in a receive
        big = None
        if rank == 0:
            big = type(req)(*[torch.cat([t] * 3) if isinstance(t, torch.Tensor) else t for t in (getattr(req, f) for f in req.__dataclass_fields__)])
        try:
            eng.step(big)
            fails.append("oversize batch was accepted")
        except (ValueError, RuntimeError):
            pass
        eng.entry.scheduler.local.close()
    elif mode in ("cosmos3_wn_engine", "cosmos3_policy_wn_engine"):
        # the multi-rank plugins through the Engine: guidance branches on two ranks (cfg = world), against the single-rank
        # plugin's scheduler on a one-rank mesh with the same weights
        from phyai_b200 import Engine, EngineArgs, ParallelConfig
        from phyai_b200.models.cosmos3 import (Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3T2VRequest, Cosmos3T2VScheduler,
                                               tiny_cosmos3_config)
        from phyai_b200.models.cosmos3.main_cosmos3_policy_wn import Cosmos3PolicyWNArgs
        from phyai_b200.models.cosmos3.main_cosmos3_wn import Cosmos3WNArgs

        policy = mode == "cosmos3_policy_wn_engine"
        cfg_ranks, tp_ranks = (2, world // 2) if world >= 4 else (world, 1)          # four ranks: two guidance branches x two tensor-parallel ranks
        ec = EngineConfig(device=DeviceConfig("cpu", torch.float32), parallel=ParallelConfig(world_size=world, cfg_size=cfg_ranks, tp_size=tp_ranks),
                          runtime=RuntimeConfig(use_cuda_graph=False))
        cfg = tiny_cosmos3_config(action_gen=policy)
        # the plugin loads a checkpoint folder in the upstream layout (transformer/ under upstream key names): written once
        # from a one-rank model's key index, so that sharded and whole models hold the same tensors
        from phyai_b200.models.cosmos3 import Cosmos3Transformer
        from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_inverse_remap
        from phyai_b200.weights import synthetic_state_dict, write_checkpoint

        ckpt = Path(tempfile.gettempdir()) / f"phyai_b200_dist_worker_{os.environ['MASTER_PORT']}"
        P.register_mesh("single", Mesh((1, 1), ("cfg", "tp"), rank=0, build_groups=False, device_type="cpu"))
        if rank == 0:
            with P.use_mesh("single"):
                probe = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu")
            write_checkpoint(ckpt / "transformer", {cosmos3_inverse_remap(k): v for k, v in synthetic_state_dict(probe, seed=4, std=0.2).items()},
                             cfg.to_dict())
        dist.barrier()
        kw = dict(checkpoint_dir=ckpt, config=cfg, weight_strict=True)
        args = Cosmos3PolicyWNArgs(**kw) if policy else Cosmos3WNArgs(load_vae=False, load_sound=False, **kw)
        eng = Engine(EngineArgs("cosmos3_policy_wn" if policy else "cosmos3_wn", args, ec))
        sch = eng.entry.scheduler
        if (sch.cfg_size, sch.cfg_rank) != (cfg_ranks, rank // tp_ranks):
            fails.append(f"plugin scheduler sees cfg {sch.cfg_rank}/{sch.cfg_size}")
        if eng.entry.transformer.gen_layers[0].mlp.down_proj.tp_size != tp_ranks:
            fails.append("the transformer is not sharded over the tensor-parallel ranks")
        g = torch.Generator().manual_seed(0)
        ids, nids = torch.randint(0, 256, (1, 6), generator=g), torch.randint(0, 256, (1, 6), generator=g)
        mask = torch.ones(1, 6, dtype=torch.long)
        if policy:
            req = Cosmos3ActionRequest(ids, mask, nids, mask, video_shape=(2, 4, 6), mode="policy", domain_id=1, action_chunk=3, raw_action_dim=5,
                                       action_dim=8, cond_video_latents=torch.randn(1, 4, 2, 4, 6, generator=g), num_inference_steps=3, guidance_scale=3.0)
        else:
            req = Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(2, 4, 6), num_inference_steps=3, guidance_scale=4.0)
        got = eng.step(req)
        with P.use_mesh("single"):
            from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_weight_remap
            from phyai_b200.weights import load_pretrained

            whole = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu").eval()      # a one-rank copy of the same checkpoint
            load_pretrained(whole, ckpt / "transformer", remap=cosmos3_weight_remap, strict=True)
            seq = (Cosmos3PolicyScheduler if policy else Cosmos3T2VScheduler)(whole, device="cpu", flow_shift=sch._flow_shift,
                                                                             use_karras_sigmas=sch._karras)      # the plugin's sampler settings
            seq.setup()
            want = seq.step(req)
        if policy:
            check("policy plugin over cfg ranks", got, want["action"], 1e-4)
        else:
            check("generation plugin over cfg ranks", got, want, 1e-4)
        gathered = [torch.zeros_like(got) for _ in range(world)]
        dist.all_gather(gathered, got.contiguous())
        check("every rank returns the same result", gathered[0], gathered[-1], 1e-6)
        eng.entry.close()
    elif mode == "seq_parallel":
        # Megatron-style sequence parallelism on the tensor-parallel axis: activations between the two linears' blocks are
        # split by tokens; the column-parallel layer gathers the tokens, the row-parallel layer reduce-scatters them back
        mesh = P.init((world,), ("tp",), device="cpu")
        L.init()
        H, I, T = 16, 24 * world, 6 * world
        g = torch.Generator().manual_seed(3)
        w1, b1, w2, b2 = torch.randn(I, H, generator=g), torch.randn(I, generator=g), torch.randn(H, I, generator=g), torch.randn(H, generator=g)
        x = torch.randn(T, H, generator=g)
        col = L.ColumnParallelLinear(H, I, bias=True, sp_axis="tp", params_dtype=torch.float32)
        row = L.RowParallelLinear(I, H, bias=True, sp_axis="tp", params_dtype=torch.float32)
        per_i, per_t = I // world, T // world
        col.weight.data.copy_(w1[rank * per_i:(rank + 1) * per_i])
        col.bias.data.copy_(b1[rank * per_i:(rank + 1) * per_i])
        row.weight.data.copy_(w2[:, rank * per_i:(rank + 1) * per_i])
        row.bias.data.copy_(b2)
        h, _ = col(x[rank * per_t:(rank + 1) * per_t].contiguous())            # this rank's tokens in, all tokens x this rank's columns out
        check("seq_parallel.column", h, (x @ w1.t() + b1)[:, rank * per_i:(rank + 1) * per_i], 1e-5)
        y, _ = row(torch.relu(h))
        want = torch.relu(x @ w1.t() + b1) @ w2.t() + b2
        check("seq_parallel.row", y, want[rank * per_t:(rank + 1) * per_t], 1e-4)   # this rank's tokens of the full result; the bias once
        if y.shape != (per_t, H):
            fails.append(f"seq_parallel: output {tuple(y.shape)} is not this rank's token shard")
    else:
        raise SystemExit(f"unknown mode {mode}")

    ok = torch.tensor([0 if fails else 1])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in fails:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print("DIST_OK" if ok.item() == 1 else "DIST_FAILED", flush=True)
    dist.destroy_process_group()
    return 0 if ok.item() == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
