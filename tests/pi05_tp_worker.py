"""Child of test_pi05_tp_gpu.py: one rank of a tensor-parallel Pi0.5 (launched with torch.distributed.run).

Every rank loads its shards of one synthetic checkpoint, serves the same request through the captured
tensor-parallel plan, and compares the action chunk with the single-rank eager model on the same weights."""

import os
import sys
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist


def config():
    from phyai_b200.models.pi05.configuration_pi05 import (GemmaExpertConfig, PaliGemmaTextConfig, PI05Config,
                                                           SiglipVisionConfig)

    return PI05Config(
        vision=SiglipVisionConfig(hidden_size=144, num_hidden_layers=2, num_attention_heads=2, intermediate_size=304,
                                  image_size=56, patch_size=14, projection_dim=256),
        text=PaliGemmaTextConfig(hidden_size=256, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                                 head_dim=256, intermediate_size=1024, vocab_size=1024),
        expert=GemmaExpertConfig(hidden_size=128, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                                 head_dim=256, intermediate_size=512, adarms_cond_dim=128),
        chunk_size=50, max_action_dim=32, num_inference_steps=4, tokenizer_max_length=48)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = f"cuda:{torch.cuda.current_device()}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    from phyai_b200 import ops
    from phyai_b200 import parallel as P
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig
    from phyai_b200.models.pi05.main_pi05_tp import PI05TPArgs
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model
    from phyai_b200.models.pi05.plan_tp_pi05 import PI05TPPlan
    from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request
    from phyai_b200.parallel.mesh import Mesh
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    cfg = config()
    ec = EngineConfig(device=DeviceConfig(dev, torch.bfloat16), parallel=ParallelConfig(world_size=world, tp_size=world))
    ckpt = Path(tempfile.gettempdir()) / f"phyai_b200_pi05_tp_{os.environ['MASTER_PORT']}"
    fails: list[str] = []

    # the engine first: it installs the engine configuration and the tp mesh the checkpoint writer below relies on
    if rank == 0:
        from phyai_b200.engine_config import init_engine_config

        init_engine_config(ec)
        P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cuda"))
        with P.use_mesh("single"):
            whole = PI05Model(cfg).eval()
        state = synthetic_state_dict(whole, seed=11, std=0.05)
        g0 = torch.Generator().manual_seed(5)
        for k in list(state):                     # norm scales away from identity, so that every fused norm is visible
            if state[k].dim() == 1 and "norm" in k and "dense" not in k:
                state[k] = (torch.randn(state[k].shape, generator=g0) * 0.2).to(state[k].dtype)
        write_checkpoint(ckpt, state)
    dist.barrier()
    shard_expert = os.environ.get("PI05_TP_SHARD_EXPERT", "0") == "1"
    eng = Engine(EngineArgs("pi05_tp", PI05TPArgs(config=cfg, checkpoint_dir=str(ckpt), max_batch_size=2, shard_expert=shard_expert,
                                                  inputs_image_shape=[[56, 56, 3]] * 2, weight_strict=False), ec))
    sch = eng.entry.scheduler
    if not isinstance(sch.plan, PI05TPPlan) or sch.plan.tp != world or sch.plan.expert_replicated == shard_expert:
        fails.append(f"plan is {type(sch.plan).__name__}, tp={getattr(sch.plan, 'tp', None)}, "
                     f"expert whole={getattr(sch.plan, 'expert_replicated', None)}")
    P.register_mesh("single", Mesh((1,), ("tp",), rank=0, build_groups=False, device_type="cuda"))
    with P.use_mesh("single"):
        whole = PI05Model(cfg).eval()
        load_pretrained(whole, ckpt, strict=False)

    g = torch.Generator().manual_seed(0)          # the same request on every rank
    for batch, lens in ((1, [40]), (2, [40, 7]), (2, [12, 30])):
        req = PI05Request((torch.rand(batch, 2, 3, 56, 56, generator=g) * 2 - 1).bfloat16().to(dev),
                          torch.randint(0, 1024, (batch, 48), generator=g).to(dev), torch.tensor(lens, device=dev),
                          torch.randn(batch, 50, 32, generator=g).bfloat16().to(dev))
        out = eng.step(req)
        again = eng.step(req)
        torch.cuda.synchronize()
        with P.use_mesh("single"):
            want = whole.sample_actions(req.pixel_values, req.input_ids, torch.tensor(lens), req.noise)
        rel = ((out.float() - want.float()).abs().max() / want.float().abs().max()).item()
        if not rel < 5e-2:
            fails.append(f"batch {batch} lens {lens}: rel err {rel:.4g}")
        if not torch.equal(out, again):
            fails.append(f"batch {batch} lens {lens}: replay differs")
        ranks = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(ranks, out.contiguous())
        if not all(torch.equal(ranks[0], r) for r in ranks):
            fails.append(f"batch {batch} lens {lens}: ranks disagree")
    status = int(ops.kernel_status())
    if status != 0:
        fails.append(f"kernel status {status}")
    # PHYAI_PEER_GUARD=1 (set by the test): no kernel of any rank stored outside its buffer of this rank's heap
    from phyai_b200.parallel.symm import PeerGroup

    groups = PeerGroup.open_groups()
    if not groups or not all(g.guard_bytes for g in groups):
        fails.append("no peer group with guard bands is open")
    for g in groups:
        g.sync()
        try:
            g.check_guards()
        except Exception as e:  # noqa: BLE001
            fails.append(str(e))
    eng.close()
    t = torch.tensor([len(fails)], device=dev)
    dist.all_reduce(t)
    for f in fails:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0 and int(t.item()) == 0:
        print("PI05_TP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if int(t.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
