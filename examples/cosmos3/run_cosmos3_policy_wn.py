"""Cosmos3 action inference over a CFG x TP mesh (plugin ``cosmos3_policy_wn``), one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/cosmos3/run_cosmos3_policy_wn.py --cfg 2 [--mode policy|forward_dynamics|inverse_dynamics]

The three modes share one request type: ``policy`` predicts the action chunk (and the future frames) from the
first frame, ``forward_dynamics`` predicts frames from clean actions, ``inverse_dynamics`` predicts actions from
clean frames. Every rank passes the same request; rank 0 prints the result. Counterpart of the reference's
examples/cosmos3/run_cosmos3_policy_wn.py.
"""

import argparse
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig, ParallelConfig  # noqa: E402
from phyai_b200.models.cosmos3 import ACTION_MODES, Cosmos3ActionRequest, Cosmos3Config  # noqa: E402
from phyai_b200.models.cosmos3.main_cosmos3_policy_wn import Cosmos3PolicyWNArgs  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=ACTION_MODES, default="policy")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cfg", type=int, default=2)
    ap.add_argument("--steps", type=int, default=4)
    a = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if world != a.tp * a.cfg:
        raise SystemExit(f"tp {a.tp} x cfg {a.cfg} needs {a.tp * a.cfg} ranks, launched {world}")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    small = Cosmos3Config(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                          intermediate_size=1024, vocab_size=512, latent_channel=16, latent_patch_size=2, patch_latent_dim=64,
                          action_gen=True, action_dim=64)
    args = Cosmos3PolicyWNArgs(checkpoint_dir=a.checkpoint) if a.checkpoint else Cosmos3PolicyWNArgs(config=small)
    engine = Engine(EngineArgs("cosmos3_policy_wn", args, EngineConfig(
        device=DeviceConfig(dev, torch.bfloat16), parallel=ParallelConfig(world_size=world, cfg_size=a.cfg, tp_size=a.tp))))
    g = torch.Generator().manual_seed(0)                      # identical inputs on every rank
    ids, mask = torch.randint(0, 512, (1, 32), generator=g), torch.ones(1, 32, dtype=torch.long)
    c = engine.entry.transformer.config.latent_channel
    req = Cosmos3ActionRequest(ids, mask, ids, mask, video_shape=(3, 16, 24), mode=a.mode, domain_id=7, action_chunk=8, raw_action_dim=10,
                               cond_video_latents=torch.randn(1, c, 3, 16, 24, generator=g), cond_action=torch.randn(1, 8, 64, generator=g),
                               num_inference_steps=a.steps, guidance_scale=3.0)
    engine.step(req)
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    action = engine.step(req)
    torch.cuda.synchronize()
    dist.barrier()
    dt = time.perf_counter() - t0
    if rank == 0:
        print(f"{a.mode} on cfg{a.cfg} x tp{a.tp}: action {tuple(action.shape)} in {dt * 1e3:.1f} ms ({dt / a.steps * 1e3:.1f} ms per denoise step)")
    engine.close()


if __name__ == "__main__":
    main()
