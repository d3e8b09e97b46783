"""Cosmos3 text-to-video over a CFG x TP mesh (plugin ``cosmos3_wn``), one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/cosmos3/run_cosmos3_wn.py --tp 4 --cfg 2 [--checkpoint DIR --prompt "..."]

Every rank builds the same request (prompts are tokenised on every rank, the starting noise is seeded); the
conditional and unconditional branches run on different ``cfg`` groups and exchange their velocity predictions
through peer memory, the transformer layers are tensor parallel inside a group (GEMM epilogues store into the
peers' slots, the owner reduces, norms and shares the rows), the VAE decodes spatial tiles on all ranks.
Rank 0 reports ``seconds / steps`` the way the reference example does
(examples/cosmos3/run_cosmos3_wn.py:244-255) and saves the clip.
Without ``--checkpoint`` a small random-weight model shows the flow (noise in, noise out).
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
from phyai_b200.models.cosmos3 import Cosmos3Config, Cosmos3T2VRequest, Cosmos3WanVAEConfig, pixel_to_latent_shape  # noqa: E402
from phyai_b200.models.cosmos3.main_cosmos3_wn import Cosmos3WNArgs  # noqa: E402
from phyai_b200.tools.cosmos3 import Cosmos3GenerationPostProcessor, Cosmos3Processor  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--prompt", default="A robot arm stacks two wooden blocks on a table.")
    ap.add_argument("--frames", type=int, default=17)
    ap.add_argument("--height", type=int, default=256)
    ap.add_argument("--width", type=int, default=320)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--guidance", type=float, default=6.0)
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--cfg", type=int, default=1)
    ap.add_argument("--out", default="cosmos3_clip.npz")
    a = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if world != a.tp * a.cfg:
        raise SystemExit(f"tp {a.tp} x cfg {a.cfg} needs {a.tp * a.cfg} ranks, launched {world}")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    cfg = EngineConfig(device=DeviceConfig(dev, torch.bfloat16), parallel=ParallelConfig(world_size=world, cfg_size=a.cfg, tp_size=a.tp))
    if a.checkpoint:
        args = Cosmos3WNArgs(checkpoint_dir=a.checkpoint)
        proc = Cosmos3Processor(str(Path(a.checkpoint) / "text_tokenizer"), fps=24, num_frames=a.frames, height=a.height, width=a.width)
        pos, neg = proc.tokenize_pair(a.prompt, device=dev)
        ids, mask, nids, nmask = pos.text_ids, pos.text_mask, neg.text_ids, neg.text_mask
    else:
        small = Cosmos3Config(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                              intermediate_size=1024, vocab_size=512, latent_channel=16, latent_patch_size=2, patch_latent_dim=64)
        vae = Cosmos3WanVAEConfig(z_dim=16, decoder_base_dim=32, base_dim=32, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
        args = Cosmos3WNArgs(config=small, vae_config=vae, load_sound=False)
        g = torch.Generator().manual_seed(0)              # the same prompt ids on every rank
        ids, nids = torch.randint(0, 512, (1, 24), generator=g).to(dev), torch.randint(0, 512, (1, 24), generator=g).to(dev)
        mask = nmask = torch.ones(1, 24, dtype=torch.long, device=dev)
    engine = Engine(EngineArgs("cosmos3_wn", args, cfg))
    req = Cosmos3T2VRequest(ids, mask, nids, nmask, video_shape=pixel_to_latent_shape(a.frames, a.height, a.width),
                            num_inference_steps=a.steps, guidance_scale=a.guidance, seed=0)
    engine.step(req)                                     # warm-up: lazy communicator and peer-memory set-up
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    pixels = engine.step(req)
    torch.cuda.synchronize()
    dist.barrier()
    dt = time.perf_counter() - t0
    if rank == 0:
        post = Cosmos3GenerationPostProcessor(fps=24)
        out = post.postprocess(pixels)
        post.save_npz(out["frames"], a.out)
        print(f"cfg{a.cfg} x tp{a.tp}: {tuple(out['frames'].shape)} frames in {dt:.2f} s "
              f"({dt / a.steps * 1e3:.1f} ms per denoise step incl. encode / decode) -> {a.out}")
    engine.close()


if __name__ == "__main__":
    main()
