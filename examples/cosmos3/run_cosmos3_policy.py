"""Cosmos3 action inference (policy / forward dynamics / inverse dynamics) with a small random-weight model.

    python examples/cosmos3/run_cosmos3_policy.py [--mode policy] [--checkpoint DIR [--image FILE --task "..."]]

With a checkpoint (its ``text_tokenizer/`` and VAE) an observation image and a task string go through
``Cosmos3PolicyProcessor``: the frame is brought to the training bucket nearest to its aspect ratio, the caption is
tokenised, and the predicted action chunk comes back cut to the embodiment's width.
"""

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import torch  # noqa: E402

from phyai_b200.engine import Engine, EngineArgs  # noqa: E402
from phyai_b200.engine_config import DeviceConfig, EngineConfig  # noqa: E402
from phyai_b200.models.cosmos3 import ACTION_MODES, Cosmos3ActionRequest, Cosmos3Config, pixel_to_latent_shape  # noqa: E402
from phyai_b200.models.cosmos3.main_cosmos3_policy import Cosmos3PolicyArgs  # noqa: E402
from phyai_b200.tools.cosmos3 import Cosmos3PolicyProcessor  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=ACTION_MODES, default="policy")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--image", default=None, help="observation frame (with --checkpoint)")
    ap.add_argument("--task", default="pick up the cup")
    ap.add_argument("--domain", default="bridge_orig_lerobot")
    a = ap.parse_args()
    dev = "cuda:0"
    small = Cosmos3Config(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=1024,
                          vocab_size=512, latent_channel=16, latent_patch_size=2, patch_latent_dim=64, action_gen=True, action_dim=64)
    args = Cosmos3PolicyArgs(checkpoint_dir=a.checkpoint) if a.checkpoint else Cosmos3PolicyArgs(config=small)
    engine = Engine(EngineArgs("cosmos3_policy", args, EngineConfig(device=DeviceConfig(dev, torch.bfloat16))))
    if a.checkpoint and a.image:
        proc = Cosmos3PolicyProcessor(tokenizer_name_or_path=str(Path(a.checkpoint) / "text_tokenizer"), mode=a.mode, domain_name=a.domain,
                                      action_chunk_size=16, image_size=480, prompt_format="json", fps=10.0)
        p = proc.preprocess({"images": a.image, "task": a.task})
        req = Cosmos3ActionRequest(p.text_ids, p.text_mask, p.neg_text_ids, p.neg_text_mask, video_shape=pixel_to_latent_shape(*p.video_shape),
                                   mode=p.mode, domain_id=p.domain_id, action_chunk=p.action_chunk, raw_action_dim=p.raw_action_dim,
                                   cond_video_pixels=p.pixel_values, cond_action=p.cond_action, cond_frame_indexes=p.cond_frame_indexes,
                                   num_inference_steps=10, guidance_scale=3.0)
        out = proc.postprocess(engine.entry.scheduler.step(req))
        print(a.mode, "->", tuple(out["action"].shape))
        engine.close()
        return
    ids, mask = torch.randint(0, 512, (1, 32)), torch.ones(1, 32, dtype=torch.long)
    c = engine.entry.transformer.config.latent_channel
    req = Cosmos3ActionRequest(ids, mask, ids, mask, video_shape=(3, 16, 24), mode=a.mode, domain_id=7, action_chunk=8, raw_action_dim=10,
                               cond_video_latents=torch.randn(1, c, 3, 16, 24), cond_action=torch.randn(1, 8, 64), num_inference_steps=4, guidance_scale=3.0)
    action = engine.step(req)
    print(a.mode, "->", tuple(action.shape))
    engine.close()


if __name__ == "__main__":
    main()
