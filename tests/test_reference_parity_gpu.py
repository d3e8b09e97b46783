"""One synthetic checkpoint, two implementations: this package and the unmodified reference installed under
``baseline/_ref`` load the same folder through their public ``Engine`` APIs and must agree on the action chunk.

What it pins down: the checkpoint key map (fused QKV / gate-up legs, AdaRMS dense layers, SigLIP names), the
request contract and the numerics of the whole request (vision tower, prefix, 4 Euler steps) across code bases.
Skipped where the reference is not installed.
"""

import json
import sys
from dataclasses import asdict
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"


def _mid_kwargs():
    return dict(
        vision=dict(hidden_size=144, num_hidden_layers=2, num_attention_heads=2, intermediate_size=304, image_size=56,
                    patch_size=14, projection_dim=256),
        text=dict(hidden_size=256, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1, head_dim=256,
                  intermediate_size=512, vocab_size=1024),
        expert=dict(hidden_size=128, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1, head_dim=256,
                    intermediate_size=256, adarms_cond_dim=128),
        top=dict(chunk_size=50, max_action_dim=32, num_inference_steps=4, tokenizer_max_length=48))


@pytest.mark.skipif(not (REF / "phyai").is_dir(), reason="the reference is not installed under baseline/_ref")
def test_pi05_same_checkpoint_same_actions(tmp_path):
    kw = _mid_kwargs()
    g = torch.Generator().manual_seed(0)
    pix = (torch.rand(1, 2, 3, 56, 56, generator=g) * 2 - 1).bfloat16().cuda()
    ids = torch.randint(0, 1024, (1, 48), generator=g).cuda()
    lens = torch.tensor([29]).cuda()
    noise = torch.randn(1, 50, 32, generator=g).bfloat16().cuda()

    # ---- this package: build, write the checkpoint from its own key index, load it back, run
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi05.configuration_pi05 import (GemmaExpertConfig, PaliGemmaTextConfig, PI05Config,
                                                           SiglipVisionConfig)
    from phyai_b200.models.pi05.main_pi05 import PI05Args
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model
    from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request
    from phyai_b200.weights import synthetic_state_dict, write_checkpoint

    cfg = PI05Config(vision=SiglipVisionConfig(**kw["vision"]), text=PaliGemmaTextConfig(**kw["text"]),
                     expert=GemmaExpertConfig(**kw["expert"]), **kw["top"])
    probe = PI05Model(cfg)
    state = synthetic_state_dict(probe, seed=3, std=0.05)
    # identity norms and zero modulation would hide key mix-ups: make every tensor random
    gs = torch.Generator().manual_seed(4)
    for k, t in state.items():
        if float(t.float().abs().sum()) == 0 or bool((t == 1).all()):
            state[k] = (torch.randn(t.shape, generator=gs) * 0.1).to(t.dtype)
    ckpt = write_checkpoint(tmp_path / "pi05_mid", state)
    del probe

    ecfg = EngineConfig(device=DeviceConfig("cuda:0", torch.bfloat16), runtime=RuntimeConfig(use_cuda_graph=True))
    eng = Engine(EngineArgs("pi05", PI05Args(checkpoint_dir=str(ckpt), config=cfg, max_batch_size=1,
                                             inputs_image_shape=[[56, 56, 3]] * 2), ecfg))
    ours = eng.step(PI05Request(pix, ids, lens, noise)).float().cpu()
    eng.close()

    # ---- the reference, from the same folder
    sys.path.insert(0, str(REF))
    try:
        from phyai.engine import Engine as REngine, EngineArgs as REngineArgs
        from phyai.engine_config import DeviceConfig as RDev, EngineConfig as RCfg, RuntimeConfig as RRun
        from phyai.models.pi05.configuration_pi05 import (GemmaExpertConfig as RE, PaliGemmaTextConfig as RT, PI05Config as RC,
                                                          SiglipVisionConfig as RV)
        from phyai.models.pi05.main_pi05 import PI05Args as RArgs
        from phyai.models.pi05.scheduler_ws1_pi05 import PI05Request as RReq

        rcfg = RC(vision=RV(**kw["vision"]), text=RT(**kw["text"]), expert=RE(**kw["expert"]), **kw["top"])
        reng = REngine(REngineArgs("pi05", RArgs(checkpoint_dir=str(ckpt), config=rcfg, max_batch_size=1,
                                                 inputs_image_shape=[[56, 56, 3]] * 2),
                                   RCfg(device=RDev(target="cuda:0", params_dtype=torch.bfloat16), runtime=RRun(use_cuda_graph=False))))
        theirs = reng.step(RReq(pixel_values=pix, input_ids=ids, lang_lens=lens, noise=noise)).float().cpu()
        reng.close()
    finally:
        sys.path.remove(str(REF))
    assert torch.isfinite(ours).all() and torch.isfinite(theirs).all()
    torch.testing.assert_close(ours, theirs, atol=6e-2, rtol=6e-2)
    assert float((ours - theirs).abs().mean()) < 1.5e-2
