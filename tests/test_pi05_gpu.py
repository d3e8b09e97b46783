"""Pi0.5 on a GPU: the CUDA execution plan against the eager fp32-softmax oracle."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mid_config():
    from phyai_b200.models.pi05.configuration_pi05 import (GemmaExpertConfig, PaliGemmaTextConfig, PI05Config,
                                                           SiglipVisionConfig)

    return PI05Config(
        vision=SiglipVisionConfig(hidden_size=144, num_hidden_layers=2, num_attention_heads=2, intermediate_size=304,
                                  image_size=56, patch_size=14, projection_dim=256),
        text=PaliGemmaTextConfig(hidden_size=256, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                                 head_dim=256, intermediate_size=512, vocab_size=1024),
        expert=GemmaExpertConfig(hidden_size=128, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                                 head_dim=256, intermediate_size=256, adarms_cond_dim=128),
        chunk_size=50, max_action_dim=32, num_inference_steps=4, tokenizer_max_length=48)


def _perturb_norms(eng, g):
    """Random init leaves the RMSNorm weights at identity: perturb them so that folding them into the
    neighbouring GEMM weights is visible, then rebuild the plan's prepared weights."""
    model = eng.entry.model
    with torch.no_grad():
        for mod in (model.paligemma_lm, model.expert_stack):
            for name, p in mod.named_parameters():
                if p.dim() == 1 and "norm" in name and "dense" not in name:
                    p.copy_((torch.randn(p.shape, generator=g) * 0.2).to(p))
    eng.entry.scheduler.plan.build_modulation_tables()


@pytest.mark.parametrize("batch,graph,overlap,expert_kernel", [(1, True, False, False), (2, True, False, False), (2, False, False, False),
                                                               (1, True, True, False), (2, False, True, False),
                                                               (1, True, False, True), (1, True, True, True)])
def test_plan_matches_eager(batch, graph, overlap, expert_kernel, monkeypatch):
    from phyai_b200.models.pi05.plan_pi05 import PI05Plan

    monkeypatch.setattr(PI05Plan, "overlap_first_step", overlap)   # first Euler step on a second stream under the prefix
    monkeypatch.setattr(PI05Plan, "use_expert_kernel", expert_kernel)   # Euler loop as one persistent kernel
    from phyai_b200 import ops
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi05.main_pi05 import PI05Args
    from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request

    cfg = _mid_config()
    # the persistent kernel serves one robot: its cases build a batch-1 engine
    eng = Engine(EngineArgs("pi05", PI05Args(config=cfg, max_batch_size=1 if expert_kernel else 2, inputs_image_shape=[[56, 56, 3]] * 2),
                            EngineConfig(device=DeviceConfig("cuda:0", torch.bfloat16),
                                         runtime=RuntimeConfig(use_cuda_graph=graph))))
    g = torch.Generator().manual_seed(batch)
    _perturb_norms(eng, g)
    assert (eng.entry.scheduler.plan.stack is not None) == expert_kernel
    lens = torch.tensor([40, 7][:batch])
    req = PI05Request((torch.rand(batch, 2, 3, 56, 56, generator=g) * 2 - 1).bfloat16().cuda(),
                      torch.randint(0, 1024, (batch, 48), generator=g).cuda(), lens.cuda(),
                      torch.randn(batch, 50, 32, generator=g).bfloat16().cuda())
    out = eng.step(req)
    out_again = eng.step(req)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    ref = eng.entry.model.sample_actions(req.pixel_values, req.input_ids, lens, req.noise)
    rel = (out.float() - ref.float()).abs().max() / ref.float().abs().max()
    if expert_kernel:   # split-K sums are fp32 reductions in L2: their order, hence the last bit, varies from run to run
        assert (out.float() - out_again.float()).abs().max() <= 2e-2 * ref.float().abs().max()
    else:
        assert torch.equal(out, out_again)
    assert rel < 5e-2, rel
    # a different prompt length re-plans the metadata without re-capturing anything it should not
    req2 = PI05Request(req.pixel_values, req.input_ids, torch.tensor([12, 30][:batch]).cuda(), req.noise)
    out2 = eng.step(req2)
    ref2 = eng.entry.model.sample_actions(req2.pixel_values, req2.input_ids, req2.lang_lens.cpu(), req2.noise)
    rel2 = (out2.float() - ref2.float()).abs().max() / ref2.float().abs().max()
    assert rel2 < 5e-2, rel2
    eng.close()


@pytest.mark.parametrize("batch,overlap", [(1, True), (2, True), (1, False)])
def test_pi0_plan_matches_eager(batch, overlap, monkeypatch):
    from phyai_b200.models.pi05.plan_pi05 import PI05Plan

    monkeypatch.setattr(PI05Plan, "overlap_first_step", overlap)   # state-token pass on a second stream under the prefix
    from phyai_b200 import ops
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi0.configuration_pi0 import PI0Config
    from phyai_b200.models.pi0.main_pi0 import PI0Args
    from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request
    from phyai_b200.models.pi05.configuration_pi05 import GemmaExpertConfig

    c5 = _mid_config()
    cfg = PI0Config(vision=c5.vision, text=c5.text,
                    expert=GemmaExpertConfig(hidden_size=128, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
                                             head_dim=256, intermediate_size=256, use_adarms=False, adarms_cond_dim=128),
                    chunk_size=50, max_state_dim=32, max_action_dim=32, num_inference_steps=4, tokenizer_max_length=48)
    eng = Engine(EngineArgs("pi0", PI0Args(config=cfg, max_batch_size=2, inputs_image_shape=[[56, 56, 3]] * 2),
                            EngineConfig(device=DeviceConfig("cuda:0", torch.bfloat16), runtime=RuntimeConfig(use_cuda_graph=True))))
    g = torch.Generator().manual_seed(10 + batch)
    _perturb_norms(eng, g)
    lens = torch.tensor([33, 9][:batch])
    req = PI0Request((torch.rand(batch, 2, 3, 56, 56, generator=g) * 2 - 1).bfloat16().cuda(),
                     torch.randint(0, 1024, (batch, 48), generator=g).cuda(), lens.cuda(),
                     torch.randn(batch, 32, generator=g).bfloat16().cuda(), torch.randn(batch, 50, 32, generator=g).bfloat16().cuda())
    out = eng.step(req)
    out2 = eng.step(req)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0 and torch.equal(out, out2)
    ref = eng.entry.model.sample_actions(req.pixel_values, req.input_ids, lens, req.state, req.noise)
    rel = (out.float() - ref.float()).abs().max() / ref.float().abs().max()
    assert rel < 5e-2, rel
    eng.close()


@pytest.mark.parametrize("batch", [1, 2])
def test_fp8_block_plan_tracks_the_bf16_plan(batch):
    """Prefix decoder and action expert served in block-scaled fp8 (weights quantised at plan build, activations by
    the norm kernels / the quantiser): the action chunk stays within fp8 noise of the bf16 plan and of the eager oracle."""
    from phyai_b200 import ops
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi05.main_pi05 import PI05Args
    from phyai_b200.models.pi05.scheduler_ws1_pi05 import PI05Request

    cfg = _mid_config()
    ecfg = EngineConfig(device=DeviceConfig("cuda:0", torch.bfloat16), runtime=RuntimeConfig(use_cuda_graph=True))
    g = torch.Generator().manual_seed(40 + batch)
    lens = torch.tensor([31, 5][:batch])
    req = PI05Request((torch.rand(batch, 2, 3, 56, 56, generator=g) * 2 - 1).bfloat16().cuda(),
                      torch.randint(0, 1024, (batch, 48), generator=g).cuda(), lens.cuda(),
                      torch.randn(batch, 50, 32, generator=g).bfloat16().cuda())
    outs = {}
    for q in ("fp8_block", None):
        eng = Engine(EngineArgs("pi05", PI05Args(config=cfg, max_batch_size=2, inputs_image_shape=[[56, 56, 3]] * 2, quantization=q), ecfg))
        plan = eng.entry.scheduler.plan
        assert plan.fp8 == (q == "fp8_block")
        if q:
            assert plan.w8["p.qkv"][0][0].dtype == torch.float8_e4m3fn and not plan.fold_norms
        outs[q] = eng.step(req).float()
        again = eng.step(req).float()
        torch.cuda.synchronize()
        assert ops.kernel_status() == 0 and torch.equal(outs[q], again)
        if q is None:
            ref = eng.entry.model.sample_actions(req.pixel_values, req.input_ids, lens, req.noise).float()
        eng.close()
    scale = ref.abs().max()
    assert torch.isfinite(outs["fp8_block"]).all()
    assert (outs["fp8_block"] - outs[None]).abs().max() < 0.12 * scale       # e4m3 has 3 mantissa bits; 6 blocks x 4 steps deep
    assert (outs["fp8_block"] - ref).abs().mean() < 0.03 * scale
