"""Cosmos3 on a B200: the fused GEN path (own kernels) against the eager PyTorch path of the same weights."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def small_real_config(**over):
    from phyai_b200.models.cosmos3 import Cosmos3Config

    base = dict(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                intermediate_size=1024, vocab_size=512, mrope_section=(24, 20, 20), latent_channel=16, latent_patch_size=2,
                patch_latent_dim=64, action_dim=32, num_embodiment_domains=4, sound_dim=16)
    base.update(over)
    return Cosmos3Config(**base)


@pytest.fixture()
def engine_cuda():
    from phyai_b200 import parallel as P
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers import linear as L

    init_engine_config(EngineConfig(device=DeviceConfig("cuda", torch.bfloat16)))
    P.init((1,), ("tp",), device="cuda")
    L.init()
    yield
    P.shutdown()


@pytest.mark.parametrize("variant", ["video", "action", "sound"])
def test_fused_gen_path_matches_eager(engine_cuda, variant):
    from phyai_b200 import ops
    from phyai_b200.models.cosmos3 import Cosmos3Transformer

    cfg = small_real_config(action_gen=variant == "action", sound_gen=variant == "sound")
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    assert model.use_fused
    g = torch.Generator().manual_seed(0)
    B, vs = 2, (3, 16, 24)
    ids = torch.randint(0, 512, (B, 20), generator=g).cuda()
    mask = torch.ones(B, 20, dtype=torch.long, device="cuda")
    lat = torch.randn(B, 16, *vs, generator=g).cuda().bfloat16()
    t = torch.full((B,), 500.0, device="cuda")
    kw, ckw = {}, {}
    if variant == "action":
        kw = dict(action_latents=torch.randn(B, 8, 32, generator=g).cuda().bfloat16(), action_domain_id=torch.tensor([1, 3]).cuda(),
                  noisy_frame_mask=torch.tensor([[0, 1, 1]] * B, dtype=torch.bool).cuda())
        ckw = dict(action_len=8)
    if variant == "sound":
        kw = dict(sound_latents=torch.randn(B, 10, 16, generator=g).cuda().bfloat16())
        ckw = dict(sound_len=10, sound_fps=25.0)
    cond = model.encode_condition(ids, mask, vs, 24.0, **ckw)
    got = model(lat, t, cond, **kw)
    got2 = model(lat, t, cond, **kw)           # second call reuses the cached workspace and K/V buffers
    model.use_fused = False
    want = model(lat, t, model.encode_condition(ids, mask, vs, 24.0, **ckw), **kw)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    got, got2, want = [x if isinstance(x, tuple) else (x,) for x in (got, got2, want)]
    for a, a2, b in zip(got, got2, want):
        scale = b.float().abs().max().item()
        assert torch.isfinite(a.float()).all()
        assert (a.float() - b.float()).abs().max().item() <= 0.05 * scale + 1e-3
        assert torch.equal(a, a2)


def test_fp8_block_gen_path_tracks_bf16(engine_cuda):
    """The generation tower with block-scaled fp8 projections (weights quantised from the bf16 tensors on first use)
    stays within e4m3 noise of the bf16 fused path and of the eager PyTorch path."""
    from phyai_b200 import ops
    from phyai_b200.models.cosmos3 import Cosmos3Transformer

    cfg = small_real_config()
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    g = torch.Generator().manual_seed(1)
    B, vs = 1, (3, 16, 24)
    ids = torch.randint(0, 512, (B, 20), generator=g).cuda()
    mask = torch.ones(B, 20, dtype=torch.long, device="cuda")
    lat = torch.randn(B, 16, *vs, generator=g).cuda().bfloat16()
    t = torch.full((B,), 500.0, device="cuda")
    bf16_out = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    model.serve_fp8 = True
    fp8_out = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    fp8_again = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    model.serve_fp8, model.use_fused = False, False
    eager = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert model.gen_layers[0]._w8["qkv"][0].dtype == torch.float8_e4m3fn
    scale = eager.abs().max().item()
    assert torch.isfinite(fp8_out).all() and torch.equal(fp8_out, fp8_again)
    assert (fp8_out - bf16_out).abs().max().item() <= 0.12 * scale
    assert (fp8_out - eager).abs().mean().item() <= 0.03 * scale
    assert (fp8_out - bf16_out).abs().max().item() > 0          # it is a different computation


def test_nvfp4_gen_path_tracks_bf16(engine_cuda):
    """The generation tower with NVFP4 projections on the block-scaled GEMM (weights and activations quantised by this
    package's kernel) stays within four-bit noise of the bf16 fused path."""
    from phyai_b200 import ops
    from phyai_b200.models.cosmos3 import Cosmos3Transformer
    from phyai_b200.ops import nvfp4

    if not nvfp4.available():
        pytest.skip("phyai_b200/_blockscaled is not built in this checkout")
    cfg = small_real_config()
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    g = torch.Generator().manual_seed(1)
    B, vs = 1, (3, 16, 24)
    ids = torch.randint(0, 512, (B, 20), generator=g).cuda()
    mask = torch.ones(B, 20, dtype=torch.long, device="cuda")
    lat = torch.randn(B, 16, *vs, generator=g).cuda().bfloat16()
    t = torch.full((B,), 500.0, device="cuda")
    bf16_out = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    model.serve_nvfp4 = True
    out = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    again = model(lat, t, model.encode_condition(ids, mask, vs, 24.0)).float()
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert model.gen_layers[0]._w4["qkv"][0].dtype == torch.uint8
    scale = bf16_out.abs().max().item()
    assert torch.isfinite(out).all() and torch.equal(out, again)
    # four-bit weights AND activations on random weights without outlier structure: every projection carries a few per
    # cent of noise, so the towers agree in direction, not to bf16 precision (the GEMM itself is checked exactly against
    # its dequantised statement in test_nvfp4_gpu.py)
    cos = torch.nn.functional.cosine_similarity(out.flatten(), bf16_out.flatten(), dim=0).item()
    assert cos > 0.9, cos
    assert (out - bf16_out).abs().mean().item() <= 0.15 * scale
    assert (out - bf16_out).abs().max().item() > 0


def test_policy_scheduler_and_vae_on_gpu(engine_cuda):
    from phyai_b200.models.cosmos3 import Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3Transformer, Cosmos3WanVAEConfig
    from phyai_b200.models.cosmos3.vae_wan import Cosmos3WanVAE

    cfg = small_real_config(action_gen=True)
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    sch = Cosmos3PolicyScheduler(model, device="cuda")
    sch.setup()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 512, (1, 20), generator=g)
    mask = torch.ones(1, 20, dtype=torch.long)
    req = Cosmos3ActionRequest(ids, mask, ids, mask, video_shape=(2, 16, 24), mode="policy", domain_id=1, action_chunk=8,
                               raw_action_dim=7, action_dim=32, cond_video_latents=torch.randn(1, 16, 2, 16, 24, generator=g),
                               num_inference_steps=4, guidance_scale=3.0)
    out = sch.step(req)
    assert out["action"].shape == (1, 8, 7) and torch.isfinite(out["action"].float()).all()
    vcfg = Cosmos3WanVAEConfig(z_dim=16, decoder_base_dim=32, base_dim=32, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    vae = Cosmos3WanVAE(vcfg, device="cuda", dtype=torch.bfloat16).eval()
    for p in vae.parameters():
        if p.dim() > 1 and p.shape[1:].numel() > 1:
            p.data.normal_(0, 1.0 / p.shape[1:].numel() ** 0.5)
    pix = vae.decode(out["video"])
    assert pix.shape == (1, 3, 5, 256, 384) and torch.isfinite(pix.float()).all()
    chunked = vae.decode(out["video"], frames_per_chunk=1)
    assert (pix.float() - chunked.float()).abs().max().item() < 0.1


@pytest.mark.parametrize("mode", ["t2v_cond_frames", "policy", "forward_dynamics"])
def test_fused_sampler_matches_tensor_op_sampler(engine_cuda, mode, monkeypatch):
    """Whole requests with the one-kernel UniPC update against the same requests with the tensor-op sampler."""
    from phyai_b200.models.cosmos3 import (Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3T2VRequest, Cosmos3T2VScheduler,
                                           Cosmos3Transformer)

    policy = mode != "t2v_cond_frames"
    cfg = small_real_config(action_gen=policy)
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    g = torch.Generator().manual_seed(0)
    ids, nids = torch.randint(0, 512, (1, 20), generator=g), torch.randint(0, 512, (1, 20), generator=g)
    mask = torch.ones(1, 20, dtype=torch.long)
    outs = []
    for fused in (True, False):
        if policy:
            sch = Cosmos3PolicyScheduler(model, device="cuda")
            monkeypatch.setattr(sch, "fused_sampler", fused, raising=False)
            sch.setup()
            req = Cosmos3ActionRequest(ids, mask, nids, mask, video_shape=(2, 16, 24), mode=mode if mode != "policy" else "policy",
                                       domain_id=1, action_chunk=8, raw_action_dim=7, action_dim=32,
                                       cond_video_latents=torch.randn(1, 16, 2, 16, 24, generator=torch.Generator().manual_seed(1)),
                                       cond_action=torch.randn(1, 8, 32, generator=torch.Generator().manual_seed(2)),
                                       num_inference_steps=4, guidance_scale=3.0)
            out = sch.step(req)
            outs.append((out["video"].float().cpu(), out["action"].float().cpu()))
        else:
            sch = Cosmos3T2VScheduler(model, device="cuda")
            monkeypatch.setattr(sch, "fused_sampler", fused, raising=False)
            sch.setup()
            req = Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(3, 16, 24), num_inference_steps=4, guidance_scale=4.0,
                                    cond_latents=torch.randn(1, 16, 3, 16, 24, generator=torch.Generator().manual_seed(1)),
                                    cond_frame_indexes=(0,))
            outs.append((sch.step(req).float().cpu(),))
    for a, b in zip(*outs):
        assert torch.isfinite(a).all()
        scale = b.abs().mean().item()
        assert (a - b).abs().mean().item() <= 0.03 * scale, ((a - b).abs().mean().item(), scale)


@pytest.mark.parametrize("mode", ["t2v", "t2v_sound", "policy"])
def test_step_graph_matches_launch_by_launch(engine_cuda, mode, monkeypatch):
    """A request whose steps replay one CUDA graph (captured at its second step) against the same request issued launch
    by launch: same kernels on the same buffers, so the latents are equal bit for bit."""
    from phyai_b200 import ops
    from phyai_b200.models.cosmos3 import (Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3T2VRequest, Cosmos3T2VScheduler,
                                           Cosmos3Transformer)

    policy = mode == "policy"
    cfg = small_real_config(action_gen=policy, sound_gen=mode == "t2v_sound")
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    g = torch.Generator().manual_seed(0)
    ids, nids = torch.randint(0, 512, (1, 20), generator=g), torch.randint(0, 512, (1, 20), generator=g)
    mask = torch.ones(1, 20, dtype=torch.long)
    steps, outs = 5, []
    for graphed in (True, False, True):
        if policy:
            sch = Cosmos3PolicyScheduler(model, device="cuda")
            monkeypatch.setattr(sch, "graph_steps", graphed, raising=False)
            sch.setup()
            req = Cosmos3ActionRequest(ids, mask, nids, mask, video_shape=(2, 16, 24), mode="policy", domain_id=1, action_chunk=8,
                                       raw_action_dim=7, action_dim=32, num_inference_steps=steps, guidance_scale=3.0,
                                       cond_video_latents=torch.randn(1, 16, 2, 16, 24, generator=torch.Generator().manual_seed(1)))
            out = sch.step(req)
            outs.append((out["video"].clone(), out["action"].clone()))
        else:
            sch = Cosmos3T2VScheduler(model, device="cuda")
            monkeypatch.setattr(sch, "graph_steps", graphed, raising=False)
            sch.setup()
            kw = dict(sound_frames=10, sound_dim=16, sound_latent_fps=25.0) if mode == "t2v_sound" else {}
            req = Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(3, 16, 24), num_inference_steps=steps, guidance_scale=4.0, **kw)
            out = sch.step(req)
            outs.append((out["video"].clone(), out["sound"].clone()) if isinstance(out, dict) else (out.clone(),))
        # the first step is eager, the second is captured and replayed, the rest replay
        assert sch.last_graph_replays == (steps - 1 if graphed else 0)
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    for a, b, c in zip(*outs):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b) and torch.equal(a, c)


@pytest.mark.parametrize("mode", ["t2v_cond_frames", "policy"])
def test_step_graph_serves_following_requests(engine_cuda, mode, monkeypatch):
    """One scheduler, three requests of one geometry with different prompts, noise, clean frames and domain: from the
    second request on every step is a replay of the graph captured in the first, reading the slot's buffers; each result
    equals the one of a scheduler that issues every launch from the host."""
    from phyai_b200 import ops
    from phyai_b200.models.cosmos3 import (Cosmos3ActionRequest, Cosmos3PolicyScheduler, Cosmos3T2VRequest, Cosmos3T2VScheduler,
                                           Cosmos3Transformer)

    policy = mode == "policy"
    cfg = small_real_config(action_gen=policy)
    model = Cosmos3Transformer(cfg, params_dtype=torch.bfloat16, device="cuda").eval().init_random(2, std=0.05)
    mask = torch.ones(1, 20, dtype=torch.long)

    def request(seed: int, steps: int):
        g = torch.Generator().manual_seed(seed)
        ids, nids = torch.randint(0, 512, (1, 20), generator=g), torch.randint(0, 512, (1, 20), generator=g)
        if policy:
            return Cosmos3ActionRequest(ids, mask, nids, mask, video_shape=(2, 16, 24), mode="policy", domain_id=seed % 4, action_chunk=8,
                                        raw_action_dim=7, action_dim=32, num_inference_steps=steps, guidance_scale=3.0, seed=seed,
                                        cond_video_latents=torch.randn(1, 16, 2, 16, 24, generator=g))
        return Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(3, 16, 24), num_inference_steps=steps, guidance_scale=4.0,
                                 seed=seed, cond_latents=torch.randn(1, 16, 3, 16, 24, generator=g), cond_frame_indexes=(seed % 3,))

    def tensors(out):
        return [out["video"], out["action"]] if isinstance(out, dict) else [out]

    cls = Cosmos3PolicyScheduler if policy else Cosmos3T2VScheduler
    plan = [(1, 4), (2, 5), (3, 3)]
    graphed, eager = cls(model, device="cuda"), cls(model, device="cuda")
    monkeypatch.setattr(eager, "graph_steps", False, raising=False)
    graphed.setup()
    eager.setup()
    got = []
    for i, (seed, steps) in enumerate(plan):
        got.append(tensors(graphed.step(request(seed, steps))))
        assert graphed.last_graph_replays == (steps - 1 if i == 0 else steps)
    want = [tensors(eager.step(request(seed, steps))) for seed, steps in plan]
    assert eager.last_graph_replays == 0
    torch.cuda.synchronize()
    assert ops.kernel_status() == 0
    assert len(graphed._loop_slots) == 1
    for a, b in zip(got, want):
        for x, y in zip(a, b):
            assert torch.isfinite(x.float()).all()
            assert torch.equal(x, y), (x.float() - y.float()).abs().max().item()
