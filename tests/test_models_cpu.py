"""CPU fp32 model tests: the cached-prefix execution equals one masked joint forward written
independently with plain torch ops on the same weights."""

import math

import pytest
import torch
import torch.nn.functional as F

from phyai_b200.ops import ref


def _rope(x, pos, theta=10000.0):
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    rot = torch.cat([-x[..., d // 2:], x[..., : d // 2]], -1)
    return x * cos + rot * sin


def _gemma_block(h, p, pos, mask, heads, kv_heads, hd, eps, norm):
    x = norm(h, p["ln1"])
    q = (x @ p["wq"].t()).reshape(-1, heads, hd)
    k = (x @ p["wk"].t()).reshape(-1, kv_heads, hd)
    v = (x @ p["wv"].t()).reshape(-1, kv_heads, hd)
    q, k = _rope(q, pos), _rope(k, pos)
    k, v = k.repeat_interleave(heads // kv_heads, 1), v.repeat_interleave(heads // kv_heads, 1)
    s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
    s = s.masked_fill(~mask[None], float("-inf"))
    a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(h.shape[0], -1)
    return a @ p["wo"].t(), x


def _weights(layer):
    a = layer.attn
    w = a.qkv.weight.data
    gu = layer.mlp.gate_up.weight.data
    return dict(wq=w[: a.qkv.q_size], wk=w[a.qkv.q_size: a.qkv.q_size + a.qkv.kv_size], wv=w[a.qkv.q_size + a.qkv.kv_size:],
                wo=a.o.weight.data, wg=gu[0::2], wu=gu[1::2], wd=layer.mlp.down.weight.data)


def _gemma_norm(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1 + w)


def _mlp(x, p):
    return (F.gelu(x @ p["wg"].t(), approximate="tanh") * (x @ p["wu"].t())) @ p["wd"].t()


def test_pi0_cached_path_equals_masked_joint_forward():
    from phyai_b200.models.pi0.configuration_pi0 import tiny_pi0_config
    from phyai_b200.models.pi0.modeling_pi0 import PI0Model

    cfg = tiny_pi0_config(num_inference_steps=1)
    m = PI0Model(cfg).init_random(3)
    for l in list(m.paligemma_lm.layers) + list(m.expert_stack.layers):
        l.input_layernorm.weight.data.normal_(0, 0.2)
        l.post_attention_layernorm.weight.data.normal_(0, 0.2)
    g = torch.Generator().manual_seed(0)
    pix = torch.rand(2, 3, 56, 56, generator=g) * 2 - 1
    ids = torch.randint(0, 1024, (16,), generator=g)
    state, noise = torch.randn(8, generator=g), torch.randn(10, 8, generator=g)
    L = 11
    got = m.sample_actions(pix[None], ids[None], torch.tensor([L]), state[None], noise[None])[0]

    # ---- independent joint forward: rows = [prefix | state | actions], two weight sets, one block mask
    img = m.vision(pix).reshape(-1, cfg.text.hidden_size)
    lang = m.paligemma_lm.embed_tokens.data[ids[:L]] * math.sqrt(cfg.text.hidden_size)
    hp = torch.cat([img, lang])
    P, C = hp.shape[0], cfg.chunk_size
    t = torch.ones(1)
    hs = state[None] @ m.heads.state_proj.weight.t() + m.heads.state_proj.bias
    a = noise @ m.heads.action_in_proj.weight.t() + m.heads.action_in_proj.bias
    te = ref.sinusoidal_time_embedding(t, cfg.expert.hidden_size, cfg.min_period, cfg.max_period).expand(C, -1)
    ha = F.silu(torch.cat([a, te], -1) @ m.heads.action_time_mlp_in.weight.t() + m.heads.action_time_mlp_in.bias)
    ha = ha @ m.heads.action_time_mlp_out.weight.t() + m.heads.action_time_mlp_out.bias
    he = torch.cat([hs, ha])
    n = P + 1 + C
    mask = torch.zeros(n, n, dtype=torch.bool)
    mask[:P, :P] = True                      # prefix: bidirectional, blind to the suffix
    mask[P, : P + 1] = True                  # state: prefix + itself
    mask[P + 1:, :] = True                   # actions: everything
    pos = torch.arange(n)
    H, KV, hd = cfg.text.num_attention_heads, cfg.text.num_key_value_heads, cfg.text.head_dim
    for lp, le in zip(m.paligemma_lm.layers, m.expert_stack.layers):
        wp, we = _weights(lp), _weights(le)
        xp = _gemma_norm(hp, lp.input_layernorm.weight.data)
        xe = _gemma_norm(he, le.input_layernorm.weight.data)
        q = torch.cat([(xp @ wp["wq"].t()), (xe @ we["wq"].t())]).reshape(n, H, hd)
        k = torch.cat([(xp @ wp["wk"].t()), (xe @ we["wk"].t())]).reshape(n, KV, hd)
        v = torch.cat([(xp @ wp["wv"].t()), (xe @ we["wv"].t())]).reshape(n, KV, hd)
        q, k = _rope(q, pos), _rope(k, pos)
        kk, vv = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(hd)
        att = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(~mask[None], float("-inf")), -1), vv).reshape(n, -1)
        hp = hp + att[:P] @ wp["wo"].t()
        he = he + att[P:] @ we["wo"].t()
        hp = hp + _mlp(_gemma_norm(hp, lp.post_attention_layernorm.weight.data), wp)
        he = he + _mlp(_gemma_norm(he, le.post_attention_layernorm.weight.data), we)
    out = _gemma_norm(he[1:], m.expert_stack.norm.weight.data) @ m.heads.action_out_proj.weight.t() + m.heads.action_out_proj.bias
    want = noise - out
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_pi05_tiny_runs_and_is_deterministic():
    from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model

    m = PI05Model(tiny_pi05_config()).init_random(0)
    for l in m.expert_stack.layers:
        for n_ in (l.input_layernorm, l.post_attention_layernorm):
            n_.dense.weight.data.normal_(0, 0.05); n_.dense.bias.data.normal_(0, 0.05)
    g = torch.Generator().manual_seed(1)
    args = (torch.rand(2, 2, 3, 56, 56, generator=g) * 2 - 1, torch.randint(0, 1024, (2, 16), generator=g),
            torch.tensor([16, 5]), torch.randn(2, 10, 8, generator=g))
    a, b = m.sample_actions(*args), m.sample_actions(*args)
    assert torch.equal(a, b) and torch.isfinite(a).all()
    # the padding tokens of the shorter prompt must not matter
    ids2 = args[1].clone(); ids2[1, 5:] = 7
    c = m.sample_actions(args[0], ids2, args[2], args[3])
    assert torch.allclose(a, c)


def test_engine_plugins_on_cpu(tmp_path):
    from phyai_b200 import DeviceConfig, Engine, EngineArgs, EngineConfig, RuntimeConfig
    from phyai_b200.models.pi0.configuration_pi0 import tiny_pi0_config
    from phyai_b200.models.pi0.main_pi0 import PI0Args
    from phyai_b200.models.pi0.modeling_pi0 import PI0Model
    from phyai_b200.models.pi0.scheduler_ws1_pi0 import PI0Request
    from phyai_b200.weights import synthetic_state_dict, write_checkpoint

    cfg = tiny_pi0_config()
    ec = EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False))
    ref_model = PI0Model(cfg)
    state = synthetic_state_dict(ref_model, seed=5)
    state["model.paligemma_with_expert.gemma_expert.lm_head.weight"] = torch.zeros(4, 4)   # upstream extra, dropped
    state = {("model." + k if not k.startswith("model.") else k): v for k, v in state.items()}
    write_checkpoint(tmp_path, state, cfg.to_dict())
    eng = Engine(EngineArgs("pi0", PI0Args(checkpoint_dir=tmp_path, max_batch_size=1, inputs_image_shape=[[56, 56, 3]] * 2), ec))
    g = torch.Generator().manual_seed(0)
    req = PI0Request(torch.rand(1, 2, 3, 56, 56, generator=g), torch.randint(0, 1024, (1, 16), generator=g),
                     torch.tensor([8]), torch.randn(1, 8, generator=g), torch.randn(1, 10, 8, generator=g))
    out = eng.step(req)
    assert out.shape == (1, 10, 8) and torch.isfinite(out).all()
    with pytest.raises(ValueError):
        eng.step(PI0Request(req.pixel_values, req.input_ids, req.lang_lens, torch.randn(1, 9), req.noise))
    eng.close()
    with pytest.raises(RuntimeError):
        eng.step(req)
    with pytest.raises(KeyError):
        Engine(EngineArgs("nope", PI0Args(), ec))
    with pytest.raises(TypeError):
        from phyai_b200.models.pi05.main_pi05 import PI05Args
        Engine(EngineArgs("pi0", PI05Args(), ec))


def test_tensor_parallel_camera_split_keeps_order_and_covers_all():
    """The tensor-parallel Pi0.5 plan gives each rank a contiguous block of cameras; equal padded blocks gathered in rank
    order must list every camera once, in order."""
    from phyai_b200.models.pi05.plan_tp_pi05 import split_cameras

    for n in (1, 2, 3, 4, 6, 9):
        for world in (2, 3, 4, 8):
            seen = []
            for rank in range(world):
                per, lo, hi = split_cameras(n, world, rank)
                assert per == -(-n // world) and 0 <= lo <= hi <= n and hi - lo <= per
                # position of camera g in the gathered (world * per)-block matrix is rank * per + (g - lo) == g
                seen += [(rank * per + j, g) for j, g in enumerate(range(lo, hi))]
            assert [g for _, g in seen] == list(range(n))
            assert all(pos == g for pos, g in seen)


def test_nvfp4_scale_layout_round_trip():
    """The interleaved 128 x 4 scale layout of the NVFP4 GEMM: the PyTorch inverse used by the tests against a direct
    statement of the forward map (checked on the GPU against the kernel, and at build time against the collective)."""
    import torch

    from phyai_b200.ops.nvfp4 import unswizzle_scales

    rows, K = 300, 1056                      # neither a multiple of 128 rows nor of 64 columns
    nkb, kbp = K // 16, (K + 63) // 64 * 4
    total = (rows + 127) // 128 * 128 * kbp
    flat = torch.zeros(total, dtype=torch.uint8)
    src = torch.randint(1, 255, (rows, nkb), dtype=torch.uint8)
    for r in range(rows):
        for kb in range(nkb):
            off = ((r // 128) * (kbp // 4) + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
            assert flat[off] == 0            # the map is injective
            flat[off] = src[r, kb]
    back = unswizzle_scales(flat, rows, K).view(torch.uint8)
    assert torch.equal(back, src)


def test_pi05_cached_path_equals_masked_joint_forward():
    """Pi0.5 (two Euler steps) against one masked joint forward per step written with plain tensor ops on the same
    weights: rows = [prefix | actions], the prefix runs the PaliGemma weights with the static Gemma norm, the action rows
    run the expert weights with the time-conditioned norm (scale, shift, gate from a dense layer on the time embedding)."""
    from phyai_b200.models.pi05.configuration_pi05 import tiny_pi05_config
    from phyai_b200.models.pi05.modeling_pi05 import PI05Model

    cfg = tiny_pi05_config(num_inference_steps=2)
    m = PI05Model(cfg).init_random(5)
    for l in m.paligemma_lm.layers:
        l.input_layernorm.weight.data.normal_(0, 0.2)
        l.post_attention_layernorm.weight.data.normal_(0, 0.2)
    for n_ in [n for l in m.expert_stack.layers for n in (l.input_layernorm, l.post_attention_layernorm)] + [m.expert_stack.norm]:
        n_.dense.weight.data.normal_(0, 0.05)
        n_.dense.bias.data.normal_(0, 0.05)
    g = torch.Generator().manual_seed(2)
    pix = torch.rand(2, 3, 56, 56, generator=g) * 2 - 1
    ids = torch.randint(0, 1024, (16,), generator=g)
    noise = torch.randn(cfg.chunk_size, cfg.max_action_dim, generator=g)
    L = 9
    got = m.sample_actions(pix[None], ids[None], torch.tensor([L]), noise[None])[0]

    def ada(x, norm, cond, eps=cfg.expert.rms_norm_eps):
        scale, shift, gate = (cond @ norm.dense.weight.t() + norm.dense.bias).chunk(3, dim=-1)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1 + scale) + shift, gate

    img = m.vision(pix).reshape(-1, cfg.text.hidden_size)
    lang = m.paligemma_lm.embed_tokens.data[ids[:L]] * math.sqrt(cfg.text.hidden_size)
    prefix0 = torch.cat([img, lang])
    P, C = prefix0.shape[0], cfg.chunk_size
    n = P + C
    mask = torch.zeros(n, n, dtype=torch.bool)
    mask[:P, :P] = True                      # prefix: bidirectional, blind to the actions
    mask[P:, :] = True                       # actions: the prefix and each other
    pos = torch.arange(n)
    H, KV, hd = cfg.text.num_attention_heads, cfg.text.num_key_value_heads, cfg.text.head_dim
    x = noise.clone()
    N = cfg.num_inference_steps
    for i in range(N):
        t = torch.full((1,), 1.0 - i / N)
        emb = ref.sinusoidal_time_embedding(t, cfg.expert.hidden_size, cfg.min_period, cfg.max_period)
        cond = F.silu(F.silu(emb @ m.heads.time_mlp_in.weight.t() + m.heads.time_mlp_in.bias) @ m.heads.time_mlp_out.weight.t()
                      + m.heads.time_mlp_out.bias)
        hp = prefix0
        he = x @ m.heads.action_in_proj.weight.t() + m.heads.action_in_proj.bias
        for lp, le in zip(m.paligemma_lm.layers, m.expert_stack.layers):
            wp, we = _weights(lp), _weights(le)
            xp = _gemma_norm(hp, lp.input_layernorm.weight.data)
            xe, g1 = ada(he, le.input_layernorm, cond)
            q = torch.cat([(xp @ wp["wq"].t()), (xe @ we["wq"].t())]).reshape(n, H, hd)
            k = torch.cat([(xp @ wp["wk"].t()), (xe @ we["wk"].t())]).reshape(n, KV, hd)
            v = torch.cat([(xp @ wp["wv"].t()), (xe @ we["wv"].t())]).reshape(n, KV, hd)
            q, k = _rope(q, pos), _rope(k, pos)
            kk, vv = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
            s = torch.einsum("qhd,khd->hqk", q, kk) / math.sqrt(hd)
            att = torch.einsum("hqk,khd->qhd", torch.softmax(s.masked_fill(~mask[None], float("-inf")), -1), vv).reshape(n, -1)
            hp = hp + att[:P] @ wp["wo"].t()
            he = he + g1 * (att[P:] @ we["wo"].t())
            hp = hp + _mlp(_gemma_norm(hp, lp.post_attention_layernorm.weight.data), wp)
            xe, g2 = ada(he, le.post_attention_layernorm, cond)
            he = he + g2 * _mlp(xe, we)
        out, _ = ada(he, m.expert_stack.norm, cond)
        x = x - (out @ m.heads.action_out_proj.weight.t() + m.heads.action_out_proj.bias) / N
    assert torch.allclose(got, x, atol=2e-4), (got - x).abs().max()
