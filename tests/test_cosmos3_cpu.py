"""Cosmos3 on CPU: sampler, VAE stream equivalence, sound decoder, schedulers and plugins (tiny geometries)."""

import math

import pytest
import torch

from phyai_b200.models.cosmos3 import (Cosmos3ActionRequest, Cosmos3AVAESoundConfig, Cosmos3T2VRequest, Cosmos3WanVAEConfig,
                                       UniPCMultistepSampler, pixel_to_latent_shape, tiny_cosmos3_config)
from phyai_b200.models.cosmos3.avae_sound import Cosmos3AVAESoundDecoder
from phyai_b200.models.cosmos3.vae_wan import (Cosmos3WanVAE, feather_1d, fold_patches, pool_down, spread_up, tile_grid, tile_span,
                                               unfold_patches)


def CPU_ENGINE():
    from phyai_b200 import DeviceConfig, EngineConfig, RuntimeConfig

    return EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False))


def tiny_vae(seed=0):
    cfg = Cosmos3WanVAEConfig(z_dim=4, decoder_base_dim=8, base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1,
                              latents_mean=tuple(0.1 * i for i in range(4)), latents_std=tuple(1.0 + 0.1 * i for i in range(4)))
    vae = Cosmos3WanVAE(cfg, device="cpu", dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(seed)
    for p in vae.parameters():
        p.data.copy_(torch.randn(p.shape, generator=g) * (0.3 if p.dim() > 1 else 0.1) + (1.0 if "gamma" in str(p.shape) else 0.0))
    return vae


# ---------------------------------------------------------------- sampler
@pytest.mark.parametrize("karras", [True, False])
def test_unipc_exact_on_linear_trajectory(karras):
    """For x_t = (1 - s) x0 + s e the flow velocity e - x0 is constant, and the solver must land on x0."""
    torch.manual_seed(0)
    x0, e = torch.randn(2, 3, 5), torch.randn(2, 3, 5)
    s = UniPCMultistepSampler(flow_shift=3.0, use_karras_sigmas=karras)
    s.set_timesteps(8)
    s0 = float(s.sigmas[0])
    x = (1 - s0) * x0 + s0 * e
    for t in s.timesteps:
        x = s.step(e - x0, t, x)
    assert torch.allclose(x, x0, atol=1e-4)


def test_unipc_timesteps_descend_and_reset():
    s = UniPCMultistepSampler(flow_shift=10.0, use_karras_sigmas=False)
    s.set_timesteps(12)
    ts = [float(t) for t in s.timesteps]
    assert len(ts) == 12 and all(a > b for a, b in zip(ts, ts[1:]))
    x = torch.ones(3)
    s.step(torch.zeros(3), s.timesteps[0], x)
    assert s.step_index == 1
    s.set_timesteps(12)
    assert s.step_index in (None, 0)


# ---------------------------------------------------------------- VAE
def test_patch_fold_round_trip_and_shortcuts():
    x = torch.randn(2, 3, 5, 8, 12)
    assert torch.equal(unfold_patches(fold_patches(x, 2), 2), x)
    y = torch.randn(1, 8, 3, 4, 4)
    up = spread_up(y, 4, 2, 2, drop_first=True)
    assert up.shape == (1, 4, 5, 8, 8)
    # every output channel group copies consecutive input channels; mean-pooling a spread tensor recovers a channel average
    down = pool_down(torch.randn(1, 4, 5, 8, 8), 8, 2, 2)
    assert down.shape == (1, 8, 3, 4, 4)


def test_vae_shapes_and_stream_equivalence():
    vae = tiny_vae()
    lat = torch.randn(1, 4, 4, 3, 2)
    whole = vae.decode(lat)
    assert whole.shape == (1, 3, 13, 48, 32)
    for chunk in (1, 2, 3):
        assert torch.allclose(vae.decode(lat, frames_per_chunk=chunk), whole, atol=1e-5), chunk
    pix = torch.rand(1, 3, 9, 32, 32) * 2 - 1
    z = vae.encode(pix)
    assert z.shape == (1, 4, 3, 2, 2)
    assert torch.allclose(vae.encode(pix, frames_per_chunk=4), z, atol=1e-5)
    with pytest.raises(ValueError):
        vae.encode(torch.zeros(1, 3, 8, 32, 32))


def test_vae_is_causal_in_time():
    vae = tiny_vae(1)
    lat = torch.randn(1, 4, 3, 2, 2)
    full = vae.decode(lat)
    assert torch.allclose(vae.decode(lat[:, :, :2]), full[:, :, :5], atol=1e-5)


def test_tile_helpers():
    assert tile_grid(4) == (2, 2) and tile_grid(8) == (2, 4) and tile_grid(2) == (1, 2) and tile_grid(7) == (1, 7)
    spans = [tile_span(45, 4, i, 2) for i in range(4)]
    assert spans[0][0] == 0 and spans[-1][1] == 45
    assert all(a[1] - 4 == b[0] for a, b in zip(spans, spans[1:]))  # neighbours overlap by 2 * halo
    w = feather_1d(10, 3, "cpu", torch.float32)
    assert w[0] == pytest.approx(0.25) and w[4] == 1 and torch.equal(w, w.flip(0))


def test_vae_key_names_match_diffusers_layout():
    names = {n for n, _ in tiny_vae().named_parameters()}
    for k in ("decoder.conv_in.weight", "decoder.mid_block.attentions.0.to_qkv.weight", "decoder.mid_block.resnets.1.norm2.gamma",
              "decoder.up_blocks.0.upsampler.time_conv.bias", "decoder.up_blocks.2.upsampler.resample.1.weight",
              "decoder.up_blocks.1.resnets.0.conv_shortcut.weight" if False else "decoder.up_blocks.3.resnets.1.conv2.weight",
              "encoder.down_blocks.1.downsampler.time_conv.weight", "encoder.down_blocks.0.downsampler.resample.1.bias",
              "quant_conv.weight", "post_quant_conv.bias", "encoder.norm_out.gamma"):
        hf = {h for n, p in tiny_vae().named_parameters() for h in getattr(p, "hf_keys", {})}
        assert k in hf, k
    assert len(names) == len({h for n, p in tiny_vae().named_parameters() for h in p.hf_keys})


# ---------------------------------------------------------------- sound
def test_avae_hop_and_range():
    cfg = Cosmos3AVAESoundConfig(dec_dim=4, latent_ch=6, audio_channels=2, dec_strides=(2, 3), dec_c_mults=(1, 2))
    dec = Cosmos3AVAESoundDecoder(cfg, dtype=torch.float32, device="cpu")
    g = torch.Generator().manual_seed(0)
    for p in dec.parameters():
        p.data.copy_(torch.randn(p.shape, generator=g) * 0.2)
    wav = dec.decode(torch.randn(1, 6, 7))
    assert dec.hop_size == 6 and wav.shape == (1, 2, 42) and wav.abs().max() <= 1


# ---------------------------------------------------------------- schedulers through the engine
def _prompts(B=1, L=5, vocab=256):
    ids = torch.randint(0, vocab, (B, L))
    mask = torch.ones(B, L, dtype=torch.long)
    return ids, mask


def test_pixel_to_latent_shape():
    assert pixel_to_latent_shape(93, 720, 1280) == (24, 45, 80)


def test_t2v_plugin_latents_cfg_and_conditioning():
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import EngineConfig
    from phyai_b200.models.cosmos3.main_cosmos3 import Cosmos3Args

    cfg = tiny_cosmos3_config(sound_gen=True)
    eng = Engine(EngineArgs("cosmos3", Cosmos3Args(config=cfg, load_vae=False, load_sound=False), CPU_ENGINE()))
    ids, mask = _prompts()
    nids, nmask = _prompts()
    cond = torch.randn(1, 4, 3, 4, 6)
    req = Cosmos3T2VRequest(ids, mask, nids, nmask, video_shape=(3, 4, 6), num_inference_steps=3, guidance_scale=2.0,
                            cond_latents=cond, cond_frame_indexes=(0,))
    out = eng.step(req)
    assert out.shape == (1, 4, 3, 4, 6) and torch.isfinite(out).all()
    assert torch.equal(out[:, :, 0], cond[:, :, 0])
    again = eng.step(req)
    assert torch.equal(out, again)  # seeded noise, fresh solver per request
    snd = eng.step(Cosmos3T2VRequest(ids, mask, nids, nmask, video_shape=(2, 4, 6), num_inference_steps=2, guidance_scale=1.0,
                                     sound_frames=5, sound_dim=8))
    assert snd["video"].shape == (1, 4, 2, 4, 6) and snd["sound"].shape == (1, 8, 5)
    eng.close()


@pytest.mark.parametrize("mode", ["policy", "forward_dynamics", "inverse_dynamics"])
def test_policy_plugin_modes(mode):
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.engine_config import EngineConfig
    from phyai_b200.models.cosmos3.main_cosmos3_policy import Cosmos3PolicyArgs

    cfg = tiny_cosmos3_config(action_gen=True)
    eng = Engine(EngineArgs("cosmos3_policy", Cosmos3PolicyArgs(config=cfg), CPU_ENGINE()))
    ids, mask = _prompts()
    cond_v = torch.randn(1, 4, 2, 4, 6)
    cond_a = torch.randn(1, 3, 8)
    req = Cosmos3ActionRequest(ids, mask, ids, mask, video_shape=(2, 4, 6), mode=mode, domain_id=1, action_chunk=3,
                               raw_action_dim=5, action_dim=8, cond_video_latents=cond_v, cond_action=cond_a,
                               num_inference_steps=3)
    act = eng.step(req)
    assert act.shape == (1, 3, 5) and torch.isfinite(act).all()
    full = eng.entry.scheduler.step(req)
    if mode == "forward_dynamics":
        assert torch.equal(full["action"], cond_a[:, :, :5])
        assert torch.equal(full["video"][:, :, 0], cond_v[:, :, 0]) and not torch.equal(full["video"][:, :, 1], cond_v[:, :, 1])
    elif mode == "inverse_dynamics":
        assert torch.equal(full["video"], cond_v)
    else:
        assert torch.equal(full["video"][:, :, 0], cond_v[:, :, 0])
    with pytest.raises(ValueError):
        eng.entry.scheduler.step(Cosmos3ActionRequest(ids, mask, ids, mask, (2, 4, 6), "dream", 0, 3, 5, 8))
    eng.close()


def test_step_graph_first_call_eager_and_capture_failure_falls_back(caplog):
    """StepGraph: off -> every call runs the function; on -> the first call is eager, and a capture that cannot be
    made (no CUDA device here) is reported once and the step runs launch by launch from then on."""
    from phyai_b200.models.cosmos3.scheduler_cosmos3 import StepGraph

    calls = []

    def fn():
        calls.append(1)
        return (torch.ones(2),)

    off = StepGraph(False)
    for _ in range(3):
        assert off.run(fn)[0].sum() == 2
    assert len(calls) == 3 and off.replays == 0
    calls.clear()
    on = StepGraph(True)
    on.run(fn)
    assert on.enabled and len(calls) == 1
    with caplog.at_level("WARNING"):
        out = on.run(fn)
    assert out[0].sum() == 2 and not on.enabled and on.replays == 0 and on.graph is None
    assert any("not captured" in r.message for r in caplog.records)
    on.run(fn)
    assert len(calls) == 3


@pytest.mark.parametrize("kind", ["t2v", "policy"])
def test_loop_slot_serves_later_requests_from_kept_buffers(kind, monkeypatch):
    """The request-geometry slot on CPU (the step function itself runs eagerly here: the tensor-op sampler never goes
    through the graph): a second request with another prompt, noise and masks, written into the slot's tensors and
    conditions in place, gives what a scheduler without slots gives; results handed out earlier are not overwritten;
    a prompt of another length gets a slot of its own and the oldest slot is dropped."""
    from phyai_b200.engine import Engine, EngineArgs
    from phyai_b200.models.cosmos3 import scheduler_cosmos3 as sc
    from phyai_b200.models.cosmos3.main_cosmos3 import Cosmos3Args
    from phyai_b200.models.cosmos3.main_cosmos3_policy import Cosmos3PolicyArgs

    policy = kind == "policy"
    cfg = tiny_cosmos3_config(action_gen=policy)
    args = Cosmos3PolicyArgs(config=cfg) if policy else Cosmos3Args(config=cfg, load_vae=False, load_sound=False)
    eng = Engine(EngineArgs("cosmos3_policy" if policy else "cosmos3", args, CPU_ENGINE()))
    sch = eng.entry.scheduler

    def request(seed: int, text_len: int = 6):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg.vocab_size, (1, 8), generator=g)
        nids = torch.randint(0, cfg.vocab_size, (1, 8), generator=g)
        mask = torch.zeros(1, 8, dtype=torch.long)
        mask[:, :text_len] = 1
        if policy:
            return Cosmos3ActionRequest(ids, mask, nids, mask, video_shape=(2, 4, 6), mode="policy", domain_id=seed % 3, action_chunk=3,
                                        raw_action_dim=5, action_dim=8, cond_video_latents=torch.randn(1, 4, 2, 4, 6, generator=g),
                                        num_inference_steps=3, guidance_scale=2.0, seed=seed)
        return Cosmos3T2VRequest(ids, mask, nids, mask, video_shape=(3, 4, 6), num_inference_steps=3, guidance_scale=2.0,
                                 cond_latents=torch.randn(1, 4, 3, 4, 6, generator=g), cond_frame_indexes=(seed % 3,), seed=seed)

    def tensors(out):
        return [out["video"], out["action"]] if isinstance(out, dict) else [out]

    want = [tensors(sch.step(request(s, n))) for s, n in ((1, 6), (2, 6), (3, 5), (4, 7))]
    assert sch.last_graph_replays == 0 and "_loop_slots" not in sch.__dict__

    monkeypatch.setattr(sch, "_graphable", lambda fused: True)
    got = [tensors(sch.step(request(1, 6)))]
    got.append(tensors(sch.step(request(2, 6))))           # same geometry: served from the slot of the first
    assert len(sch._loop_slots) == 1
    slot = next(iter(sch._loop_slots.values()))
    assert set(slot.conds) == {"cond", "uncond"} and "video" in slot.tensors and "tval" in slot.tensors
    got.append(tensors(sch.step(request(3, 5))))           # another prompt length: a second slot
    assert len(sch._loop_slots) == 2
    got.append(tensors(sch.step(request(4, 7))))           # a third: the least recently used one goes
    assert len(sch._loop_slots) == 2 and slot not in sch._loop_slots.values()
    for a, b in zip(got, want):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    sch.drop_loop_slots()
    assert "_loop_slots" not in sch.__dict__
    eng.close()


def test_transformer_matches_a_restatement_from_checkpoint_tensors(tmp_path):
    """A checkpoint written under the upstream key names (one layer index feeding both towers), loaded through the key
    remap, against the forward pass written out with plain tensor ops on those same checkpoint tensors: text tower
    (causal, K/V kept per layer), generation tower over [text K/V | its own], interleaved three-axis rotary positions with
    the frame-rate rescaling, additive time embedding, patch folding."""
    from safetensors.torch import save_file

    from phyai_b200.models.cosmos3 import Cosmos3Transformer
    from phyai_b200.models.cosmos3.transformer_cosmos3 import cosmos3_weight_remap
    from phyai_b200.weights import load_pretrained

    cfg = tiny_cosmos3_config()
    H, D, Hq, Hkv, I, nl = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size, cfg.num_hidden_layers
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s, std=0.2: torch.randn(*s, generator=g) * std  # noqa: E731
    ck = {"embed_tokens.weight": rnd(cfg.vocab_size, H, std=1.0), "norm.weight": 1 + rnd(H), "lm_head.weight": rnd(4, 4),
          "proj_in.weight": rnd(H, cfg.patch_latent_dim), "proj_in.bias": rnd(H), "proj_out.weight": rnd(cfg.patch_latent_dim, H),
          "proj_out.bias": rnd(cfg.patch_latent_dim), "norm_moe_gen.weight": 1 + rnd(H),
          "time_embedder.linear_1.weight": rnd(H, 256), "time_embedder.linear_1.bias": rnd(H),
          "time_embedder.linear_2.weight": rnd(H, H), "time_embedder.linear_2.bias": rnd(H)}
    und = dict(q="self_attn.to_q", k="self_attn.to_k", v="self_attn.to_v", o="self_attn.to_out", nq="self_attn.norm_q", nk="self_attn.norm_k",
               ln1="input_layernorm", ln2="post_attention_layernorm", gate="mlp.gate_proj", up="mlp.up_proj", down="mlp.down_proj")
    gen = dict(q="self_attn.add_q_proj", k="self_attn.add_k_proj", v="self_attn.add_v_proj", o="self_attn.to_add_out",
               nq="self_attn.norm_added_q", nk="self_attn.norm_added_k", ln1="input_layernorm_moe_gen",
               ln2="post_attention_layernorm_moe_gen", gate="mlp_moe_gen.gate_proj", up="mlp_moe_gen.up_proj", down="mlp_moe_gen.down_proj")
    shapes = dict(q=(Hq * D, H), k=(Hkv * D, H), v=(Hkv * D, H), o=(H, Hq * D), nq=(D,), nk=(D,), ln1=(H,), ln2=(H,),
                  gate=(I, H), up=(I, H), down=(H, I))
    for i in range(nl):
        for names in (und, gen):
            for short, leaf in names.items():
                t = rnd(*shapes[short])
                ck[f"layers.{i}.{leaf}.weight"] = 1 + t if len(shapes[short]) == 1 else t
    save_file({k: v.contiguous() for k, v in ck.items()}, str(tmp_path / "model.safetensors"))
    model = Cosmos3Transformer(cfg, params_dtype=torch.float32, device="cpu").eval()
    report = load_pretrained(model, tmp_path, remap=cosmos3_weight_remap, strict=True)
    assert not report.missing and not report.unexpected

    B, L, vs, fps = 1, 6, (3, 4, 6), 12.0
    ids = torch.randint(0, cfg.vocab_size, (B, L), generator=g)
    lat = torch.randn(B, cfg.latent_channel, *vs, generator=g)
    tval = torch.tensor([437.0])
    got = model(lat, tval, model.encode_condition(ids, torch.ones(B, L, dtype=torch.long), vs, fps))

    # ------------------------------------------------------------------ by hand
    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(x, pos3):
        """x (T, heads, D); pos3 (3, T). Band i of the D/2 frequency bands follows the time axis, except bands
        1, 4, 7, ... (as many as the height section holds) and 2, 5, 8, ... (width section)."""
        half = D // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        ang = pos3[0].float()[:, None] * inv[None]
        for axis in (1, 2):
            idx = torch.arange(axis, cfg.mrope_section[axis] * 3, 3)
            ang[:, idx] = pos3[axis].float()[:, None] * inv[None, idx]
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def block(h, names, i, pos3, extra_kv=None, causal=False):
        w = lambda s: ck[f"layers.{i}.{names[s]}.weight"]  # noqa: E731
        x = rms(h, w("ln1"))
        T = x.shape[0]
        q = rope(rms((x @ w("q").t()).reshape(T, Hq, D), w("nq")), pos3)
        k = rope(rms((x @ w("k").t()).reshape(T, Hkv, D), w("nk")), pos3)
        v = (x @ w("v").t()).reshape(T, Hkv, D)
        kk, vv = (k, v) if extra_kv is None else (torch.cat([extra_kv[0], k]), torch.cat([extra_kv[1], v]))
        rep = Hq // Hkv
        s = torch.einsum("qhd,khd->hqk", q, kk.repeat_interleave(rep, 1)) / math.sqrt(D)
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1)[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv.repeat_interleave(rep, 1)).reshape(T, Hq * D)
        h = h + a @ w("o").t()
        y = rms(h, w("ln2"))
        return h + (torch.nn.functional.silu(y @ w("gate").t()) * (y @ w("up").t())) @ w("down").t(), k, v

    text_pos = torch.arange(L)[None].expand(3, -1)
    h = ck["embed_tokens.weight"][ids[0]]
    text_kv = []
    for i in range(nl):
        h, k, v = block(h, und, i, text_pos, causal=True)
        text_kv.append((k, v))
    t_lat, h_lat, w_lat = vs
    p = cfg.latent_patch_size
    hp, wp = h_lat // p, w_lat // p
    first = L + cfg.temporal_modality_margin
    # frame positions rescaled to the base frame rate: frame f sits at f / (fps / 4) * (24 / 4)
    tt = torch.arange(t_lat, dtype=torch.float32) / (fps / cfg.temporal_compression_factor) * (cfg.base_fps / cfg.temporal_compression_factor) + first
    gen_pos = torch.stack([tt[:, None, None].expand(t_lat, hp, wp).reshape(-1),
                           torch.arange(hp, dtype=torch.float32)[None, :, None].expand(t_lat, hp, wp).reshape(-1),
                           torch.arange(wp, dtype=torch.float32)[None, None, :].expand(t_lat, hp, wp).reshape(-1)])
    tokens = torch.zeros(t_lat * hp * wp, p * p * cfg.latent_channel)
    for f in range(t_lat):
        for y in range(hp):
            for x_ in range(wp):
                patch = lat[0, :, f, y * p:(y + 1) * p, x_ * p:(x_ + 1) * p]            # (c, py, px)
                tokens[(f * hp + y) * wp + x_] = patch.permute(1, 2, 0).reshape(-1)       # ordered (py, px, c)
    freqs = torch.exp(-math.log(10000.0) * torch.arange(128, dtype=torch.float32) / 128)
    a = (tval * cfg.timestep_scale)[:, None] * freqs[None]
    te = torch.nn.functional.silu(torch.cat([a.cos(), a.sin()], -1) @ ck["time_embedder.linear_1.weight"].t() + ck["time_embedder.linear_1.bias"])
    te = te @ ck["time_embedder.linear_2.weight"].t() + ck["time_embedder.linear_2.bias"]
    hg = tokens @ ck["proj_in.weight"].t() + ck["proj_in.bias"] + te
    for i in range(nl):
        hg, _, _ = block(hg, gen, i, gen_pos, extra_kv=text_kv[i])
    out_tok = rms(hg, ck["norm_moe_gen.weight"]) @ ck["proj_out.weight"].t() + ck["proj_out.bias"]
    want = torch.zeros_like(lat)
    for f in range(t_lat):
        for y in range(hp):
            for x_ in range(wp):
                want[0, :, f, y * p:(y + 1) * p, x_ * p:(x_ + 1) * p] = out_tok[(f * hp + y) * wp + x_].reshape(p, p, -1).permute(2, 0, 1)
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max()
