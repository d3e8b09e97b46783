"""Qwen3-VL / Qwen3.5 reference models on CPU: shapes, ragged vision attention, causality, padding, checkpoint round trip."""

import torch

from phyai_b200.models.qwen3_5 import Qwen3_5ForConditionalGeneration, tiny_qwen3_5_config
from phyai_b200.models.qwen3_vl import Qwen3VLForConditionalGeneration, tiny_qwen3_vl_config
from phyai_b200.models.qwen3_vl.modeling_qwen3_vl import get_vision_cu_seqlens, get_vision_position_ids


def _init(m, seed=0):
    g = torch.Generator().manual_seed(seed)
    for n, p in m.named_parameters():
        if p.dim() > 1:
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
        elif "A_log" in n or "dt_bias" in n:
            p.data.copy_(torch.rand(p.shape, generator=g))
    return m.eval()


def _vision_inputs(cfg, grids, seed=1):
    v = cfg.vision_config
    g = torch.Generator().manual_seed(seed)
    thw = torch.tensor(grids)
    n = int((thw[:, 0] * thw[:, 1] * thw[:, 2]).sum())
    return torch.randn(n, v.in_channels * v.temporal_patch_size * v.patch_size ** 2, generator=g), thw


def test_vision_helpers():
    thw = torch.tensor([[1, 4, 4], [2, 2, 4]])
    assert get_vision_cu_seqlens(thw).tolist() == [0, 16, 24, 32]
    pos = get_vision_position_ids(torch.tensor([[1, 4, 4]]), 2)
    assert pos[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]] and pos[4].tolist() == [0, 2]     # merge-block-major order


def test_qwen3_vl_images_do_not_mix_and_deepstack_applies():
    cfg = tiny_qwen3_vl_config()
    m = _init(Qwen3VLForConditionalGeneration(cfg, dtype=torch.float32))
    pa, ga = _vision_inputs(cfg, [[1, 4, 4]], 1)
    pb, gb = _vision_inputs(cfg, [[1, 2, 4]], 2)
    fa, da = m.model.visual(pa, ga)
    fb, _ = m.model.visual(pb, gb)
    both, dboth = m.model.visual(torch.cat([pa, pb]), torch.cat([ga, gb]))
    assert fa.shape == (4, 48) and fb.shape == (2, 48) and len(da) == 2
    assert torch.allclose(both[:4], fa, atol=1e-5) and torch.allclose(both[4:], fb, atol=1e-5)
    ids = torch.tensor([[5, 119, 120, 120, 120, 120, 7, 8, 9]])
    logits = m(ids, pixel_patches=pa, grid_thw=ga)
    assert logits.shape == (1, 9, 128) and torch.isfinite(logits).all()
    pos = m.model.get_rope_index(ids, ga)
    assert pos[0, 0].tolist() == [0, 1, 2, 2, 2, 2, 4, 5, 6] and pos[1, 0, 2:6].tolist() == [2, 2, 3, 3] and pos[2, 0, 2:6].tolist() == [2, 3, 2, 3]
    # causality: changing a later text token leaves earlier positions alone
    ids2 = ids.clone()
    ids2[0, 8] = 33
    assert torch.allclose(m(ids2, pixel_patches=pa, grid_thw=ga)[:, :8], logits[:, :8], atol=1e-5)
    # the DeepStack taps feed the first text layers
    for p in m.model.visual.deepstack_merger_list.parameters():
        p.data.zero_()
    assert not torch.allclose(m(ids, pixel_patches=pa, grid_thw=ga), logits, atol=1e-4)


def test_qwen3_5_hybrid_stack_causal_and_padding_safe():
    cfg = tiny_qwen3_5_config()
    m = _init(Qwen3_5ForConditionalGeneration(cfg, dtype=torch.float32))
    kinds = [layer.kind for layer in m.model.language_model.layers]
    assert kinds == ["linear_attention"] * 3 + ["full_attention"]
    ids = torch.randint(0, 100, (2, 10), generator=torch.Generator().manual_seed(0))
    out = m(ids)
    assert out.shape == (2, 10, 128) and torch.isfinite(out).all()
    ids2 = ids.clone()
    ids2[:, 7:] = 3
    assert torch.allclose(m(ids2)[:, :7], out[:, :7], atol=1e-5)                 # both layer kinds are causal
    mask = torch.ones(2, 10, dtype=torch.long)
    mask[1, 6:] = 0
    padded = m(ids, attention_mask=mask)
    short = m(ids[1:, :6])
    assert torch.allclose(padded[1, :6], short[0], atol=1e-4)
    pa, ga = _vision_inputs(cfg, [[1, 4, 4]])
    seq = torch.tensor([[1, 120, 120, 120, 120, 2]])
    assert m(seq, pixel_patches=pa, grid_thw=ga).shape == (1, 6, 128)


def test_checkpoint_round_trip(tmp_path):
    from phyai_b200.weights import load_pretrained, synthetic_state_dict, write_checkpoint

    cfg = tiny_qwen3_vl_config()
    a = Qwen3VLForConditionalGeneration(cfg, dtype=torch.float32)
    state = synthetic_state_dict(a, seed=4, std=0.1)
    assert "model.visual.blocks.0.attn.qkv.weight" in state and "model.language_model.layers.2.self_attn.q_norm.weight" in state
    k = "model.visual.patch_embed.proj.weight"
    v = cfg.vision_config
    state[k] = state[k].reshape(v.hidden_size, v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)   # checkpoints hold a Conv3d kernel
    write_checkpoint(tmp_path, state)
    load_pretrained(a, tmp_path)
    b = Qwen3VLForConditionalGeneration(cfg, dtype=torch.float32)
    load_pretrained(b, tmp_path)
    ids = torch.tensor([[1, 2, 3, 4]])
    assert torch.equal(a.eval()(ids), b.eval()(ids))
