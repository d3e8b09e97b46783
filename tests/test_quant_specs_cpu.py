"""Quantisation IR and weight specs on CPU: spec ids, matchers and plan resolution order, the active-plan context,
allocation shapes per granularity, scale fan-out after loading, quantise / dequantise error bounds, NVFP4 packing."""

import pytest
import torch
import torch.nn as nn

from phyai_b200.layers.quant import scheme as S
from phyai_b200.layers.quant.specs import FP8_MAX, AllocationRequest, Bf16Spec, Fp8Spec, Nvfp4Spec, materialize


def test_spec_ids_and_block_shape_rule():
    assert S.FP8_BLOCK_128.spec_id == "fp8_block_128_128" and S.FP8_PER_TENSOR.spec_id == "fp8_per_tensor"
    assert S.FP8_PER_CHANNEL.spec_id == "fp8_per_channel" and S.NVFP4_BLOCK_16.spec_id == "nvfp4_block_16"
    assert S.QuantScheme(S.TensorQuant(S.QDType.BF16)).spec_id == "bf16"
    assert S.QuantScheme(S.TensorQuant(S.QDType.FP8_E4M3, S.Granularity.BLOCK, (64, 32))).spec_id == "fp8_block_64_32"
    with pytest.raises(ValueError, match="needs a block_shape"):
        S.TensorQuant(S.QDType.FP8_E4M3, S.Granularity.BLOCK)


def test_matchers_combine_their_criteria():
    class Lin(nn.Linear):
        pass

    m = S.Matcher
    assert m(name="a.b").matches("a.b") and not m(name="a.b").matches("a.b.c")
    assert m(glob="layers.*.mlp.*").matches("layers.3.mlp.down_proj") and not m(glob="layers.*.mlp").matches("layers.3.attn")
    assert m(regex=r"\.(q|k)_proj$").matches("x.q_proj") and not m(regex=r"\.(q|k)_proj$").matches("x.v_proj")
    assert m(module_cls="Linear").matches("any", Lin)                      # a base class name matches too
    assert m(module_cls=nn.Linear).matches("any", Lin) and not m(module_cls="Conv2d").matches("any", Lin)
    assert not m(module_cls="Linear").matches("any")                       # a class criterion needs the class
    assert m(glob="vision.*", regex="fc1").matches("vision.mlp.fc1") and not m(glob="vision.*", regex="fc1").matches("vision.mlp.fc2")
    assert m().matches("everything")


def test_plan_first_match_wins_then_default_and_context_nesting():
    plan = S.QuantPlan((S.Rule(S.Matcher(glob="vision.*"), None),                       # an ignore rule
                        S.Rule(S.Matcher(regex="down_proj"), S.FP8_PER_CHANNEL),
                        S.Rule(S.Matcher(glob="*"), S.FP8_BLOCK_128)), default=S.NVFP4_BLOCK_16)
    assert plan.resolve("vision.layers.0.down_proj") is None
    assert plan.resolve("lm.layers.0.down_proj") is S.FP8_PER_CHANNEL
    assert plan.resolve("lm.layers.0.up_proj") is S.FP8_BLOCK_128
    assert S.QuantPlan(default=S.FP8_PER_TENSOR).resolve("x") is S.FP8_PER_TENSOR and S.QuantPlan().resolve("x") is None
    assert S.get_active_plan() is None
    with S.use_quant_plan(plan) as p:
        assert p is plan and S.get_active_plan() is plan
        with S.use_quant_plan(None):
            assert S.get_active_plan() is None
        assert S.get_active_plan() is plan
    assert S.get_active_plan() is None
    assert S.load_quant_plan(None) is None


def test_materialize_picks_the_spec_class():
    assert isinstance(materialize(None), Bf16Spec) and isinstance(materialize(S.QuantScheme(S.TensorQuant(S.QDType.FP16))), Bf16Spec)
    assert isinstance(materialize(S.FP8_BLOCK_128), Fp8Spec) and isinstance(materialize(S.NVFP4_BLOCK_16), Nvfp4Spec)
    assert materialize(S.FP8_PER_CHANNEL).spec_id == "fp8_per_channel"


@pytest.mark.parametrize("scheme,scale_shape", [(S.FP8_PER_TENSOR, (1,)), (S.FP8_PER_CHANNEL, (200,)), (S.FP8_BLOCK_128, (2, 3))])
def test_fp8_allocation_shapes(scheme, scale_shape):
    layer = nn.Module()
    Fp8Spec(scheme).allocate(layer, AllocationRequest(200, 300, torch.bfloat16, "cpu"))
    assert layer.weight.shape == (200, 300) and layer.weight.dtype == torch.float8_e4m3fn
    assert tuple(layer.weight_scale.shape) == scale_shape and layer.weight_scale.dtype == torch.float32
    assert layer.input_scale.shape == (1,) and not layer.weight.requires_grad


def test_per_tensor_scales_fan_out_per_fused_leg():
    layer = nn.Module()
    spec = Fp8Spec(S.FP8_PER_TENSOR)
    spec.allocate(layer, AllocationRequest(12, 16, torch.bfloat16, "cpu"))
    layer.weight_scale = nn.Parameter(torch.tensor([1.0, 2.0, 3.0]), requires_grad=False)      # q, k, v legs
    spec.process_after_loading(layer)
    assert layer.weight_scale.tolist() == [1.0] * 4 + [2.0] * 4 + [3.0] * 4
    spec.process_after_loading(layer)                                                            # already per channel
    assert layer.weight_scale.numel() == 12


@pytest.mark.parametrize("scheme", [S.FP8_PER_TENSOR, S.FP8_PER_CHANNEL, S.FP8_BLOCK_128])
def test_fp8_weight_round_trip_error_and_reference_product(scheme):
    g = torch.Generator().manual_seed(0)
    spec = Fp8Spec(scheme)
    w = torch.randn(200, 300, generator=g) * torch.logspace(-2, 1, 200)[:, None]              # rows of very different size
    layer = nn.Module()
    spec.allocate(layer, AllocationRequest(200, 300, torch.float32, "cpu"))
    q, sc = spec.quantize_weight(w)
    assert q.dtype == torch.float8_e4m3fn and q.float().abs().max() <= FP8_MAX
    layer.weight.data.copy_(q)
    layer.weight_scale = nn.Parameter(sc, requires_grad=False)
    spec.process_after_loading(layer)
    back = spec.dequant_weight(layer)
    # e4m3 keeps three mantissa bits: relative error at most 2^-4 of the largest value sharing the scale
    if scheme is S.FP8_PER_TENSOR:
        assert (back - w).abs().max() <= w.abs().max() / 16
    elif scheme is S.FP8_PER_CHANNEL:
        assert ((back - w).abs().amax(1) <= w.abs().amax(1) / 16 + 1e-9).all()
    else:
        assert (back - w).abs().max() <= w.abs().max() / 16 and torch.allclose(back[-1], w[-1], rtol=0.07, atol=w[-1].abs().max().item() / 16)
    x = torch.randn(7, 300, generator=g)
    y = spec.reference_apply(layer, x, torch.ones(200))
    want = x @ w.t() + 1
    assert (y - want).norm() / want.norm() < 0.06
    assert spec.reference_apply(layer, x.reshape(1, 7, 300), None).shape == (1, 7, 200)


def test_fp8_activation_scales_per_token_and_per_group():
    x = torch.tensor([[1.0] * 256, [0.0] * 128 + [448.0 * 2] * 128])
    q, s = Fp8Spec(S.FP8_PER_TENSOR).quantize_activation(x)
    assert s.shape == (2,) and torch.allclose(s, torch.tensor([1 / FP8_MAX, 2.0]))
    assert q.float()[0, 0] == FP8_MAX and q.float()[1, -1] == FP8_MAX
    q, s = Fp8Spec(S.FP8_BLOCK_128).quantize_activation(x)
    assert s.shape == (2, 2) and s[1, 0] == pytest.approx(1e-12 / FP8_MAX) and s[1, 1] == 2.0   # an all-zero group keeps a tiny scale
    assert torch.isfinite(q.float()).all()
    q, s = Fp8Spec(S.FP8_BLOCK_128).quantize_activation(torch.ones(1, 130))                      # ragged tail group
    assert q.shape == (1, 130) and s.shape == (1, 2)


def test_nvfp4_pack_layout_and_exactness_on_the_grid():
    g = torch.Generator().manual_seed(1)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    codes = torch.randint(0, 16, (4, 64), generator=g)
    w = grid[codes & 7] * torch.where((codes & 8) > 0, -1.0, 1.0)
    w[:, ::16] = 6.0                                                                            # every block spans the full range
    codes[:, ::16] = 7
    packed, bs, gs = Nvfp4Spec.quantize(w)
    assert packed.shape == (4, 32) and packed.dtype == torch.uint8 and bs.shape == (4, 4) and bs.dtype == torch.float8_e4m3fn
    back = Nvfp4Spec.dequantize(packed, bs, gs)
    assert torch.allclose(back, w, rtol=0, atol=1e-6)                                          # grid values survive exactly
    # the low nibble is the even column, the high nibble the odd one, bit 3 is the sign (a signed zero may differ)
    nz = w != 0
    lo, hi = packed & 0xF, packed >> 4
    assert torch.equal(lo[nz[:, 0::2]], codes[:, 0::2][nz[:, 0::2]].to(torch.uint8))
    assert torch.equal(hi[nz[:, 1::2]], codes[:, 1::2][nz[:, 1::2]].to(torch.uint8))


def test_nvfp4_layer_allocation_load_and_reference_product():
    spec = Nvfp4Spec()
    layer = nn.Module()
    spec.allocate(layer, AllocationRequest(24, 64, torch.bfloat16, "cpu"))
    assert layer.weight.shape == (24, 32) and layer.weight_scale.shape == (24, 4) and layer.weight_global_scale.shape == (1,)
    g = torch.Generator().manual_seed(2)
    w, x = torch.randn(24, 64, generator=g), torch.randn(5, 64, generator=g)
    spec.load_full_precision(layer, w)
    y = spec.reference_apply(layer, x, None)
    want = x @ w.t()
    assert (y - want).norm() / want.norm() < 0.15                                               # four-bit weights
    with pytest.raises(ValueError, match="divisible by 16"):
        spec.allocate(nn.Module(), AllocationRequest(8, 40, torch.bfloat16, "cpu"))
    with pytest.raises(ValueError, match="scale layout"):
        Nvfp4Spec(layout="swizzled")
