"""NVFP4 block-scaled GEMM and its quantiser on a B200 against fp32 PyTorch statements of the same operations."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def nv():
    from phyai_b200.ops import nvfp4

    if not nvfp4.available():
        pytest.skip("phyai_b200/_blockscaled is not built in this checkout (needs a CUTLASS header tree at build time)")
    return nvfp4


@pytest.mark.parametrize("M,K", [(50, 1024), (300, 2048), (129, 96)])
def test_activation_quantiser(nv, M, K):
    from phyai_b200.layers.quant.specs import Nvfp4Spec

    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 4).bfloat16().cuda()
    gs = 0.01
    q, sf = nv.quantize_activation(x, gs, cached=False)
    torch.cuda.synchronize()
    sfl = nv.unswizzle_scales(sf, M, K)
    # scales: amax / 6 / global rounded to e4m3
    want_sf = (x.float().reshape(M, K // 16, 16).abs().amax(-1) / 6.0 / gs).to(torch.float8_e4m3fn)
    assert torch.equal(sfl.view(torch.uint8), want_sf.view(torch.uint8))
    # values: what comes back is within half an e2m1 step (relative to the block scale) of the input
    deq = Nvfp4Spec.dequantize(q, sfl, torch.tensor([gs], device="cuda"))
    step = (sfl.float() * gs).repeat_interleave(16, 1)          # e2m1 spacing is at most 2 near the top of its range
    assert torch.all((deq - x.float()).abs() <= 1.0 * step + 1e-6)
    # padding bytes of the interleaved scale buffer were not touched
    assert int(sf.sum().item()) == int(sfl.view(torch.uint8).sum().item())


@pytest.mark.parametrize("M,K,N,tile", [(50, 1024, 2560, 0), (300, 2048, 1000, 128), (1000, 512, 4096, 256), (129, 96, 72, 64), (700, 768, 1024, 512)])
def test_gemm_matches_dequantised_fp32(nv, M, K, N, tile):
    from phyai_b200.layers.quant.specs import Nvfp4Spec

    g = torch.Generator().manual_seed(N)
    x = (torch.randn(M, K, generator=g) * 0.7).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).cuda()
    w4, wsf, wg = Nvfp4Spec.quantize(w)
    sfw = nv.swizzle_scales(wsf, K)
    x4, sfx = nv.quantize_activation(x, 1.0, cached=False)
    out = nv.gemm_nvfp4(x4, sfx, w4, sfw, float(wg), tile=tile)
    torch.cuda.synchronize()
    want = nv.ref_gemm_nvfp4(x4, nv.unswizzle_scales(sfx, M, K), w4, wsf, float(wg))
    assert torch.allclose(out.float(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2), float((out.float() - want).abs().max())


def test_nvfp4_layer_runs_on_the_block_scaled_gemm(nv):
    """A linear built with the NVFP4 spec on the b200 kernel path: same result as its dequantising restatement up to the
    activation's own quantisation."""
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers import linear as L
    from phyai_b200.layers.linear import ReplicatedLinear
    from phyai_b200.layers.quant.scheme import NVFP4_BLOCK_16, QuantPlan, use_quant_plan

    init_engine_config(EngineConfig(device=DeviceConfig("cuda", torch.bfloat16)))
    L.init()
    with use_quant_plan(QuantPlan(default=NVFP4_BLOCK_16)):
        lin = ReplicatedLinear(1024, 512, bias=False, params_dtype=torch.bfloat16, prefix="t")
    assert lin.spec.spec_id == "nvfp4_block_16"
    g = torch.Generator().manual_seed(0)
    lin.spec.load_full_precision(lin, torch.randn(512, 1024, generator=g) * 0.05)
    x = (torch.randn(40, 1024, generator=g) * 0.5).bfloat16().cuda()
    y, _ = lin(x)
    want = lin.spec.reference_apply(lin, x, None).float()
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), want.flatten(), dim=0)
    assert cos > 0.99, float(cos)
    assert hasattr(lin, "_nvfp4_prepared")
