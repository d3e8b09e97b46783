"""Block-scaled fp8 GEMM on the CUTLASS pair / single tiles of ``phyai_b200._blockscaled`` against the fp32 restatement."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def fb():
    from phyai_b200.ops import fp8_block, nvfp4

    if not nvfp4.available():
        pytest.skip("phyai_b200/_blockscaled is not built in this checkout (needs a CUTLASS header tree at build time)")
    return fp8_block


def _operands(M, K, N, seed):
    from phyai_b200.ops import fp8_block

    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 0.5).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).cuda()
    xb = x.reshape(M, K // 128, 128)
    xs = xb.abs().amax(-1).clamp_min(1e-12) / 448.0
    x8 = (xb / xs[..., None]).clamp(-448, 448).reshape(M, K).to(torch.float8_e4m3fn)
    w8, ws = fp8_block.quantize_weight_block(w)
    return x8, xs.contiguous(), w8, ws.contiguous()


@pytest.mark.parametrize("M,K,N,tile", [(300, 512, 1000, 1), (520, 1024, 1536, 2), (777, 256, 2048, 3), (1024, 2048, 4096, 0)])
def test_tiles_match_fp32(fb, M, K, N, tile):
    x8, xs, w8, ws = _operands(M, K, N, M)
    want = fb.ref_gemm_fp8_block(x8, xs, w8, ws)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    fb.gemm_fp8_blockwise_tiles(x8, xs, w8, ws, out, tile=tile)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2), float((out.float() - want).abs().max())
    # residual added in place
    res = torch.randn(M, N, device="cuda").bfloat16()
    h = res.clone()
    fb.gemm_fp8_blockwise_tiles(x8, xs, w8, ws, h, residual=h, tile=tile)
    torch.cuda.synchronize()
    want_h = want + res.float()
    assert torch.allclose(h.float(), want_h, atol=2e-2 * float(want_h.abs().max()), rtol=2e-2)


def test_many_row_calls_are_routed_to_the_tiles_and_agree_with_the_in_tree_kernel(fb, monkeypatch):
    from phyai_b200 import ops

    M, K, N = 640, 1024, 2048
    x8, xs, w8, ws = _operands(M, K, N, 3)
    monkeypatch.setattr(fb, "TILE_MODULE_MIN_ROWS", 0)
    own = fb.gemm_fp8_block(x8, xs, w8, ws, act="gelu_tanh", glu=True)
    c0 = ops.launch_counter()
    monkeypatch.setattr(fb, "TILE_MODULE_MIN_ROWS", 256)
    routed = fb.gemm_fp8_block(x8, xs, w8, ws, act="gelu_tanh", glu=True)
    torch.cuda.synchronize()
    assert ops.launch_counter() == c0 + 1          # only the gated-activation pass is this library's launch on the routed path
    assert routed.shape == own.shape == (M, N // 2)
    assert torch.allclose(routed.float(), own.float(), atol=2e-2 * float(own.float().abs().max()), rtol=3e-2)
