"""Row permutation behind the rotating QKV epilogue, checked on the CPU against the plain rope formula."""

import torch

from phyai_b200 import ops
from phyai_b200.ops import ref


def test_permuted_rows_put_rotation_pairs_side_by_side():
    Hq, Hkv, D, K, M = 3, 1, 16, 32, 5
    g = torch.Generator().manual_seed(0)
    w = torch.randn((Hq + 2 * Hkv) * D, K, generator=g)
    x = torch.randn(M, K, generator=g)
    wp = ops.permute_rope_rows(w, Hq, Hkv, D)
    assert wp.shape == w.shape
    assert torch.equal(wp[(Hq + Hkv) * D:], w[(Hq + Hkv) * D:])          # v rows keep their order
    y, yp = x @ w.T, x @ wp.T
    half = D // 2
    pos = torch.arange(M) + 2
    cs = ref.rope_cos_sin(pos, D)                                          # (M, D): cos | sin
    cos, sin = cs[:, :half], cs[:, half:]
    for h in range(Hq + Hkv):
        cols = yp[:, h * D:(h + 1) * D]
        a, b = cols[:, 0::2], cols[:, 1::2]                                 # dimension i and its partner i + D/2
        assert torch.allclose(a, y[:, h * D:h * D + half]) and torch.allclose(b, y[:, h * D + half:(h + 1) * D])
        rot = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=1)      # what the epilogue writes to [i] and [i + D/2]
        want = ref.apply_rope(y[:, h * D:(h + 1) * D].reshape(M, 1, D), cs).reshape(M, D)
        assert torch.allclose(rot, want, atol=1e-5)


def test_permutation_applies_to_bias_vectors():
    Hq, Hkv, D = 2, 1, 8
    b = torch.arange((Hq + 2 * Hkv) * D, dtype=torch.float32)
    bp = ops.permute_rope_rows(b, Hq, Hkv, D)
    assert bp[:D].tolist() == [0, 4, 1, 5, 2, 6, 3, 7] and bp[-D:].tolist() == b[-D:].tolist()
