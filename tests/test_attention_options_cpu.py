"""Attention layer options on CPU against a per-query statement written out by hand: grouped heads, causal offset when
the query is shorter than the keys, sliding window, logit soft cap, explicit mask, ragged batches with options."""

import math

import pytest
import torch

from phyai_b200.layers.attention import Attention
from phyai_b200.layers.attention.common import RaggedMeta


def by_hand(q, k, v, *, scale, causal=False, window=None, cap=None, mask=None):
    """q (Sq, Hq, D), k / v (Sk, Hkv, D) -> (Sq, Hq, D), one query row and head at a time."""
    Sq, Hq, D = q.shape
    Sk, Hkv, _ = k.shape
    out = torch.zeros(Sq, Hq, D)
    for i in range(Sq):
        pos = i + (Sk - Sq)                       # the last query sits on the last key
        for h in range(Hq):
            g = h // (Hq // Hkv)
            s = (k[:, g] @ q[i, h]) * scale
            if cap is not None:
                s = cap * torch.tanh(s / cap)
            keep = torch.ones(Sk, dtype=torch.bool)
            j = torch.arange(Sk)
            if causal:
                keep &= j <= pos
            if window is not None:
                keep &= (pos - j) < window
            if mask is not None:
                keep &= mask[i]
            s = s.masked_fill(~keep, float("-inf"))
            out[i, h] = torch.softmax(s, dim=0) @ v[:, g]
    return out


@pytest.mark.parametrize("causal,window,cap", [(False, None, None), (True, None, None), (True, 3, None), (False, None, 5.0),
                                                (True, 2, 3.0), (False, 4, None)])
@pytest.mark.parametrize("sq,sk", [(6, 6), (2, 7)])
def test_padded_batches_match_the_per_query_statement(causal, window, cap, sq, sk):
    g = torch.Generator().manual_seed(sq * 10 + sk)
    q, k, v = torch.randn(2, sq, 4, 8, generator=g), torch.randn(2, sk, 2, 8, generator=g), torch.randn(2, sk, 2, 8, generator=g)
    att = Attention(4, 8, 2, causal=causal, sliding_window=window, logits_soft_cap=cap, backend="torch")
    got = att(q, k, v)
    for b in range(2):
        want = by_hand(q[b], k[b], v[b], scale=8 ** -0.5, causal=causal, window=window, cap=cap)
        assert torch.allclose(got[b], want, atol=1e-5), (got[b] - want).abs().max()


def test_explicit_mask_and_custom_scale():
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(1, 4, 2, 8, generator=g), torch.randn(1, 5, 2, 8, generator=g), torch.randn(1, 5, 2, 8, generator=g)
    mask = torch.rand(4, 5, generator=g) > 0.3
    mask[:, 0] = True                              # every query keeps at least one key
    att = Attention(2, 8, scale=0.25, backend="torch")
    got = att(q, k, v, mask=mask)
    want = by_hand(q[0], k[0], v[0], scale=0.25, mask=mask)
    assert torch.allclose(got[0], want, atol=1e-5)


def test_ragged_batches_with_and_without_options():
    g = torch.Generator().manual_seed(5)
    lens = [3, 5, 1]
    T = sum(lens)
    q, k, v = torch.randn(T, 4, 8, generator=g), torch.randn(T, 1, 8, generator=g), torch.randn(T, 1, 8, generator=g)
    cu = torch.tensor([0, 3, 8, 9], dtype=torch.int32)
    for kw in (dict(causal=True), dict(causal=True, sliding_window=2), dict(causal=False, logits_soft_cap=2.0)):
        att = Attention(4, 8, 1, backend="torch", **kw)
        got = att(q, k, v, RaggedMeta(cu, max(lens)))
        s = 0
        for n in lens:
            want = by_hand(q[s:s + n], k[s:s + n], v[s:s + n], scale=8 ** -0.5, causal=kw.get("causal", False),
                           window=kw.get("sliding_window"), cap=kw.get("logits_soft_cap"))
            assert torch.allclose(got[s:s + n], want, atol=1e-5), kw
            s += n
    with pytest.raises(ValueError, match="RaggedMeta"):
        Attention(4, 8, 1, backend="torch")(q, k, v)
    with pytest.raises(NotImplementedError):
        Attention(4, 8, 1, backend="torch")(q, k, v, RaggedMeta(cu, 5), mask=torch.ones(T, T, dtype=torch.bool))


def test_head_grouping_must_divide():
    with pytest.raises(ValueError, match="multiple of num_kv_heads"):
        Attention(6, 8, 4, backend="torch")
    assert math.isclose(Attention(4, 16, backend="torch").scale, 0.25)
