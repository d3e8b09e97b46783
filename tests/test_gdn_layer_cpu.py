"""The gated-delta-net layer in the reference's calling convention (gates built from a, b, a_log, dt_bias; value heads in
groups per query head; padded or token-major inputs; states as (sequences, value heads, Dv, Dk)) against the rule written
out token by token."""

import pytest
import torch
import torch.nn.functional as F

from phyai_b200.layers.attention import GatedDeltaNet, GatedDeltaNetCtx, list_gdn_backends


def token_by_token(q, k, v, a, b, a_log, dt_bias, cu, state, scale):
    """q, k (T, Hq, D); v (T, Hv, D); a, b (T, Hv); state (N, Hv, Dv, Dk) -> (out (T, Hv, D), final state)."""
    rep = v.shape[-2] // q.shape[-2]
    q, k = q.float().repeat_interleave(rep, -2), k.float().repeat_interleave(rep, -2)
    q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + 1e-6)
    k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + 1e-6)
    g = -a_log.exp()[None] * F.softplus(a.float() + dt_bias.float())
    beta = b.float().sigmoid()
    out, final = torch.empty_like(v, dtype=torch.float32), state.float().clone()
    for n, (s0, s1) in enumerate(zip(cu[:-1], cu[1:])):
        S = final[n]
        for t in range(s0, s1):
            S.mul_(g[t].exp()[:, None, None])
            seen = torch.einsum("hvk,hk->hv", S, k[t])
            S.add_(((v[t].float() - seen) * beta[t, :, None])[:, :, None] * k[t, :, None, :])
            out[t] = torch.einsum("hvk,hk->hv", S, q[t]) * scale
    return out, final


def make(T, Hq, Hv, D, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return dict(q=r(T, Hq, D), k=r(T, Hq, D), v=r(T, Hv, D), a=r(T, Hv), b=r(T, Hv), a_log=r(Hv) * 0.5, dt_bias=r(Hv) * 0.5)


@pytest.mark.parametrize("backend", ["chunked", "recurrent", "flashinfer"])
@pytest.mark.parametrize("Hq,Hv", [(2, 2), (2, 6)])
def test_token_major_batches_with_initial_states(backend, Hq, Hv):
    D, lens = 8, [5, 1, 70]
    cu = [0, 5, 6, 76]
    x = make(sum(lens), Hq, Hv, D, seed=Hv)
    state0 = torch.randn(3, Hv, D, D, generator=torch.Generator().manual_seed(9)) * 0.3
    layer = GatedDeltaNet(Hq, D, num_value_heads=Hv, backend=backend, backend_kwargs={"chunk": 16})
    out, final = layer(**x, cu_seqlens=torch.tensor(cu, dtype=torch.int32), initial_state=state0, return_state=True)
    want, want_state = token_by_token(**x, cu=cu, state=state0, scale=D ** -0.5)
    assert out.shape == (76, Hv, D) and final.shape == (3, Hv, D, D)
    assert torch.allclose(out.float(), want, atol=2e-4, rtol=1e-4), (out.float() - want).abs().max()
    assert torch.allclose(final, want_state, atol=2e-4, rtol=1e-4)


def test_padded_batches_state_pool_and_decode_steps():
    Hq, Hv, D, B, T = 2, 4, 8, 2, 9
    layer = GatedDeltaNet(Hq, D, num_key_heads=Hq, num_value_heads=Hv, scale=0.5)
    flat = make(B * T, Hq, Hv, D, seed=1)
    padded = {k: (v.reshape(B, T, *v.shape[1:]) if v.dim() > 1 else v) for k, v in flat.items()}
    pool = torch.zeros(5, Hv, D, D)
    slots = torch.tensor([3, 1])
    ctx = GatedDeltaNetCtx(state_pool=pool, state_indices=slots)
    out = layer(**padded, ctx=ctx)
    want, want_state = token_by_token(**flat, cu=[0, T, 2 * T], state=torch.zeros(B, Hv, D, D), scale=0.5)
    assert torch.allclose(out.reshape(B * T, Hv, D).float(), want, atol=2e-4)
    assert torch.allclose(pool[slots], want_state, atol=2e-4) and pool[[0, 2, 4]].abs().sum() == 0      # only the two slots were written
    # one more token per sequence continues from the pool
    step = make(B, Hq, Hv, D, seed=2)
    one = {k: (v.reshape(B, 1, *v.shape[1:]) if v.dim() > 1 else v) for k, v in step.items()}
    out1 = layer(**one, ctx=ctx)
    want1, want_state1 = token_by_token(**step, cu=[0, 1, 2], state=want_state, scale=0.5)
    assert torch.allclose(out1.reshape(B, Hv, D).float(), want1, atol=2e-4) and torch.allclose(pool[slots], want_state1, atol=2e-4)


def test_construction_rules_and_names():
    assert list_gdn_backends() == ["chunked", "recurrent"]
    layer = GatedDeltaNet(2, 128, num_key_heads=2, num_value_heads=4)
    assert layer.num_state_heads == 4 and layer.scale == 128 ** -0.5 and "backend='chunked'" in repr(layer)
    assert GatedDeltaNet(2, 8, backend="fla").backend == "chunked"                 # the reference's backend names are accepted
    with pytest.raises(ValueError, match="as many key heads as query heads"):
        GatedDeltaNet(4, 8, num_key_heads=2)
    with pytest.raises(ValueError, match="multiple of num_query_heads"):
        GatedDeltaNet(4, 8, num_value_heads=6)
    with pytest.raises(ValueError, match="must be positive"):
        GatedDeltaNet(0, 8)
    with pytest.raises(KeyError, match="unknown gated-delta-net backend"):
        GatedDeltaNet(2, 8, backend="triton")
    with pytest.raises(ValueError, match="need cu_seqlens"):
        GatedDeltaNet(2, 8)(**make(4, 2, 2, 8, 0))
    with pytest.raises(ValueError, match="do not fit"):
        GatedDeltaNet(2, 8)(**make(4, 3, 3, 8, 0), cu_seqlens=torch.tensor([0, 4]))
