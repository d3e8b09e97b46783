import pytest
import torch

from phyai_b200.layers.attention import Attention, ARAttention, DiffusionAttention, PagedAttnCtx, PagedAttnMetadata, RaggedMeta, eager_attn
from phyai_b200.layers.attention.gdn import GatedDeltaNetAttention, gated_delta_rule_recurrent
from phyai_b200.layers.activation import Snake1d
from phyai_b200.layers.conv import Conv1d, Conv3d, ConvTranspose1d
from phyai_b200.layers.layer_norm import AdaRMSNorm, GemmaRMSNorm, LayerNorm, RMSNorm
from phyai_b200.layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear, QKVParallelLinear,
                                      ReplicatedLinear, RowParallelLinear)
from phyai_b200.layers.mlp import DenseMLP
from phyai_b200.layers.rotary_embedding import MRotaryEmbedding, RotaryEmbedding, apply_rotary_pos_emb
from phyai_b200.layers.transformer_block import SIGLIP_NAMES, TransformerBlock
from phyai_b200.layers.vocab_embedding import ParallelLMHead, VocabParallelEmbedding
from phyai_b200.cache import KVCachePool, StaticCache
from phyai_b200.ops import ref
from phyai_b200.parallel.mesh import Mesh
from phyai_b200.weights import build_index


def fake_mesh(tp, rank):
    return Mesh((tp,), ("tp",), rank=rank, build_groups=False)


def test_norms_match_manual():
    x = torch.randn(5, 16)
    n = RMSNorm(16); n.weight.data.uniform_(0.5, 1.5)
    assert torch.allclose(n(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * n.weight, atol=1e-6)
    g = GemmaRMSNorm(16); g.weight.data.normal_(0, 0.1)
    assert torch.allclose(g(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + g.weight), atol=1e-6)
    r = torch.randn(5, 16); r0 = r.clone()
    y, r2 = g(x, r)
    assert r2 is r and torch.allclose(r, r0 + x) and torch.allclose(y, g(r0 + x), atol=1e-6)
    ln = LayerNorm(16)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (16,), ln.weight, ln.bias, 1e-6), atol=1e-6)


def test_adarmsnorm_identity_at_init_and_modulation_paths():
    a = AdaRMSNorm(16, 8)
    x, cond = torch.randn(2, 3, 16), torch.randn(2, 8)
    y, gate = a(x, cond)
    assert torch.allclose(y, ref.rms_norm(x), atol=1e-6) and gate.abs().max() == 0 and gate.shape == (2, 1, 16)
    a.dense.weight.data.normal_(0, 0.1); a.dense.bias.data.normal_(0, 0.1)
    y1, g1 = a(x, cond)
    table = a.project_modulation(cond)
    y2, g2 = a(x, modulation=table)
    assert torch.allclose(y1, y2, atol=1e-6) and torch.allclose(g1, g2)
    with pytest.raises(ValueError):
        a(x)
    with pytest.raises(ValueError):
        a.project_modulation(torch.randn(2, 7))


def test_column_row_tp_shapes_and_bias_rank0():
    c = ColumnParallelLinear(8, 12, mesh=fake_mesh(2, 1), prefix="m.c")
    assert c.weight.shape == (6, 8) and c.tp_rank == 1
    r0 = RowParallelLinear(12, 8, mesh=fake_mesh(2, 0), reduce_results=False, prefix="m.r")
    r1 = RowParallelLinear(12, 8, mesh=fake_mesh(2, 1), reduce_results=False, prefix="m.r")
    for r in (r0, r1):
        r.weight.data.zero_(); r.bias.data.fill_(3.0)
    x = torch.randn(4, 6)
    assert torch.allclose(r0(x)[0], torch.full((4, 8), 3.0)) and r1(x)[0].abs().max() == 0
    with pytest.raises(ValueError):
        ColumnParallelLinear(8, 13, mesh=fake_mesh(2, 0))


def test_qkv_gqa_replica_share_kv_slot():
    a = QKVParallelLinear(16, 4, 8, 2, bias=False, mesh=fake_mesh(4, 2), prefix="a.qkv_proj")
    b = QKVParallelLinear(16, 4, 8, 2, bias=False, mesh=fake_mesh(4, 3), prefix="a.qkv_proj")
    assert a.num_heads == 2 and a.num_kv_heads == 1 and a.num_kv_head_replicas == 2
    k = torch.arange(8 * 16.).reshape(8, 16)
    for m in (a, b):
        m.weight.weight_loader(m.weight, k, "k")
    assert torch.equal(a.weight.data[8:12], k[4:8]) and torch.equal(b.weight.data[8:12], k[4:8])


def test_skip_bias_add_and_replicated():
    l = ReplicatedLinear(4, 3, skip_bias_add=True)
    l.weight.data.normal_(); l.bias.data.normal_()
    y, b = l(torch.randn(2, 4))
    assert b is l.bias and y.shape == (2, 3)


def test_dense_mlp_gated_matches_manual():
    m = DenseMLP(8, 16, gated=True, activation="gelu_tanh", prefix="x.mlp")
    for p in m.parameters():
        p.data.normal_(0, 0.3)
    x = torch.randn(3, 8)
    w = m.gate_up_proj.weight
    g, u = x @ w[0::2].t(), x @ w[1::2].t()
    want = (torch.nn.functional.gelu(g, approximate="tanh") * u) @ m.down_proj.weight.t()
    assert torch.allclose(m(x), want, atol=1e-5)
    idx, _ = build_index(m)
    assert {"x.mlp.gate_proj.weight", "x.mlp.up_proj.weight", "x.mlp.down_proj.weight"} <= set(idx)
    p = DenseMLP(8, 16, gated=False, activation="gelu_tanh", bias=True)
    assert p(x).shape == (3, 8)


def test_rope_matches_hf_convention_and_mrope():
    rope = RotaryEmbedding(8, 64, 10000.0)
    pos = torch.tensor([0, 3, 7])
    q, k = torch.randn(3, 2, 8), torch.randn(3, 1, 8)
    q1, k1 = rope(pos, q, k)
    cs = rope.cos_sin_cache[pos]
    cos = torch.cat([cs[:, :4], cs[:, :4]], -1)[:, None]
    sin = torch.cat([cs[:, 4:], cs[:, 4:]], -1)[:, None]
    q2, k2 = apply_rotary_pos_emb(q, k, cos, sin)
    assert torch.allclose(q1, q2, atol=1e-6) and torch.allclose(k1, k2, atol=1e-6)
    mr = MRotaryEmbedding(16, (4, 2, 2), 1e4, interleaved=True)
    same = torch.arange(5.)[None].expand(3, 5)
    plain = ref.rope_cos_sin(torch.arange(5.), 16, 1e4)
    assert torch.allclose(mr.cos_sin(same), plain, atol=1e-5)   # equal axes collapse to ordinary RoPE
    with pytest.raises(ValueError):
        MRotaryEmbedding(16, (4, 2, 1))


def test_attention_backends_agree_and_ragged():
    att = Attention(4, 8, 2, causal=True, backend="torch")
    q, k, v = torch.randn(2, 5, 4, 8), torch.randn(2, 5, 2, 8), torch.randn(2, 5, 2, 8)
    a = att(q, k, v)
    e = eager_attn(q, k, v, causal=True)
    assert torch.allclose(a, e, atol=1e-5)
    cu = torch.tensor([0, 5, 10], dtype=torch.int32)
    r = att(q.reshape(10, 4, 8), k.reshape(10, 2, 8), v.reshape(10, 2, 8), RaggedMeta(cu, 5))
    assert torch.allclose(r.reshape(2, 5, 4, 8), e, atol=1e-5)
    sw = Attention(4, 8, 2, causal=True, sliding_window=2, backend="torch")(q, k, v)
    assert not torch.allclose(sw, e)


def test_paged_attention_matches_dense_and_cross_lengths():
    pool = KVCachePool(1, 32, 1, 8, dtype=torch.float32, device="cpu")
    prefix = StaticCache(pool, base_offset=1, capacity=20)
    layer = DiffusionAttention(0, 4, 8, 1, backend="torch")
    kp, vp = torch.randn(6, 1, 8), torch.randn(6, 1, 8)
    slots_p = prefix.allocate(6)
    pool.write_kv(0, kp, vp, slots_p)
    q, k, v = torch.randn(3, 4, 8), torch.randn(3, 1, 8), torch.randn(3, 1, 8)
    slots_s = prefix.allocate(3)
    md = PagedAttnMetadata(torch.tensor([0, 3], dtype=torch.int32), torch.tensor([0, 9], dtype=torch.int32),
                           torch.cat([slots_p, slots_s]).int(), slots_s, max_q_len=3)
    out = layer(q, k, v, PagedAttnCtx(pool, md))
    want = eager_attn(q[None], torch.cat([kp, k])[None], torch.cat([vp, v])[None])[0]
    assert torch.allclose(out, want, atol=1e-5)
    st = layer.init_cuda_graph_state(8, 2, 16, "cpu")
    layer.init_capture_metadata(md)
    assert int(st.paged_kv_indptr[1]) == 9
    with pytest.raises(RuntimeError):
        prefix.allocate(100)
    ar = ARAttention(0, 4, 8, 1, backend="torch")
    assert ar.causal and not layer.causal


def test_gdn_chunked_equals_stepwise_decode():
    B, T, H, Dk, Dv = 2, 6, 2, 4, 3
    q, k, v = torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dv)
    g, beta = -torch.rand(B, T, H), torch.rand(B, T, H)
    o, S = gated_delta_rule_recurrent(q, k, v, g, beta)
    layer = GatedDeltaNetAttention(H, Dk, Dv)
    pool = torch.zeros(4, H, Dk, Dv)
    idx = torch.tensor([1, 3])
    outs = [layer.decode(q[:, t], k[:, t], v[:, t], g[:, t], beta[:, t], state_pool=pool, state_indices=idx) for t in range(T)]
    assert torch.allclose(torch.stack(outs, 1), o, atol=1e-5) and torch.allclose(pool[idx], S, atol=1e-5)


def test_gdn_chunked_prefill_matches_the_token_recurrence():
    from phyai_b200.layers.attention.gdn import gated_delta_rule_chunked

    g0 = torch.Generator().manual_seed(11)
    for B, T, H, Dk, Dv, chunk in [(2, 150, 3, 32, 48, 64), (1, 64, 2, 16, 16, 64), (1, 37, 1, 8, 12, 16)]:
        q, k = torch.randn(B, T, H, Dk, generator=g0), torch.randn(B, T, H, Dk, generator=g0)
        v = torch.randn(B, T, H, Dv, generator=g0)
        g, beta = -torch.rand(B, T, H, generator=g0) * 0.7, torch.rand(B, T, H, generator=g0)
        s0 = torch.randn(B, H, Dk, Dv, generator=g0) * 0.3
        o1, S1 = gated_delta_rule_recurrent(q, k, v, g, beta, s0)
        o2, S2 = gated_delta_rule_chunked(q, k, v, g, beta, s0, chunk=chunk)
        assert torch.allclose(o1, o2, atol=2e-5) and torch.allclose(S1, S2, atol=2e-5)
    # the layer's prefill takes the chunked path and leaves the same states in the pool
    layer = GatedDeltaNetAttention(3, 32, 48)
    pool = torch.zeros(5, 3, 32, 48)
    idx = torch.tensor([4, 0])
    q, k, v = torch.randn(2, 70, 3, 32, generator=g0), torch.randn(2, 70, 3, 32, generator=g0), torch.randn(2, 70, 3, 48, generator=g0)
    g, beta = -torch.rand(2, 70, 3, generator=g0), torch.rand(2, 70, 3, generator=g0)
    o = layer.prefill(q, k, v, g, beta, state_pool=pool, state_indices=idx)
    o_ref, S_ref = gated_delta_rule_recurrent(q, k, v, g, beta)
    assert torch.allclose(o, o_ref, atol=2e-5) and torch.allclose(pool[idx], S_ref, atol=2e-5)


def test_vocab_parallel_embedding_masks_other_ranks():
    e0 = VocabParallelEmbedding(100, 8, mesh=fake_mesh(2, 0), prefix="emb")
    e1 = VocabParallelEmbedding(100, 8, mesh=fake_mesh(2, 1), prefix="emb")
    assert e0.padded == 128 and e0.per_rank == 64
    full = torch.randn(100, 8)
    for e in (e0, e1):
        e.weight.weight_loader(e.weight, full, None)
        e.tp_size = 1   # keep the test single-process: skip the all-reduce, sum by hand
    ids = torch.tensor([[1, 70, 99, 63]])
    got = e0(ids) + e1(ids)
    assert torch.allclose(got, full[ids], atol=1e-6) and e1.weight.data[36:].abs().max() == 0
    head = ParallelLMHead(VocabParallelEmbedding(10, 8, prefix="e"))
    assert head(torch.randn(2, 8)).shape == (2, 10)


def test_conv_wrappers_and_snake():
    c = Conv3d(2, 4, 3, pad_sides=(1, 1, 1, 1, 2, 0), prefix="c")   # causal in time
    c.weight.data.normal_(); x = torch.randn(1, 2, 5, 6, 6)
    assert c(x).shape == (1, 4, 5, 6, 6)
    wn = Conv1d(3, 5, 3, padding=1, weight_norm=True, prefix="w")
    v, g = torch.randn(5, 3, 3), torch.rand(5, 1, 1) + 0.5
    wn.weight.weight_loader(wn.weight, g, "g"); wn.weight.weight_loader(wn.weight, v, "v")
    assert torch.allclose(wn.weight.data, g * v / v.norm(dim=(1, 2), keepdim=True), atol=1e-6)
    t = ConvTranspose1d(4, 2, 4, stride=2, padding=1, prefix="t"); t.weight.data.normal_()
    assert t(torch.randn(1, 4, 8)).shape == (1, 2, 16)
    s = Snake1d(3, prefix="s"); s.alpha.data.fill_(0.3); s.beta.data.fill_(-0.2)
    x1 = torch.randn(2, 3, 7); before = s(x1); s.post_load()
    assert torch.allclose(before, s(x1), atol=1e-6)
    a, b = torch.tensor(0.3).exp(), torch.tensor(-0.2).exp()
    assert torch.allclose(s(x1), x1 + torch.sin(a * x1) ** 2 / (b + 1e-9), atol=1e-5)


def test_transformer_block_siglip_keys_and_forward():
    blk = TransformerBlock(16, 2, 8, 32, attn_bias=True, attn_out_bias=True, mlp_gated=False,
                           mlp_activation="gelu_pytorch_tanh", mlp_bias=True, norm_type="layernorm", names=SIGLIP_NAMES,
                           attn_backend="torch", prefix="enc.layers.0")
    for p in blk.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.1)
    keys = set(build_index(blk)[0])
    assert {"enc.layers.0.layer_norm1.weight", "enc.layers.0.self_attn.q_proj.bias", "enc.layers.0.self_attn.out_proj.weight",
            "enc.layers.0.mlp.fc1.weight", "enc.layers.0.mlp.fc2.bias"} <= keys
    assert blk(torch.randn(2, 5, 16)).shape == (2, 5, 16)
    dec = TransformerBlock(16, 2, 8, 32, num_kv_heads=1, attn_causal=True, qk_norm=True, rope=RotaryEmbedding(8, 32),
                           attn_backend="torch", prefix="m.layers.1")
    for p in dec.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.1)
    h = torch.randn(1, 6, 16)
    full = dec(h, position_ids=torch.arange(6)[None])
    part = dec(h[:, :4], position_ids=torch.arange(4)[None])
    assert torch.allclose(full[:, :4], part, atol=1e-5)          # causal: a prefix does not see later tokens
