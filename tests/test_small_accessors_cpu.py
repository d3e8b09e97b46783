"""Small accessors and argument spellings that code written against the reference uses: pool and slab views, graph
registry book-keeping, rotary tables as (cos, sin), norm without a shift, vocabulary padding."""

import pytest
import torch

from phyai_b200.cache import KVCachePool, StaticCache
from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
from phyai_b200.layers.rotary_embedding import MRotaryEmbedding, RotaryEmbedding, apply_rotary_pos_emb
from phyai_b200.runtime import CudaGraph, CudaGraphError, CudaGraphRegistry


def test_pool_and_slab_views():
    pool = KVCachePool(2, 8, 1, 4, dtype=torch.float32, device="cpu")
    k, v = pool.kv_buffer(1)
    assert k.data_ptr() == pool.k_buffer(1).data_ptr() == pool.k[1].data_ptr() and v.data_ptr() == pool.v_buffer(1).data_ptr()
    pool.k_buffer(0)[3] = 7.0                                  # a view: the write lands in the pool
    assert pool.k[0, 3].eq(7).all()
    slab = StaticCache(pool, base_offset=2, capacity=5)
    slab.allocate(3)
    assert slab.slot_range() == (2, 7) and slab.used_slot_range() == (2, 5)


def test_graph_registry_bookkeeping_without_a_gpu():
    reg = CudaGraphRegistry()
    g = CudaGraph("a", num_warmup_iters=0, mempool="pool-handle")
    assert g.warmup_iters == 0 and g.mempool == "pool-handle" and CudaGraph("b", 2).warmup_iters == 2
    assert reg.register("a", g) is g and reg.has("a") and reg.get("a") is g and reg.get("zz") is None and "a" in reg
    assert reg.register("a", g) is g                           # the same object again is fine
    with pytest.raises(CudaGraphError, match="already registered"):
        reg.register("a", CudaGraph("other"))
    g.static_inputs = {"x": torch.zeros(2)}
    assert g.input_buffer("x") is g.static_inputs["x"] and set(g.input_buffers) == {"x"}
    with pytest.raises(KeyError, match="has no input 'y'"):
        g.input_buffer("y")
    with pytest.raises(CudaGraphError, match="replayed before capture"):
        g.replay()
    assert reg.deregister("a") is g and not reg.has("a") and reg.deregister("a") is None and g.static_inputs == {}


def test_rotary_tables_as_cos_and_sin():
    r = RotaryEmbedding(8, max_position_embeddings=64, rope_theta=100.0, device="cpu")
    same = RotaryEmbedding(8, 64, 100.0, device="cpu")
    assert torch.equal(r.cos_sin_cache, same.cos_sin_cache)
    pos = torch.tensor([[0, 3, 9], [1, 1, 63]])
    cos, sin = r.get_cos_sin(pos)
    inv = 1.0 / (100.0 ** (torch.arange(0, 8, 2).float() / 8))
    ang = pos[..., None].float() * inv
    assert cos.shape == (2, 3, 8) and torch.allclose(cos, torch.cat([ang.cos(), ang.cos()], -1), atol=1e-6)
    assert torch.allclose(sin, torch.cat([ang.sin(), ang.sin()], -1), atol=1e-6)
    q, k = torch.randn(2, 3, 2, 8), torch.randn(2, 3, 1, 8)
    a, b = apply_rotary_pos_emb(q, k, cos[:, :, None], sin[:, :, None])           # the (cos, sin) pair feeds the HF-style helper
    fa, fb = r(pos.reshape(-1), q.reshape(6, 2, 8), k.reshape(6, 1, 8))
    assert torch.allclose(a.reshape(6, 2, 8), fa, atol=1e-6) and torch.allclose(b.reshape(6, 1, 8), fb, atol=1e-6)
    part = RotaryEmbedding(16, 32, partial_rotary_factor=0.5, device="cpu")
    assert part.rotary_dim == 8 and part.cos_sin_cache.shape == (32, 8)
    lin = RotaryEmbedding(8, 16, rope_type="linear", rope_scaling={"factor": 2.0}, device="cpu")
    assert torch.allclose(lin.cos_sin_cache[4], RotaryEmbedding(8, 16, device="cpu").cos_sin_cache[2], atol=1e-6)    # positions stretched by the factor
    with pytest.raises(NotImplementedError):
        RotaryEmbedding(8, interleave=True, device="cpu")
    with pytest.raises(ValueError, match="partial_rotary_factor"):
        RotaryEmbedding(8, partial_rotary_factor=1.5, device="cpu")
    m = MRotaryEmbedding(16, (4, 2, 2), 1e4)
    flat = torch.arange(5)[None]
    cos3, sin3 = m.get_cos_sin(flat)                                                # (B, S): the same index on the three axes
    plain = RotaryEmbedding(16, 8, 1e4, device="cpu").get_cos_sin(flat)
    assert cos3.shape == (1, 5, 16) and torch.allclose(cos3, plain[0], atol=1e-6) and torch.allclose(sin3, plain[1], atol=1e-6)
    with pytest.raises(ValueError, match="position ids are"):
        m.get_cos_sin(torch.zeros(2, 1, 5))


def test_layer_norm_without_shift_and_vocabulary_padding():
    from phyai_b200.layers.layer_norm import LayerNorm
    from phyai_b200.layers.vocab_embedding import VocabParallelEmbedding, pad_vocab, pad_vocab_to
    from phyai_b200.weights import build_index

    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    ln = LayerNorm(8, bias=False, prefix="ln")
    index, optional = build_index(ln)
    assert "ln.weight" in index and "ln.bias" not in index and not ln.has_bias
    x = torch.randn(3, 8)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (8,), eps=1e-6), atol=1e-6)
    assert LayerNorm(8, prefix="ln").bias.hf_keys == {"ln.bias": None}
    assert pad_vocab_to(100, 2, 128) == pad_vocab(100, 2, 128) == 256 and pad_vocab(100, 2) == 128
    with pytest.raises(ValueError, match="must be positive"):
        pad_vocab(100, 0)
    emb = VocabParallelEmbedding(100, 4, params_dtype=torch.float32, device="cpu", padding_multiple=16)
    assert emb.padded == 112 and emb.weight.shape == (112, 4)
