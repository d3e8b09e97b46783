"""The page-size-1 KV pool and the bump allocator over its slots."""

import pytest
import torch

from phyai_b200.cache import KVCachePool, StaticCache


def test_pool_geometry_write_gather_and_sentinel_slot():
    pool = KVCachePool(2, 16, 3, 4, dtype=torch.float32, device="cpu")
    assert pool.k.shape == (2, 16, 3, 4) and pool.total_bytes == 2 * 2 * 16 * 3 * 4 * 4
    k1, v1 = pool.layer(1)
    assert k1.shape == (16, 3, 4) and k1.data_ptr() == pool.k[1].data_ptr()           # a view, not a copy
    g = torch.Generator().manual_seed(0)
    k, v = torch.randn(5, 3, 4, generator=g), torch.randn(5, 3, 4, generator=g)
    slots = torch.tensor([7, 2, 9, 0, 3])                                               # slot 0 takes a padding row
    pool.write_kv(1, k, v, slots)
    gk, gv = pool.gather_kv(1, torch.tensor([2, 7, 9], dtype=torch.int32))              # any integer index type reads
    assert torch.equal(gk, k[[1, 0, 2]]) and torch.equal(gv, v[[1, 0, 2]])
    assert pool.k[0].abs().sum() == 0                                                   # the other layer is untouched
    untouched = [s for s in range(16) if s not in slots.tolist()]
    assert pool.k[1][untouched].abs().sum() == 0
    pool.write_kv(1, k[:1] * 2, v[:1] * 2, torch.tensor([7]))                           # overwrite in place
    assert torch.equal(pool.gather_kv(1, torch.tensor([7]))[0][0], k[0] * 2)
    pool.zero_()
    assert pool.k.abs().sum() == 0 and pool.v.abs().sum() == 0


def test_pool_casts_to_its_dtype_and_checks_arguments():
    pool = KVCachePool(1, 4, 1, 2, dtype=torch.bfloat16, device="cpu")
    pool.write_kv(0, torch.full((1, 1, 2), 1.00390625), torch.ones(1, 1, 2), torch.tensor([1]))
    assert pool.k.dtype == torch.bfloat16 and float(pool.k[0, 1, 0, 0]) == 1.0           # rounded to bf16
    with pytest.raises(TypeError, match="int64"):
        pool.write_kv(0, torch.ones(1, 1, 2), torch.ones(1, 1, 2), torch.tensor([1], dtype=torch.int32))
    with pytest.raises(ValueError, match="page_size=1"):
        KVCachePool(1, 4, 1, 2, device="cpu", page_size=16)
    with pytest.raises(ValueError, match="positive"):
        KVCachePool(1, 0, 1, 2, device="cpu")


def test_static_cache_bump_allocation_and_reset():
    pool = KVCachePool(1, 32, 1, 2, dtype=torch.float32, device="cpu")
    prefix, suffix = StaticCache(pool, base_offset=1, capacity=20), StaticCache(pool, base_offset=21, capacity=11)
    a, b = prefix.allocate(6), prefix.allocate(3)
    assert a.tolist() == list(range(1, 7)) and b.tolist() == [7, 8, 9] and a.dtype == torch.int64
    assert (prefix.used, prefix.free) == (9, 11)
    assert suffix.allocate(11).tolist() == list(range(21, 32)) and suffix.free == 0
    assert prefix.allocate(0).numel() == 0
    with pytest.raises(RuntimeError, match="want 12, free 11 of 20"):
        prefix.allocate(12)
    assert prefix.used == 9                                  # a refused request takes nothing
    with pytest.raises(ValueError, match="non-negative"):
        prefix.allocate(-1)
    prefix.reset()
    assert prefix.allocate(2).tolist() == [1, 2]
    for off, cap in ((-1, 4), (0, 0), (30, 3)):
        with pytest.raises(ValueError, match="does not fit"):
            StaticCache(pool, base_offset=off, capacity=cap)
