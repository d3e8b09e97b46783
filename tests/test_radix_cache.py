"""C++ prefix cache: tree behaviour, tiers, eviction policies, two-phase moves, hybrid slots, storage, facades."""

import struct
import threading

import pytest

from phyai_b200.cache.radix_cache import (CacheConfig, CacheEventKind, HybridCache, HybridCacheConfig, ImageSegment, Modality,
                                          MultimodalCache, MultiPatternCache, NestedCache, PairedCache, PairedCacheConfig,
                                          PrefixCache, Tier, encode_eagle_bigram_atoms, encode_prompt_to_atoms,
                                          encode_text_atoms_int32, file_storage_backend, hash64, in_memory_storage_backend,
                                          page_align)
from phyai_b200.cache import radix_cache as rc


def toks(*ids):
    return encode_text_atoms_int32(ids)


def put(cache, ids, tier=Tier.DEVICE):
    atoms, _ = page_align(toks(*ids), cache.page_bytes)
    units = cache.allocate(tier, len(atoms) // cache.page_bytes)
    return cache.insert(tier, atoms, units)


def test_insert_match_split_and_overlap():
    c = PrefixCache(atom_bytes=4, atoms_per_unit=2, device_total_units=64)
    assert c.page_bytes == 8 and c.total(Tier.DEVICE) == 64 and c.available(Tier.DEVICE) == 63
    node, inserted, freed = put(c, range(8))
    assert (inserted, freed) == (8, 0) and c.active(Tier.DEVICE) == 4
    m = c.match(toks(*range(8)))
    assert m.matched_atoms[0] == 8 and m.last_node[0] == node
    m2 = c.match(toks(0, 1, 2, 3, 99, 98))                       # diverges inside the edge: split at the page boundary
    assert m2.matched_atoms[0] == 4 and c.node_count == 3
    assert c.collect_units(m2.last_node[0], Tier.DEVICE).tolist() == [1, 2]
    n2, inserted, freed = put(c, [0, 1, 2, 3, 99, 98, 97, 96])
    assert (inserted, freed) == (4, 2) and c.active(Tier.DEVICE) == 6   # the shared pages' fresh units went back
    assert c.collect_units(n2, Tier.DEVICE).tolist()[:2] == [1, 2]
    assert c.match(toks(0, 1, 2)).matched_atoms[0] == 2           # partial trailing page is ignored
    assert c.match(toks(7, 7)).matched_atoms[0] == 0
    with pytest.raises(rc.CacheUsageError):
        c.insert(Tier.DEVICE, toks(1, 2, 3), c.allocate(Tier.DEVICE, 1))     # not page aligned
    with pytest.raises(rc.CacheUsageError):
        c.collect_units(12345, Tier.DEVICE)                                    # foreign handle
    assert c.node_path_hash(node) != c.node_path_hash(n2)
    kinds = [e.kind for e in c.take_events()]
    assert kinds.count(int(CacheEventKind.INSERT)) == 2 and c.take_events() == []


def test_owned_units_raii_and_capacity_error():
    c = PrefixCache(4, 1, device_total_units=8)
    u = c.allocate(Tier.DEVICE, 5)
    assert len(u) == 5 and c.available(Tier.DEVICE) == 2
    head = u.take_first(2)
    tail = u.take_last(1)
    assert (len(head), len(u), len(tail)) == (2, 2, 1)
    head.append(tail)
    assert len(head) == 3 and len(tail) == 0
    with pytest.raises(rc.CacheCapacityError):
        c.allocate(Tier.DEVICE, 3)
    del u, head, tail
    assert c.available(Tier.DEVICE) == 7


@pytest.mark.parametrize("policy", ["lru", "lfu", "slru", "priority"])
def test_eviction_policies_and_pins(policy):
    c = PrefixCache(4, 1, device_total_units=7, eviction_policy=policy, slru_threshold=2)
    a, _, _ = put(c, [1, 2])
    b, _, _ = put(c, [3, 4])
    d, _, _ = put(c, [5, 6])
    assert c.available(Tier.DEVICE) == 0
    c.match(toks(1, 2)); c.match(toks(1, 2))          # a: hot
    c.match(toks(5, 6))                                # d: touched last
    c.set_priority(b, 10); c.set_priority(a, 5); c.set_priority(d, 1)
    seen = []
    oid = c.add_evict_observer(lambda node, tier: seen.append((node, tier)))
    c.ensure_capacity(Tier.DEVICE, 2)
    victim = seen[0][0]
    expect = {"lru": b, "lfu": b, "slru": b, "priority": d}[policy]
    assert victim == expect and c.available(Tier.DEVICE) == 2
    assert c.remove_evict_observer(oid) and not c.remove_evict_observer(oid)
    ref = c.lock(Tier.DEVICE, a)
    other = d if expect == b else b
    c.ensure_capacity(Tier.DEVICE, 4)                  # evicts the other unpinned prefix, not the pinned one
    assert c.match(toks(1, 2)).matched_atoms[0] == 2 and c.match(toks(*([5, 6] if other == d else [3, 4]))).matched_atoms[0] == 0
    with pytest.raises(rc.CacheCapacityError):
        c.ensure_capacity(Tier.DEVICE, 6)              # only the pinned prefix is left
    ref.release()
    c.ensure_capacity(Tier.DEVICE, 6)
    assert c.node_count == 1 and c.available(Tier.DEVICE) == 6


def test_children_keep_parents_resident_and_named_predicates():
    c = PrefixCache(4, 1, device_total_units=16)
    put(c, [1, 2]); put(c, [1, 2, 3, 4]); put(c, [1, 2, 7, 8])
    c.advance_step(10)
    c.match(toks(1, 2, 3, 4))                          # path 1,2 -> 3,4 touched at step 10
    assert c.evict_by_named_predicate(Tier.DEVICE, "step_lt", 10) == 2      # only the cold leaf (7, 8)
    assert c.match(toks(1, 2, 7, 8)).matched_atoms[0] == 2
    assert c.evict_by_predicate(Tier.DEVICE, lambda node, depth, hits, step, prio: depth >= 2) == 4   # leaf first, then its parent
    assert c.node_count == 1
    with pytest.raises(rc.CacheUsageError):
        c.evict_by_named_predicate(Tier.DEVICE, "nope", 0)


def test_demote_promote_two_phase():
    c = PrefixCache(4, 1, device_total_units=5, host_total_units=9, host_max_pending_units=4)
    a, _, _ = put(c, [1, 2])
    b, _, _ = put(c, [3, 4])
    assert c.tier_enabled(Tier.HOST) and not c.tier_enabled(Tier.DISK)
    op = c.start_demote(a, Tier.DEVICE, Tier.HOST)
    assert c.inflight_ops() == [op] and c.pending_units(Tier.HOST) == 2
    ev = [e for e in c.take_events() if e.kind == CacheEventKind.DEMOTE_START][0]
    assert ev.units_from == [1, 2] and len(ev.units_to) == 2 and ev.op == op       # the caller copies these
    assert c.match(toks(1, 2)).matched_atoms[Tier.HOST] == 0                           # pending is not a hit
    done = []
    t = threading.Thread(target=lambda: done.append(c.wait_op(op, 2000)))
    t.start()
    c.complete_op(op, True)
    t.join()
    assert done == [True] and c.available(Tier.DEVICE) == 2 and c.pending_units(Tier.HOST) == 0
    m = c.match(toks(1, 2))
    assert m.matched_atoms[Tier.DEVICE] == 0 and m.matched_atoms[Tier.HOST] == 2
    up = c.start_promote(a, Tier.HOST, Tier.DEVICE)
    c.complete_op(up, False)                                                           # the copy failed: device side rolled back
    assert c.match(toks(1, 2)).matched_atoms[Tier.DEVICE] == 0 and c.available(Tier.DEVICE) == 2
    up = c.start_promote(a, Tier.HOST, Tier.DEVICE)
    c.complete_op(up, True)
    m = c.match(toks(1, 2))
    assert m.matched_atoms[Tier.DEVICE] == 2 and m.matched_atoms[Tier.HOST] == 2     # promotion keeps the lower copy
    # eviction with demotion: device space is promised once the in-flight copies finish
    c.ensure_capacity(Tier.DEVICE, 2, promote_to=Tier.HOST)
    ops = c.inflight_ops()
    assert len(ops) == 1
    assert c.fail_all_inflight() == 1 and c.inflight_ops() == []
    with pytest.raises(rc.CacheUsageError):
        c.complete_op(ops[0], True)


def test_hybrid_slots():
    h = HybridCache(HybridCacheConfig(CacheConfig(4, 1, device_total_units=32), num_mamba_slots=2, layer_kinds=("attn", "mamba", "attn")))
    assert h.num_layers == 3 and h.is_mamba_layer(1) and not h.is_mamba_layer(0) and h.total_slots == 2
    a, _, _ = put(h.kv, [1, 2, 3, 4])
    s = h.allocate_mamba_slot()
    h.attach_mamba(a, s)
    assert h.active_slots == 1 and not s.valid
    b, _, _ = put(h.kv, [1, 2, 3, 4, 5, 6])
    m = h.match(toks(1, 2, 3, 4, 5, 6, 7, 8))
    assert m.kv.matched_atoms[0] == 6 and m.mamba_node == a and m.mamba_atoms == 4 and m.mamba_slot == s.index
    s2, s3 = h.allocate_mamba_slot(), h.allocate_mamba_slot()
    assert s2 is not None and s3 is None
    del s2                                                   # an unattached slot returns to the pool
    assert h.available_slots == 1
    h.attach_mamba(b, h.allocate_mamba_slot())
    assert h.available_slots == 0 and h.ensure_mamba_capacity_by_evict(1) and h.available_slots == 1
    got = h.detach_mamba(b) or h.detach_mamba(a)
    assert got is not None
    h.kv.ensure_capacity(Tier.DEVICE, 31)                    # evicting the nodes frees attached slots too
    del got
    assert h.available_slots == 2


def test_storage_backends(tmp_path):
    for be in (in_memory_storage_backend(16), file_storage_backend(str(tmp_path / "tier.bin"), 16)):
        assert be.unit_bytes == 16 and be.entries() == 0
        assert be.write(7, b"a" * 32) and be.write(9, b"b" * 16) and not be.write(1, b"short")
        assert be.read(7) == b"a" * 32 and be.contains(9) and be.read(123) is None
        assert be.write(7, b"c" * 16) and be.read(7) == b"c" * 16     # overwrite
        assert be.erase(9) and not be.erase(9) and be.entries() == 1
        be.drain()
    assert hash64(b"abc") == hash64(b"abc") != hash64(b"abd") and hash64(b"abc", 1) != hash64(b"abc")


def test_encodings_and_facades():
    assert encode_eagle_bigram_atoms([5, 6, 7]) == struct.pack("<iiii", 5, 6, 6, 7) and encode_eagle_bigram_atoms([1]) == b""
    atoms = encode_prompt_to_atoms([10, 11, 12], [ImageSegment(0xAB, 0xCD, insert_position=1, length=2)])
    rows = [struct.unpack("<QQ", atoms[i:i + 16]) for i in range(0, len(atoms), 16)]
    assert rows == [(10, 0), (0xAB, 0xCD), (0xAB, 0xCD ^ 1), (11, 0), (12, 0)]
    with pytest.raises(ValueError):
        encode_prompt_to_atoms([1], [ImageSegment(1, 1, 5, 2)])
    assert page_align(b"x" * 10, 4) == (b"x" * 8, 2)
    mm = MultimodalCache({Modality.TEXT: CacheConfig(4, 1, 8), Modality.IMAGE: CacheConfig(16, 4, 8, host_total_units=4)})
    assert Modality.TEXT in mm and mm.stats()[Modality.IMAGE] == {"device_avail": 7, "device_active": 0, "host_avail": 3, "host_active": 0}
    mp = MultiPatternCache({"full": CacheConfig(4, 1, 8), "swa": CacheConfig(4, 1, 8)})
    assert mp.cache_of("swa") is mp["swa"]
    nested = NestedCache({Modality.TEXT: mp, Modality.IMAGE: mm[Modality.IMAGE]})
    assert nested[Modality.TEXT]["full"].total(Tier.DEVICE) == 8
    pc = PairedCache(PairedCacheConfig(CacheConfig(4, 1, 32), CacheConfig(4, 1, 32), window_size=4))
    pc.advance(5)
    fu, su = pc.allocate_pair(2)
    pc.insert_pair(toks(1, 2), fu, su)                       # last touched at step 5
    assert pc.advance(3) == 0 and pc.match(toks(1, 2)).swa.matched_atoms[0] == 2    # now 8, cutoff 4; the match touches at 8
    assert pc.advance(3) == 0     # now 11, cutoff 7 < 8: still inside the window
    assert pc.advance(1) == 2     # now 12, cutoff 8: the window copy goes, the full copy stays
    r = pc.match(toks(1, 2))
    assert r.full.matched_atoms[0] == 2 and r.swa.matched_atoms[0] == 0 and pc.stats()["cur_step"] == 12
