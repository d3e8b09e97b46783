"""Python face of the C++ prefix cache (``phyai_b200._radix``).

The cache stores *unit ids*, never payloads: a unit is one page of caller-owned storage (a KV page,
a row block of embeddings). Atoms travel as ``bytes``. Node handles are opaque integers that stay
valid until the node is evicted everywhere; a stale handle raises :class:`CacheUsageError`.

Reference surface: phyai-ext/src/phyai_ext/radix_cache/__init__.py:48-725.
"""

from __future__ import annotations

import enum
import importlib
from typing import Callable, Optional, Sequence

_mod = None


def _native():
    global _mod
    if _mod is None:
        try:
            _mod = importlib.import_module("phyai_b200._radix")
        except ImportError as e:  # pragma: no cover
            raise RuntimeError("phyai_b200._radix is not built; run `python -m phyai_b200.build_ext`") from e
    return _mod


class Tier(enum.IntEnum):
    DEVICE = 0
    HOST = 1
    DISK = 2
    REMOTE = 3


class CacheEventKind(enum.IntEnum):
    INSERT = 0
    EVICT = 1
    DEMOTE_START = 2
    PROMOTE_START = 3
    OP_DONE = 4
    OP_FAILED = 5
    MAMBA_EVICT = 6


class CacheError(Exception):
    pass


def _exc(name: str):
    return getattr(_native(), name)


def __getattr__(name: str):
    if name in ("CacheCapacityError", "CacheUsageError", "CacheInvariantError"):
        return _exc(name)
    raise AttributeError(name)


def _to_bytes(x) -> bytes:
    if isinstance(x, bytes):
        return x
    if isinstance(x, (bytearray, memoryview)):
        return bytes(x)
    raise TypeError(f"atoms must be bytes-like, got {type(x).__name__}")


class MatchResult:
    """Per tier: the deepest node whose whole path is resident there, and how many atoms it covers."""

    __slots__ = ("last_node", "matched_atoms")

    def __init__(self, last_node: Sequence[int], matched_atoms: Sequence[int]) -> None:
        self.last_node, self.matched_atoms = list(last_node), list(matched_atoms)

    def __repr__(self) -> str:
        return f"MatchResult(matched_atoms={self.matched_atoms})"


class HybridMatchResult:
    __slots__ = ("kv", "mamba_node", "mamba_atoms", "mamba_slot")

    def __init__(self, kv: MatchResult, mamba_node: int, mamba_atoms: int, mamba_slot: int) -> None:
        self.kv, self.mamba_node, self.mamba_atoms, self.mamba_slot = kv, mamba_node, mamba_atoms, mamba_slot


class PrefixCache:
    def __init__(self, atom_bytes: int, atoms_per_unit: int, device_total_units: int, host_total_units: int = 0,
                 disk_total_units: int = 0, remote_total_units: int = 0, eviction_policy: str = "lru", slru_threshold: int = 2,
                 max_events_buffered: int = 16384, device_max_pending_units: int = 0, host_max_pending_units: int = 0,
                 disk_max_pending_units: int = 0, remote_max_pending_units: int = 0) -> None:
        self._atom_bytes, self._atoms_per_unit = int(atom_bytes), int(atoms_per_unit)
        self._policy, self._slru = str(eviction_policy), int(slru_threshold)
        self._impl = _native().PrefixCache(
            self._atom_bytes, self._atoms_per_unit,
            [int(device_total_units), int(host_total_units), int(disk_total_units), int(remote_total_units)],
            [int(device_max_pending_units), int(host_max_pending_units), int(disk_max_pending_units), int(remote_max_pending_units)],
            self._policy, self._slru, int(max_events_buffered))

    # ---- configuration
    atom_bytes = property(lambda s: s._atom_bytes)
    atoms_per_unit = property(lambda s: s._atoms_per_unit)
    page_bytes = property(lambda s: s._atom_bytes * s._atoms_per_unit)
    policy_name = property(lambda s: s._policy)
    slru_threshold = property(lambda s: s._slru)
    impl = property(lambda s: s._impl)

    def tier_enabled(self, tier: Tier) -> bool:
        return self._impl.tier_enabled(int(tier))

    # ---- query / write
    def match(self, atoms) -> MatchResult:
        return MatchResult(*self._impl.match(_to_bytes(atoms)))

    def collect_units(self, last_node: int, tier: Tier):
        """Unit ids on the path root -> ``last_node`` as an int32 tensor (a fresh copy: it stays valid after evictions)."""
        ids = self._impl.collect_units(int(last_node), int(tier))
        try:
            import torch

            return torch.tensor(ids, dtype=torch.int32)
        except ImportError:  # pragma: no cover
            return ids

    def insert(self, tier: Tier, atoms, units) -> tuple[int, int, int]:
        """-> (last node, atoms newly cached, units returned to the pool because their pages were cached already)."""
        return tuple(self._impl.insert(int(tier), _to_bytes(atoms), units))

    def allocate(self, tier: Tier, n: int):
        return self._impl.allocate(int(tier), int(n))

    def lock(self, tier: Tier, last_node: int):
        return self._impl.lock(int(last_node), [int(tier)])

    def lock_multi(self, last_node: int, tiers: Sequence[Tier]):
        return self._impl.lock(int(last_node), [int(t) for t in tiers])

    # ---- capacity
    def ensure_capacity(self, tier: Tier, n: int, promote_to: Optional[Tier] = None) -> None:
        self._impl.ensure_capacity(int(tier), int(n), -1 if promote_to is None else int(promote_to))

    def evict_by_predicate(self, tier: Tier, callback: Callable[[int, int, int, int, int], bool]) -> int:
        """``callback(node_handle, depth_atoms, hits, last_step, priority)`` -> evict?"""
        return int(self._impl.evict_by_predicate(int(tier), callback))

    def evict_by_named_predicate(self, tier: Tier, predicate: str, arg: int) -> int:
        """Built-in predicates: step_le, step_lt, hits_lt, priority_le, age_ns_ge."""
        return int(self._impl.evict_by_named_predicate(int(tier), str(predicate), int(arg)))

    def available(self, tier: Tier) -> int:
        return self._impl.available(int(tier))

    def total(self, tier: Tier) -> int:
        return self._impl.total(int(tier))

    def active(self, tier: Tier) -> int:
        return self._impl.active(int(tier))

    def pending_units(self, tier: Tier) -> int:
        return self._impl.pending_units(int(tier))

    def max_pending_units(self, tier: Tier) -> int:
        return self._impl.max_pending_units(int(tier))

    # ---- two-phase moves between tiers
    def start_demote(self, node: int, src: Tier, dst: Tier) -> int:
        return self._impl.start_demote(int(node), int(src), int(dst))

    def start_promote(self, node: int, src: Tier, dst: Tier) -> int:
        return self._impl.start_promote(int(node), int(src), int(dst))

    def complete_op(self, handle: int, success: bool) -> None:
        self._impl.complete_op(int(handle), bool(success))

    def wait_op(self, handle: int, timeout_ms: int = 0) -> bool:
        return self._impl.wait_op(int(handle), int(timeout_ms))

    def fail_all_inflight(self) -> int:
        return self._impl.fail_all_inflight()

    def inflight_ops(self) -> list[int]:
        return list(self._impl.inflight_ops())

    # ---- observers / events / steps
    def add_evict_observer(self, callback: Callable[[int, int], None]) -> int:
        return self._impl.add_evict_observer(callback)

    def remove_evict_observer(self, observer_id: int) -> bool:
        return self._impl.remove_evict_observer(int(observer_id))

    def take_events(self):
        return self._impl.take_events()

    dropped_events = property(lambda s: s._impl.dropped_events)
    current_step = property(lambda s: s._impl.current_step)
    node_count = property(lambda s: s._impl.node_count)

    def advance_step(self, n: int) -> None:
        self._impl.advance_step(int(n))

    def touch_step(self, node_handle: int) -> None:
        self._impl.touch_step(int(node_handle))

    def node_path_hash(self, node_handle: int) -> int:
        return self._impl.node_path_hash(int(node_handle))

    def node_info(self, node_handle: int) -> dict:
        return dict(self._impl.node_info(int(node_handle)))

    def set_priority(self, node_handle: int, priority: int) -> None:
        self._impl.set_priority(int(node_handle), int(priority))


class MambaSlot:
    """A recurrent-state slot taken from the hybrid cache's pool; goes back unless attached to a node."""

    def __init__(self, owner: "HybridPrefixCache", index: int) -> None:
        self._owner, self.index, self._held = owner, int(index), True

    @property
    def valid(self) -> bool:
        return self._held

    def _consume(self) -> int:
        self._held = False
        return self.index

    def __del__(self):
        if getattr(self, "_held", False):
            try:
                self._owner._impl.free_slot(self.index)
            except Exception:
                pass


class HybridPrefixCache:
    def __init__(self, kv: PrefixCache, num_mamba_slots: int) -> None:
        self._kv = kv
        self._impl = _native().HybridPrefixCache(kv.impl, int(num_mamba_slots))

    kv = property(lambda s: s._kv)

    def match(self, atoms) -> HybridMatchResult:
        ln, ma, node, atoms_n, slot = self._impl.match(_to_bytes(atoms))
        return HybridMatchResult(MatchResult(ln, ma), node, atoms_n, slot)

    def allocate_mamba_slot(self) -> Optional[MambaSlot]:
        i = self._impl.allocate_slot()
        return None if i < 0 else MambaSlot(self, i)

    def attach_mamba(self, node_handle: int, slot: MambaSlot) -> None:
        if not slot.valid:
            raise _exc("CacheUsageError")("slot was already attached or released")
        self._impl.attach(int(node_handle), slot.index)
        slot._consume()

    def detach_mamba(self, node_handle: int) -> Optional[MambaSlot]:
        i = self._impl.detach(int(node_handle))
        return None if i < 0 else MambaSlot(self, i)

    def find_last_mamba_node(self, from_handle: int) -> int:
        return self._impl.find_last_mamba_node(int(from_handle))

    def ensure_mamba_capacity_by_evict(self, n: int) -> bool:
        return self._impl.ensure_slots_by_evict(int(n))

    available_slots = property(lambda s: s._impl.available_slots)
    total_slots = property(lambda s: s._impl.total_slots)
    active_slots = property(lambda s: s._impl.active_slots)


class StorageBackend:
    """Payload store of a lower tier, keyed by a 64-bit id (for instance ``node_path_hash``)."""

    def __init__(self, impl) -> None:
        self._impl = impl

    impl = property(lambda s: s._impl)
    name = property(lambda s: s._impl.name)
    unit_bytes = property(lambda s: s._impl.unit_bytes)

    def write(self, key: int, payload) -> bool:
        return self._impl.write(int(key), _to_bytes(payload))

    def read(self, key: int) -> Optional[bytes]:
        return self._impl.read(int(key))

    def contains(self, key: int) -> bool:
        return self._impl.contains(int(key))

    def erase(self, key: int) -> bool:
        return self._impl.erase(int(key))

    def entries(self) -> int:
        return self._impl.entries()

    def drain(self) -> None:
        self._impl.drain()


def in_memory_storage_backend(unit_bytes: int) -> StorageBackend:
    return StorageBackend(_native().memory_backend(int(unit_bytes)))


def file_storage_backend(path: str, unit_bytes: int) -> StorageBackend:
    return StorageBackend(_native().file_backend(str(path), int(unit_bytes)))


def hash64(data, seed: int = 0) -> int:
    return _native().hash64(_to_bytes(data), int(seed))
