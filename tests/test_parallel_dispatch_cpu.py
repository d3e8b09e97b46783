"""Collective backend registry, policies and dispatcher with stand-in backends: capture filter, preferences per op,
forced backend, cache key (size bucket, mode, mesh identity), the capture-mode context."""

import pytest
import torch

from phyai_b200.parallel import state as pstate
from phyai_b200.parallel.backend import Backend, Call, Mode, Op
from phyai_b200.parallel.dispatch import Dispatcher, size_bucket
from phyai_b200.parallel.exceptions import CaptureUnsafeError, NoBackendError, PhyaiDistError
from phyai_b200.parallel.registry import DefaultPolicy, ForcedPolicy, Registry


class FakeBackend:
    def __init__(self, name, *, ops=tuple(Op), capture=True, max_bytes=None, dtypes=None):
        self.name, self.ops, self.capture, self.max_bytes, self.dtypes = name, set(ops), capture, max_bytes, dtypes
        self.ran = []

    def can_handle(self, call):
        return (call.op in self.ops and (self.max_bytes is None or call.nbytes <= self.max_bytes)
                and (self.dtypes is None or call.dtype in self.dtypes))

    def supports_capture(self):
        return self.capture

    def execute(self, call, *tensors, **kw):
        self.ran.append(call.op)
        return tensors[0] if tensors else None


MESH = object()


def call(op=Op.ALL_REDUCE, nbytes=1024, *, mode=Mode.EAGER, axis="tp", dtype=torch.bfloat16, mesh=MESH, extra=()):
    return Call(op, axis, mesh, dtype, nbytes, mode, "cuda", extra)


def test_stand_in_satisfies_the_backend_protocol():
    assert isinstance(FakeBackend("x"), Backend)


def test_candidates_keep_registration_order_and_honour_preferences():
    reg = Registry()
    reg.register(FakeBackend("nccl"))
    reg.register(FakeBackend("peer", ops=(Op.ALL_REDUCE, Op.ALL_GATHER), max_bytes=4 << 20), prefer_for=[Op.ALL_REDUCE])
    assert [b.name for b in reg.candidates(call())] == ["peer", "nccl"]
    assert [b.name for b in reg.candidates(call(Op.ALL_GATHER))] == ["nccl", "peer"]      # able, not preferred
    assert [b.name for b in reg.candidates(call(nbytes=8 << 20))] == ["nccl"]              # too large for the peer path
    assert [b.name for b in reg.candidates(call(Op.BROADCAST))] == ["nccl"]
    assert reg.names() == ["nccl", "peer"] and reg.get("peer").name == "peer"
    with pytest.raises(KeyError):
        reg.get("gloo")
    with pytest.raises(ValueError, match="already registered"):
        reg.register(FakeBackend("nccl"))


def test_capture_mode_drops_unsafe_backends_and_says_so_when_nothing_is_left():
    reg = Registry()
    reg.register(FakeBackend("unsafe", capture=False))
    reg.register(FakeBackend("safe", ops=(Op.ALL_REDUCE,)))
    capturing = call(mode=Mode.GRAPH_CAPTURING)
    assert [b.name for b in reg.candidates(capturing)] == ["safe"]
    assert [b.name for b in reg.candidates(call())] == ["unsafe", "safe"]
    with pytest.raises(CaptureUnsafeError, match=r"all_gather.*\['unsafe'\]"):
        reg.candidates(call(Op.ALL_GATHER, mode=Mode.GRAPH_CAPTURING))
    assert issubclass(CaptureUnsafeError, PhyaiDistError) and issubclass(NoBackendError, PhyaiDistError)


def test_policies():
    a, b = FakeBackend("a"), FakeBackend("b")
    assert DefaultPolicy().choose(call(), [a, b]) is a
    with pytest.raises(NoBackendError, match=r"all_reduce.*'tp'.*1024 B.*eager"):
        DefaultPolicy().choose(call(), [])
    assert ForcedPolicy("b").choose(call(), [a, b]) is b
    with pytest.raises(NoBackendError, match="forced backend 'c'"):
        ForcedPolicy("c").choose(call(), [a, b])
    with pytest.raises(NoBackendError):
        Registry().validate()


def test_dispatcher_cache_key():
    reg = Registry()
    small, big = FakeBackend("small", max_bytes=4096), FakeBackend("big")
    reg.register(small)
    reg.register(big)
    d = Dispatcher(reg, DefaultPolicy())
    assert d.select(call(nbytes=1024)) is small and (d.hits, d.misses) == (0, 1)
    assert d.select(call(nbytes=1500)) is small and (d.hits, d.misses) == (1, 1)          # same power-of-two bucket
    assert d.select(call(nbytes=8192)) is big and d.misses == 2
    assert d.select(call(nbytes=1024, mode=Mode.GRAPH_CAPTURING)) is small and d.misses == 3
    assert d.select(call(nbytes=1024, mesh=object())) is small and d.misses == 4          # another mesh, another entry
    assert d.select(call(nbytes=1024, axis="cfg")) is small and d.misses == 5
    assert d.select(call(nbytes=1024, dtype=torch.float32)) is small and d.misses == 6
    assert d.select(call(nbytes=1024, extra=("sum",))) is small and d.misses == 7
    d.clear()
    assert d.select(call(nbytes=1024)) is small and d.misses == 8
    assert [size_bucket(n) for n in (0, 1, 2, 3, 4, 1023, 1024)] == [1, 1, 2, 2, 3, 10, 11]


def test_forced_backend_from_the_environment(monkeypatch):
    monkeypatch.setenv("PHYAI_FORCE_BACKEND", "b")
    reg = Registry()
    reg.register(FakeBackend("a"))
    reg.register(FakeBackend("b"))
    d = Dispatcher(reg)
    assert isinstance(d.policy, ForcedPolicy) and d.select(call()).name == "b"
    monkeypatch.delenv("PHYAI_FORCE_BACKEND")
    assert isinstance(Dispatcher(reg).policy, DefaultPolicy)


def test_capture_mode_context_nests_and_restores():
    assert pstate.current_mode() is Mode.EAGER
    with pstate.graph_capture():
        assert pstate.current_mode() is Mode.GRAPH_CAPTURING
        with pstate.graph_capture():
            assert pstate.current_mode() is Mode.GRAPH_CAPTURING
        assert pstate.current_mode() is Mode.GRAPH_CAPTURING
    assert pstate.current_mode() is Mode.EAGER
    with pytest.raises(KeyError, match="no mesh registered"):
        pstate.resolve_mesh("never-registered")
