"""Host-side runtime pieces: shared-memory buffers, SM partitioning against a fake driver, the JIT scaffold,
metrics, heartbeats and device-status translation."""

import ctypes
import multiprocessing as mp
import time

import numpy as np
import pytest
import torch


# ---------------------------------------------------------------- host shm
def _child_writes(handle_json, q):
    from phyai_b200.runtime.ipc_buffer import HostShmBuffer, HostShmHandle

    with HostShmBuffer.attach(HostShmHandle.from_json(handle_json)) as b:
        b.as_numpy((4,), np.float32, offset=16)[:] = [1.0, 2.0, 3.0, 4.0]
        q.put(b.is_creator)


def test_host_shm_buffer_between_processes():
    from phyai_b200.runtime.ipc_buffer import HostShmBuffer, HostShmHandle

    buf = HostShmBuffer.create(64)
    try:
        assert buf.is_creator and buf.nbytes == 64 and HostShmHandle.from_json(buf.handle.to_json()) == buf.handle
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        p = ctx.Process(target=_child_writes, args=(buf.handle.to_json(), q))
        p.start()
        assert q.get(timeout=120) is False
        p.join(60)
        t = buf.as_tensor((4,), torch.float32, offset=16)
        assert t.tolist() == [1.0, 2.0, 3.0, 4.0]
        with pytest.raises(ValueError):
            buf.as_tensor((100,), torch.float32)
        del t
    finally:
        buf.close()


# ---------------------------------------------------------------- vgpu with a fake driver
class FakeDriver:
    def __init__(self, cc=(10, 0), sms=148):
        self.cc, self.sms, self.destroyed, self.made = cc, sms, [], []

    def capability(self, device):
        return self.cc

    def sm_count(self, device):
        return self.sms

    def split(self, device, counts):
        left = self.sms
        out = []
        for c in counts:
            out.append((("res", c), c))
            left -= c
        out.append((("rem", left), left))
        return out

    def make_stream(self, device, resource):
        self.made.append(resource)
        return ("ctx", resource), ("stream", resource)

    def destroy(self, ctx):
        self.destroyed.append(ctx)


def test_vgpu_partitioning_rules_and_lifecycle():
    from phyai_b200 import vgpu

    vgpu._reset_for_tests()
    assert vgpu.get_sm_count_constraint((8, 0)) == (4, 2) and vgpu.get_sm_count_constraint((10, 0)) == (8, 8)
    assert vgpu.round_up_sm_count(1, (10, 0)) == 8 and vgpu.round_up_sm_count(17, (10, 0)) == 24 and vgpu.round_up_sm_count(5, (8, 6)) == 6
    with pytest.raises(vgpu.VGPURuntimeError):
        vgpu.round_up_sm_count(0, (9, 0))
    with pytest.raises(vgpu.VGPURuntimeError):
        vgpu.split_device(2, 8)                      # before init
    with pytest.raises(vgpu.VGPUNotApplicableError):
        vgpu.init(0, driver=FakeDriver(), world_size=2)
    with pytest.raises(vgpu.VGPUNotApplicableError):
        vgpu.init(0, driver=FakeDriver(cc=(7, 5)))
    drv = vgpu.init(0, driver=FakeDriver())
    shards = vgpu.split_device_by_sm_count([20, 100])
    assert [(s.sm_count, s.requested_sm_count, s.is_remainder) for s in shards] == [(24, 20, False), (104, 100, False), (20, 20, True)]
    assert shards[2].name == "shard_2_rem"
    with pytest.raises(vgpu.VGPURuntimeError):
        vgpu.split_device_by_sm_count([100, 60])
    vs = vgpu.create_vgpus([64, 64], include_remainder=False)
    assert len(vs) == 2 and vs[0].sm_count == 64
    with vs[0].activate() as v:
        assert v is vs[0]
    vgpu.close_all()
    assert len(drv.destroyed) == 2
    with pytest.raises(vgpu.VGPURuntimeError):
        with vs[0].activate():
            pass
    vgpu._reset_for_tests()


# ---------------------------------------------------------------- jit (host source: no GPU needed)
def test_jit_compiles_caches_and_specialises(tmp_path, monkeypatch):
    from phyai_b200 import jit as J

    monkeypatch.setenv("PHYAI_B200_JIT_CACHE", str(tmp_path / "cache"))
    (tmp_path / "inc.h").write_text("#define BIAS 5\n")
    src = tmp_path / "k.cpp"
    src.write_text('#include "inc.h"\nextern "C" long long scaled(long long x) { return x * FACTOR + BIAS; }\n')
    assert J.template_macros({"N": 4, "FAST": True, "T": "float"}) == ["-DFAST=1", "-DN=4", "-DT=float"]
    with pytest.raises(ValueError):
        J.template_macros({"bad name": 1})

    def make(factor):
        @J.jit(name="scaled", sources=[src], template_args={"FACTOR": factor}, signatures={"scaled": (ctypes.c_longlong, [ctypes.c_longlong])})
        def call(lib, x):
            return lib.scaled(x)
        return call

    f3, f7 = make(3), make(7)
    assert f3(10) == 35 and f7(10) == 75
    built = sorted(p.name for p in (tmp_path / "cache").iterdir())
    assert len(built) == 2
    lib = J.compile_library("scaled", [src], template_args={"FACTOR": 3})
    stamp = lib.stat().st_mtime_ns
    assert J.compile_library("scaled", [src], template_args={"FACTOR": 3}) == lib and lib.stat().st_mtime_ns == stamp   # cache hit
    (tmp_path / "inc.h").write_text("#define BIAS 6\n")                                                                 # an included header changed
    assert J.compile_library("scaled", [src], template_args={"FACTOR": 3}) != lib
    src.write_text("this is not C++")
    with pytest.raises(RuntimeError):
        J.compile_library("broken", [src])
    assert J.specializations({"T": "float"}, N=[1, 2], FAST=[False, True]) == [
        {"T": "float", "N": 1, "FAST": False}, {"T": "float", "N": 1, "FAST": True},
        {"T": "float", "N": 2, "FAST": False}, {"T": "float", "N": 2, "FAST": True}]


# ---------------------------------------------------------------- metrics
def test_metrics_registry(tmp_path):
    from phyai_b200.utils.metrics import MetricsRegistry

    m = MetricsRegistry()
    for v in (1.0, 2.0, 3.0, 100.0):
        m.observe("step_ms", v)
    m.inc("graph_replays", 3)
    m.inc("plan_hit", 9)
    m.inc("plan_miss")
    m.set("kv_slots_in_use", 42)
    with m.timer("host_ms"):
        time.sleep(0.002)
    s = m.snapshot()
    h = s["histograms"]["step_ms"]
    assert h["count"] == 4 and h["max"] == 100.0 and h["p50"] == 2.5 and h["buckets"]["1.0"] == 1 and h["buckets"]["100.0"] == 1
    assert s["counters"]["graph_replays"] == 3 and m.hit_rate("plan_hit", "plan_miss") == 0.9 and s["histograms"]["host_ms"]["min"] >= 1.5
    assert '"kv_slots_in_use": 42.0' in m.dump(tmp_path / "m.json").read_text()
    text = m.prometheus_text()
    assert 'phyai_b200_step_ms_bucket{le="+Inf"} 4' in text and "phyai_b200_graph_replays 3" in text


# ---------------------------------------------------------------- failure detection on the host
def test_heartbeat_and_status_translation():
    from phyai_b200.parallel import CommTimeoutError, PeerLostError
    from phyai_b200.parallel.health import DictStore, Heartbeat, raise_for_kernel_status

    store, now = DictStore(), [100.0]
    a = Heartbeat(store, 0, 3, interval_s=0, clock=lambda: now[0]).start()
    b = Heartbeat(store, 1, 3, interval_s=0, clock=lambda: now[0]).start()
    assert a.stale_peers(1.0) == [2]                     # rank 2 never joined
    Heartbeat(store, 2, 3, interval_s=0, clock=lambda: now[0]).start()
    a.check_peers(1.0)
    now[0] += 5.0
    b.beat()                                             # rank 1 is alive, rank 2 went silent
    assert a.stale_peers(2.0) == [2]
    with pytest.raises(PeerLostError):
        a.check_peers(2.0)
    raise_for_kernel_status(0)
    with pytest.raises(CommTimeoutError):
        raise_for_kernel_status(4, what="o-proj reduce")
    with pytest.raises(RuntimeError):
        raise_for_kernel_status(1)
    live = Heartbeat(DictStore(), 0, 1, interval_s=0.01).start()
    time.sleep(0.05)
    live.stop()
    assert live._n >= 2


def test_show_env_cli(capsys):
    from phyai_b200.__main__ import main

    assert main(["show-env"]) == 0
    out = capsys.readouterr().out
    import json as _json

    info = _json.loads(out)
    assert "torch" in info and "PHYAI_PEER_COMM" in info["env"] and "jit_cache_dir" in info
    assert main(["nope"]) == 2


def test_vgpu_backend_registry(monkeypatch):
    from phyai_b200 import vgpu

    vgpu._reset_for_tests()
    assert vgpu.known_backends() == ["cuda", "torch"] and vgpu.get_backend() == "auto" and vgpu.GreenCtxBackend is vgpu.TorchGreenDriver
    monkeypatch.setenv("PHYAI_VGPU_BACKEND", "torch")
    assert vgpu.get_backend() == "torch"

    @vgpu.register_vgpu_backend("fake")
    class Fake(FakeDriver):
        pass

    try:
        assert "fake" in vgpu.known_backends()
        vgpu.set_backend("fake")                             # an explicit choice wins over the environment
        assert vgpu.get_backend() == "fake" and isinstance(vgpu.default_driver(), Fake)
        assert isinstance(vgpu.init(0), Fake)
        with pytest.raises(ValueError, match="already registered"):
            vgpu.register_vgpu_backend("fake")(FakeDriver)
        with pytest.raises(vgpu.VGPURuntimeError, match="unknown vGPU backend 'nope'"):
            vgpu.set_backend("nope")
        vgpu.set_backend(None)
        assert vgpu.get_backend() == "torch"
    finally:
        vgpu._BACKENDS.pop("fake", None)
        vgpu._reset_for_tests()
