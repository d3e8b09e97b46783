"""Host-side bookkeeping of the peer-memory all-reduce backend and of the per-step status check (no GPU)."""

import pytest
import torch

from phyai_b200.parallel.backend import Call, Mode, Op
from phyai_b200.parallel.backends.peer import PeerBackend
from phyai_b200.parallel.exceptions import CommTimeoutError


class _FakeStream:
    def __init__(self, rows, cols):
        self.max_rows, self.max_cols, self.calls = rows, cols, []

    def all_reduce(self, flat):
        assert flat.dim() == 2 and flat.shape[1] == self.max_cols and flat.shape[0] <= self.max_rows
        self.calls.append(tuple(flat.shape))
        return flat * 2          # "sum over two ranks holding the same tensor"


class _FakeGroup:
    def __init__(self, heap_bytes):
        self.heap_bytes, self.used, self.streams, self.closed = heap_bytes, 0, {}, False

    def stream(self, name, rows, cols):
        if name not in self.streams:
            need = 2 * 2 * rows * cols * 2          # two parities x two ranks x bf16
            if self.used + need > self.heap_bytes:
                raise MemoryError("symmetric heap exhausted")
            self.used += need
            self.streams[name] = _FakeStream(rows, cols)
        return self.streams[name]

    def close(self):
        self.closed = True


class _Mesh:
    device_type = "cuda"

    def axis_size(self, axis):
        return 2


def _call(mesh, x, axis="tp"):
    return Call(op=Op.ALL_REDUCE, axis=axis, mesh=mesh, dtype=x.dtype, device_type="cuda", nbytes=x.numel() * 2, mode=Mode.EAGER, extra=("sum",))


def test_fifty_shapes_share_one_stream(monkeypatch):
    mesh = _Mesh()
    be = PeerBackend(mesh)
    group = _FakeGroup(256 << 20)
    monkeypatch.setattr(be, "_open_group", lambda axis: group)
    for L in range(1, 51):                      # one distinct (768 + L) x 2048 prefix shape per prompt length
        x = torch.randn(7 + L, 264, dtype=torch.float32).bfloat16()
        call = _call(mesh, x)
        assert be.can_handle(call)
        out = be.execute(call, x)
        assert out.shape == x.shape and torch.equal(out, x * 2)
    assert len(group.streams) == 1              # slots are sized once, for max_bytes
    st = next(iter(group.streams.values()))
    assert len(st.calls) == 50 and group.used == 2 * 2 * be.max_rows * be.COLS * 2
    be.close()
    assert group.closed


def test_exhausted_heap_declines_instead_of_raising(monkeypatch):
    mesh = _Mesh()
    be = PeerBackend(mesh)
    monkeypatch.setattr(be, "_open_group", lambda axis: _FakeGroup(1 << 20))   # too small for the stream
    x = torch.zeros(64, 1024, dtype=torch.bfloat16)
    assert not be.can_handle(_call(mesh, x))    # the dispatcher moves on to NCCL
    assert not be.can_handle(_call(mesh, x))    # and the failure is remembered, not retried per call
    with pytest.raises(RuntimeError):
        be.execute(_call(mesh, x), x)


def test_flatten_pads_the_tail():
    x = torch.arange(3000, dtype=torch.float32).bfloat16()
    flat = PeerBackend.flatten(x)
    assert flat.shape == (3, 1024) and torch.equal(flat.view(-1)[:3000], x) and float(flat.view(-1)[3000:].abs().sum()) == 0
    y = torch.zeros(4, 512, dtype=torch.bfloat16)
    assert PeerBackend.flatten(y).data_ptr() == y.data_ptr()      # a view when the size divides


def test_step_status_check_raises_and_is_silent_when_clean(monkeypatch):
    from phyai_b200 import ops
    from phyai_b200.parallel import health

    seen = iter([0, 4, 3])
    monkeypatch.setattr(ops, "kernel_status", lambda: next(seen))
    health.check_step_status(force=True)                       # 0: nothing
    with pytest.raises(CommTimeoutError):
        health.check_step_status(what="cosmos3.step", force=True)
    with pytest.raises(RuntimeError):
        health.check_step_status(force=True)


def test_collectives_are_registered_ops_with_shape_only_fakes():
    """The tensor-valued collectives exist as ``torch.ops.phyai_b200.*`` and can be traced with fake tensors."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from phyai_b200.parallel import state
    from phyai_b200.parallel.mesh import Mesh

    mesh = Mesh((1, 4), ("cfg", "tp"), rank=1, build_groups=False, device_type="cpu")
    state.register_mesh("fake_tp4", mesh)
    try:
        with FakeTensorMode():
            x = torch.empty(8, 6)
            assert tuple(torch.ops.phyai_b200.all_reduce(x, "fake_tp4", "tp", "sum").shape) == (8, 6)
            assert tuple(torch.ops.phyai_b200.all_gather(x, "fake_tp4", "tp", 1).shape) == (8, 24)
            assert tuple(torch.ops.phyai_b200.reduce_scatter(x, "fake_tp4", "tp", 0, "sum").shape) == (2, 6)
            assert tuple(torch.ops.phyai_b200.all_to_all(x, "fake_tp4", "tp", 0, 1).shape) == (2, 24)
            assert tuple(torch.ops.phyai_b200.broadcast(x, "fake_tp4", "tp", 0).shape) == (8, 6)
            with pytest.raises(Exception):
                torch.ops.phyai_b200.reduce_scatter(torch.empty(7, 6), "fake_tp4", "tp", 0, "sum")
        assert state.mesh_name(mesh) == "fake_tp4"
    finally:
        state.unregister_mesh("fake_tp4")


def test_symmetric_heap_guard_bands():
    """The heap allocator with guard bands (host arithmetic on a CPU slab): allocations stay aligned and apart, the
    bands are found intact, and a store one byte past a buffer, or one byte in front of it, is reported with its offset."""
    from phyai_b200.parallel import symm

    def heap(guard: int):
        g = object.__new__(symm.PeerGroup)
        g.pos, g.sig_bytes, g.heap_bytes, g.guard_bytes = 0, 1024, 1024 + 8192, guard
        g.slab = torch.zeros(g.heap_bytes, dtype=torch.uint8)
        g._top, g._guards = g.sig_bytes, []
        return g

    plain = heap(0)
    assert [plain.alloc(n) for n in (100, 256, 257)] == [1024, 1280, 1536] and plain._top == 2048
    plain.check_guards()                                   # nothing to check, nothing raised

    g = heap(256)
    offs = [g.alloc(n) for n in (100, 256, 257)]
    assert offs == [1280, 1792, 2304] and all(o % 256 == 0 for o in offs)
    assert g._guards == [(1024, 1280), (1380, 1792), (2048, 2304), (2561, 3072)] and g._top == 3072
    g.check_guards()
    g.slab[offs[1]:offs[1] + 256].fill_(7)                 # a full write of the buffer leaves the bands alone
    g.check_guards()
    g.slab[offs[1] + 256] = 1                              # one byte behind it
    with pytest.raises(symm.PeerGuardError, match="offset 2048"):
        g.check_guards()
    g.slab[offs[1] + 256] = 0xA5
    g.slab[offs[2] - 1] = 0                                # one byte in front of the next buffer
    with pytest.raises(symm.PeerGuardError, match="offset 2303"):
        g.check_guards()
    g.slab[offs[2] - 1] = 0xA5
    g.slab[offs[0] + 100] = 3                              # one byte behind a buffer whose size is not a multiple of the alignment
    with pytest.raises(symm.PeerGuardError, match="offset 1380"):
        g.check_guards()
    with pytest.raises(MemoryError):
        g.alloc(8192)
