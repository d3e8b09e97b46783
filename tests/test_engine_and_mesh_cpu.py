"""The plugin host (registration rules, argument type check, lifecycle, metrics, tensor dump forcing the eager path) and
the named-axis mesh (row-major layout with ``tp`` innermost, axis groups, validation), on CPU with a toy plugin."""

from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

from phyai_b200 import DeviceConfig, EngineConfig, RuntimeConfig
from phyai_b200.engine import Engine, EngineArgs, Entry, EntryArgs
from phyai_b200.parallel.mesh import Mesh


def cpu_config(**runtime):
    return EngineConfig(device=DeviceConfig("cpu", torch.float32), runtime=RuntimeConfig(use_cuda_graph=False, **runtime))


@dataclass
class ToyArgs(EntryArgs):
    scale: float = 2.0


class ToyEntry(Entry):
    name: ClassVar[str] = "toy_scale"
    args_cls: ClassVar[type[EntryArgs]] = ToyArgs
    events: ClassVar[list] = []

    def setup(self, args: ToyArgs) -> None:
        self.lin = torch.nn.Linear(4, 4, bias=False)
        with torch.no_grad():
            self.lin.weight.copy_(torch.eye(4) * args.scale)
        self.events.append("setup")

    def step(self, request):
        self.events.append("step")
        return self.lin(request)

    def close(self) -> None:
        self.events.append("close")

    def dump_targets(self):
        return {"toy": self.lin}


@pytest.fixture()
def toy():
    Engine.register(ToyEntry)
    ToyEntry.events.clear()
    yield ToyEntry
    Engine._plugins.pop("toy_scale", None)


def test_register_rules(toy):
    assert Engine.register(ToyEntry) is ToyEntry                  # registering the same class again is harmless

    class Clash(ToyEntry):
        pass

    with pytest.raises(ValueError, match="already taken by ToyEntry"):
        Engine.register(Clash)

    class NoName(Entry):
        args_cls = ToyArgs

    with pytest.raises(TypeError, match="non-empty class attribute `name`"):
        Engine.register(NoName)

    class BadArgs(Entry):
        name = "bad_args"
        args_cls = dict

    with pytest.raises(TypeError, match="must subclass EntryArgs"):
        Engine.register(BadArgs)
    assert "toy_scale" in Engine.plugin_names() and "pi05" in Engine.plugin_names() and "cosmos3_policy_wn" in Engine.plugin_names()


def test_unknown_plugin_and_wrong_argument_type(toy):
    with pytest.raises(KeyError, match="unknown plugin 'nope'"):
        Engine(EngineArgs("nope", ToyArgs(), cpu_config()))

    @dataclass
    class OtherArgs(EntryArgs):
        pass

    with pytest.raises(TypeError, match="expects ToyArgs, got OtherArgs"):
        Engine(EngineArgs("toy_scale", OtherArgs(), cpu_config()))


def test_lifecycle_metrics_and_context_manager(toy):
    from phyai_b200.utils.metrics import metrics

    before = metrics().snapshot()["counters"].get("engine.steps.toy_scale", 0)
    with Engine(EngineArgs("toy_scale", ToyArgs(scale=3.0), cpu_config())) as eng:
        assert eng.plugin_name == "toy_scale" and eng.device.type == "cpu" and eng.mesh.world_size == 1
        out = eng.step(torch.ones(1, 4))
        assert torch.equal(out, torch.full((1, 4), 3.0))
        eng.step(torch.ones(1, 4))
    assert toy.events == ["setup", "step", "step", "close"]
    eng.close()                                                   # a second close is a no-op
    assert toy.events.count("close") == 1
    with pytest.raises(RuntimeError, match="after close"):
        eng.step(torch.ones(1, 4))
    snap = metrics().snapshot()
    assert snap["counters"]["engine.steps.toy_scale"] == before + 2
    assert "engine.step_host_ms.toy_scale" in snap["histograms"]


def test_tensor_dump_switches_graphs_off_and_hooks_the_dump_targets(toy, tmp_path):
    cfg = EngineConfig(device=DeviceConfig("cpu", torch.float32),
                       runtime=RuntimeConfig(use_cuda_graph=True, debug_tensor_dump_dir=str(tmp_path)))
    eng = Engine(EngineArgs("toy_scale", ToyArgs(), cfg))
    assert eng.config.runtime.use_cuda_graph is False             # hooks do not fire on graph replay
    from phyai_b200.runtime.tensor_dump import TensorDumper

    eng.step(torch.ones(2, 4))
    eng.step(torch.ones(2, 4) * 2)
    eng.close()
    files = sorted(tmp_path.rglob("*.pt"))
    assert [f.name for f in files] == ["pass00000.pt", "pass00001.pt"]                   # one file per engine step
    assert files[0].parent.name.startswith("rank0_pid")
    second = TensorDumper.load_pass(files[0].parent, 1)
    assert list(second) == ["toy"] and torch.equal(second["toy"], torch.full((2, 4), 4.0))


# ------------------------------------------------------------------- mesh
AXES = ("dp", "cfg", "ep", "sp", "cp", "tp")


def test_mesh_layout_is_row_major_with_tp_innermost():
    m = Mesh((1, 2, 1, 1, 1, 4), AXES, rank=6, build_groups=False)
    assert m.world_size == 8 and m.coords() == (0, 1, 0, 0, 0, 2) and m.rank_of(m.coords()) == 6
    assert m.axis_ranks("tp") == (4, 5, 6, 7)                     # a TP group is a block of consecutive ranks
    assert m.axis_ranks("cfg") == (2, 6)                          # the partner of the other guidance branch: same tp index
    assert m.axis_local_rank("tp") == 2 and m.axis_local_rank("cfg") == 1 and m.axis_local_rank("dp") == 0
    assert m.axis_size("tp") == 4 and m.axis_size("ep") == 1 and m.axis_size("not_an_axis") == 1
    assert m.axis_ranks("not_an_axis") == (6,) and not m.has_axis("pp") and m.has_axis("sp")
    assert m.axis_group("tp") is None                             # groups were not built
    assert [m.coords(r) for r in (0, 3, 4)] == [(0, 0, 0, 0, 0, 0), (0, 0, 0, 0, 0, 3), (0, 1, 0, 0, 0, 0)]
    top = m.topology("tp")
    assert (top.world_size, top.axis_size) == (8, 4)
    assert "tp=4" in repr(m) and "rank 6/8" in repr(m)


def test_mesh_every_rank_agrees_on_the_groups():
    sizes = (2, 2, 1, 1, 1, 2)
    for axis in ("dp", "cfg", "tp"):
        groups = {Mesh(sizes, AXES, rank=r, build_groups=False).axis_ranks(axis) for r in range(8)}
        assert len(groups) == 8 // sizes[AXES.index(axis)]        # a partition of the ranks
        assert sorted(r for g in groups for r in g) == list(range(8))


def test_mesh_validation():
    with pytest.raises(ValueError, match="differ in length"):
        Mesh((2, 2), ("tp",), build_groups=False)
    with pytest.raises(ValueError, match="duplicate axis names"):
        Mesh((2, 2), ("tp", "tp"), build_groups=False)
    with pytest.raises(ValueError, match="covers 4 ranks, world_size is 8"):
        Mesh((2, 2), ("cfg", "tp"), world_size=8, build_groups=False)
    with pytest.raises(ValueError, match="rank 4 outside"):
        Mesh((2, 2), ("cfg", "tp"), rank=4, build_groups=False)
