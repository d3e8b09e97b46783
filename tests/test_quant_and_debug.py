"""Quantisation plans / specs, tensor dumper, timeline profiler, CUDA-graph manager fallbacks, payloads (CPU)."""

import json

import pytest
import torch
import torch.nn as nn


def test_importers_recognise_the_three_checkpoint_dialects(tmp_path):
    from phyai_b200.layers.quant import load_quant_plan
    from phyai_b200.layers.quant.importers import import_plan
    from phyai_b200.layers.quant.scheme import Granularity

    hf = import_plan({"quant_method": "fp8", "weight_block_size": [128, 128], "modules_to_not_convert": ["lm_head"]})
    assert hf.resolve("model.layers.0.mlp.down_proj").weight.granularity is Granularity.BLOCK
    assert hf.resolve("lm_head") is None
    ct = import_plan({"quant_method": "compressed-tensors", "ignore": ["re:.*vision.*"], "config_groups": {
        "g0": {"targets": ["Linear"], "weights": {"num_bits": 8, "type": "float", "strategy": "channel"},
               "input_activations": {"num_bits": 8, "type": "float", "dynamic": True}}}})
    from phyai_b200.layers.linear import LinearBase

    assert ct.resolve("decoder.q_proj", LinearBase).spec_id == "fp8_per_channel"
    assert ct.resolve("model.vision.proj", LinearBase) is None
    mo = import_plan({"quantization": {"quant_algo": "NVFP4", "exclude_modules": ["*embed*"]}})
    assert mo.resolve("layers.3.fc1").spec_id == "nvfp4_block_16" and mo.resolve("tok_embed.proj") is None
    with pytest.raises(ValueError):
        import_plan({"quant_algo": "INT3"})
    assert import_plan({"something": "else"}) is None
    (tmp_path / "config.json").write_text(json.dumps({"hidden_size": 8, "quantization_config": {"quant_method": "fp8"}}))
    assert load_quant_plan(tmp_path).resolve("any.linear").spec_id == "fp8_per_tensor"
    assert load_quant_plan(None) is None and load_quant_plan(tmp_path / "missing") is None


@pytest.mark.parametrize("spec_id,tol", [("fp8_per_tensor", 0.08), ("fp8_per_channel", 0.06), ("fp8_block_128_128", 0.06), ("nvfp4_block_16", 0.25)])
def test_quantised_linear_reference_path_tracks_the_dense_product(spec_id, tol):
    from phyai_b200.layers.quant import scheme as S
    from phyai_b200.layers.quant.specs import Fp8Spec, Nvfp4Spec, materialize

    sch = {"fp8_per_tensor": S.FP8_PER_TENSOR, "fp8_per_channel": S.FP8_PER_CHANNEL, "fp8_block_128_128": S.FP8_BLOCK_128,
           "nvfp4_block_16": S.NVFP4_BLOCK_16}[spec_id]
    spec = materialize(sch, sm=100)
    assert spec.spec_id == spec_id
    g = torch.Generator().manual_seed(0)
    w, x = torch.randn(256, 384, generator=g) * 0.1, torch.randn(5, 384, generator=g)
    if isinstance(spec, Fp8Spec):
        q, s = spec.quantize_weight(w)
        assert q.dtype == torch.float8_e4m3fn
        layer = nn.Module()
        layer.weight, layer.weight_scale, layer.spec = nn.Parameter(q, requires_grad=False), nn.Parameter(s, requires_grad=False), spec
        y = spec.reference_apply(layer, x, None)
    else:
        assert isinstance(spec, Nvfp4Spec)
        packed, bs, gs = spec.quantize(w)
        y = x @ spec.dequantize(packed, bs, gs).t()
    want = x @ w.t()
    assert (y.float() - want).abs().max() / want.abs().max() < tol


def test_tensor_dumper_hooks_filters_and_repeated_calls(tmp_path):
    from phyai_b200.runtime.tensor_dump import TensorDumper

    net = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 2))
    d = TensorDumper(tmp_path, patterns=(r"^net\.[02]$",))
    assert d.attach(net, "net") == 2
    x = torch.randn(3, 4)
    net(x)
    net(x)                                   # second call of the same modules inside one pass
    d.record("net.sampler_state", torch.ones(2))      # filtered out by the patterns
    path = d.flush()
    got = TensorDumper.load_pass(d.dir, 0)
    assert path.name == "pass00000.pt" and set(got) == {"net.0", "net.2", "net.0::call1", "net.2::call1"}
    assert torch.equal(got["net.2"], net(x)) and d.flush().name == "pass00001.pt" and d.flush() is None
    d.detach()
    net(x)
    assert d.flush() is None
    with pytest.raises(ValueError):
        TensorDumper(tmp_path, patterns=("a",), predicate=lambda n: True)


def test_timeline_profiler_and_event_scope(tmp_path):
    from phyai_b200.utils.profile import ProfilerConfig, event_scope, get_profiler, install_profiler

    prof = install_profiler(ProfilerConfig(kind="timeline", output_dir=str(tmp_path)))
    prof.start()
    for _ in range(3):
        with event_scope("stage.a"):
            sum(range(1000))
    with event_scope("stage.b"):
        pass
    prof.stop()
    with event_scope("stage.a"):           # not recorded after stop
        pass
    s = get_profiler().summary()
    assert s["stage.a"]["count"] == 3 and s["stage.b"]["count"] == 1 and s["stage.a"]["total_ms"] >= s["stage.a"]["max_ms"] > 0
    assert json.loads(prof.dump().read_text())["stage.a"]["count"] == 3
    install_profiler(None)
    with event_scope("ignored"):
        pass


def test_payload_dataclasses():
    from phyai_b200.payload import ExpertForwardBatch, LLMForwardBatch, VisionForwardBatch

    v = VisionForwardBatch(pixel_values=torch.zeros(3, 3, 8, 8))
    l = LLMForwardBatch(hidden_states=torch.zeros(5, 4), position_ids=torch.arange(5), write_indices=torch.arange(5))
    e = ExpertForwardBatch(x_t=torch.zeros(1, 10, 8), time_emb=torch.zeros(1, 16))
    assert v.pixel_values.shape[0] == 3 and l.position_ids[-1] == 4 and e.x_t.shape == (1, 10, 8)


def test_tensor_dump_filter_function_from_a_file_sees_the_module(tmp_path):
    """The filter function named in the runtime configuration is called with the module as well as its name."""
    from types import SimpleNamespace

    from phyai_b200.runtime.tensor_dump import TensorDumper, load_pass

    src = tmp_path / "pick.py"
    src.write_text("import torch\n\ndef only_linear(name, module):\n    return isinstance(module, torch.nn.Linear)\n\ndef by_name(name):\n    return name.endswith('1')\n")
    net = torch.nn.Sequential(torch.nn.Linear(3, 3), torch.nn.ReLU(), torch.nn.Linear(3, 2))
    for func, want in (("only_linear", ["net.0", "net.2"]), ("by_name", ["net.1"])):
        rt = SimpleNamespace(debug_tensor_dump_dir=tmp_path / func, debug_tensor_dump_filter=None, debug_tensor_dump_filter_fn=f"{src}:{func}")
        d = TensorDumper.from_config(rt)
        assert d.attach(net, prefix="net") == len(want)
        net(torch.ones(1, 3))
        assert list(load_pass(d.flush())) == want
        d.detach()
    with pytest.raises(FileNotFoundError):
        TensorDumper.from_config(SimpleNamespace(debug_tensor_dump_dir=tmp_path, debug_tensor_dump_filter=None, debug_tensor_dump_filter_fn=f"{tmp_path}/absent.py:f"))
