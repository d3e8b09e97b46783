import pytest
import torch

from phyai_b200 import engine_config as ec
from phyai_b200.env import envs, parse_bool, parse_regex_list


def test_defaults_and_validation():
    c = ec.EngineConfig()
    assert c.backends.attn == "auto" and c.device.params_dtype == torch.bfloat16
    assert c.parallel.layout == (1, 1, 1, 1, 1, 1)
    with pytest.raises(ValueError):
        ec.ParallelConfig(world_size=4, tp_size=2)
    with pytest.raises(ValueError):
        ec.BackendConfig(attn="nope")
    with pytest.raises(ValueError):
        ec.DeviceConfig(target="tpu")
    with pytest.raises(ValueError):
        ec.RuntimeConfig(debug_tensor_dump_filter=("a",), debug_tensor_dump_filter_fn="m:f")


def test_reference_backend_names_are_aliases():
    b = ec.BackendConfig(attn="flashinfer", norm="phyai-kernel")
    assert b.attn == "b200" and b.norm == "b200"
    assert ec.BackendConfig(attn="sdpa").attn == "torch"


def test_env_overlay_and_explicit_precedence(monkeypatch):
    monkeypatch.setenv("PHYAI_USE_CUDA_GRAPH", "0")
    monkeypatch.setenv("PHYAI_TP_SIZE", "2")
    monkeypatch.setenv("PHYAI_PARAMS_DTYPE", "fp16")
    c = ec.EngineConfig.from_env(base=ec.EngineConfig())
    assert c.runtime.use_cuda_graph is False
    assert c.parallel.tp_size == 2 and c.parallel.world_size == 2
    assert c.device.params_dtype == torch.float16
    explicit = ec.EngineConfig(device=ec.DeviceConfig("cpu", torch.float32))
    c2 = ec.EngineConfig.from_env(base=explicit, explicit=explicit)
    assert c2.device.params_dtype == torch.float32      # explicit field beats the environment
    assert c2.runtime.use_cuda_graph is False            # untouched field still takes the environment


def test_replace_and_singleton():
    c = ec.EngineConfig().replace(runtime={"use_cuda_graph": False})
    assert c.runtime.use_cuda_graph is False
    ec.set_engine_config(c)
    assert ec.get_engine_config() is c
    with pytest.raises(TypeError):
        ec.set_engine_config("x")
    with pytest.raises(TypeError):
        c.replace(nope={})


def test_resolve_defaults_by_device():
    ec.set_engine_config(ec.EngineConfig(device=ec.DeviceConfig("cpu", torch.float32)))
    dt, attn, norm = ec.resolve_engine_defaults()
    assert (dt, attn, norm) == (torch.float32, "torch", "torch")
    ec.set_engine_config(ec.EngineConfig(device=ec.DeviceConfig("cuda", torch.bfloat16)))
    assert ec.resolve_engine_defaults()[1:] == ("b200", "b200")
    assert ec.resolve_engine_defaults(norm_backend="torch")[2] == "torch"


def test_env_parsers(monkeypatch):
    assert parse_bool("Yes") and not parse_bool("off")
    with pytest.raises(ValueError):
        parse_bool("maybe")
    assert parse_regex_list('["a.*", "b"]') == ("a.*", "b")
    assert parse_regex_list("layers\\.0") == ("layers\\.0",)
    monkeypatch.setenv("PHYAI_WORLD_SIZE", "x")
    with pytest.raises(ValueError):
        envs.PHYAI_WORLD_SIZE.get()
    assert "PHYAI_TP_SIZE" in envs.fields()


def test_native_env_switches_are_registered():
    """Every PHYAI_* variable the native sources read with getenv() is listed in the env catalogue."""
    import re
    from pathlib import Path

    from phyai_b200.env import envs

    root = Path(__file__).resolve().parents[1] / "phyai_b200" / "csrc"
    used = set()
    for src in list(root.glob("*.cu")) + list(root.glob("*.cuh")) + list(root.glob("*.cpp")):
        used |= set(re.findall(r'getenv\("(PHYAI_[A-Z0-9_]+)"\)', src.read_text()))
    assert used, "expected the kernels to read at least one switch"
    missing = used - set(envs.fields())
    assert not missing, f"register in phyai_b200/env.py: {sorted(missing)}"
