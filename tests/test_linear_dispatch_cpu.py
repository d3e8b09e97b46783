"""Linear kernel registry and dispatcher on CPU with stand-in kernels: preference per (spec, regime), capture filter,
SM and device gating, forced kernel, the cache key, and where an unsupported spec is reported."""

import pytest
import torch

from phyai_b200.layers.linear import kernels as K


class FakeKernel:
    def __init__(self, name, specs=("bf16",), *, min_sm=0, capture=True, devices=("cpu", "cuda")):
        self.name, self.specs, self.min_sm = name, frozenset(specs), min_sm
        self.device_types, self._capture, self.calls = frozenset(devices), capture, 0

    def supports_capture(self):
        return self._capture

    def apply(self, layer, x, bias):
        self.calls += 1
        return torch.nn.functional.linear(x, layer.weight, bias)


def probe(spec="bf16", M=16, *, device="cpu", capturing=False):
    return K.KernelProbe(spec, M, 64, 32, torch.bfloat16, torch.bfloat16, device, capturing)


def select(d, spec="bf16", M=16, **kw):
    return d.select(spec_id=spec, M=M, N=64, K=32, in_dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                    device_type=kw.pop("device", "cpu"), **kw)


def test_regime_is_decode_up_to_four_rows():
    assert [probe(M=m).regime for m in (1, 4, 5, 4096)] == ["decode", "decode", "prefill", "prefill"]


def test_registration_order_then_preference_per_spec_and_regime():
    reg = K.Registry()
    a, b = FakeKernel("a"), FakeKernel("b")
    reg.register(a)
    reg.register(b, prefer_for=[("bf16", "decode")])
    assert [k.name for k in reg.candidates(probe(M=1), 0)] == ["b", "a"]          # preferred for decode
    assert [k.name for k in reg.candidates(probe(M=64), 0)] == ["a", "b"]         # registration order elsewhere
    with pytest.raises(ValueError, match="already registered"):
        reg.register(FakeKernel("a"))
    assert reg.names() == ["a", "b"]


def test_candidates_filter_spec_device_sm_and_capture():
    reg = K.Registry()
    reg.register(FakeKernel("fp8only", specs=("fp8_per_tensor",)))
    reg.register(FakeKernel("gpu100", min_sm=100, devices=("cuda",)))
    reg.register(FakeKernel("nocapture", capture=False))
    names = lambda p, sm: [k.name for k in reg.candidates(p, sm)]  # noqa: E731
    assert names(probe(), 0) == ["nocapture"]                                       # CPU: the CUDA-only kernel is out
    assert names(probe(device="cuda"), 90) == ["nocapture"]                         # an older SM: still out
    assert names(probe(device="cuda"), 100) == ["gpu100", "nocapture"]
    assert names(probe(device="cuda", capturing=True), 100) == ["gpu100"]           # capture drops the unsafe one
    assert names(probe("fp8_per_tensor"), 0) == ["fp8only"]
    assert reg.supported_specs_for_sm(90) == {"fp8_per_tensor", "bf16"}
    assert reg.supported_specs_for_sm(0, "cpu") == {"fp8_per_tensor", "bf16"}


def test_empty_registry_does_not_validate():
    with pytest.raises(RuntimeError, match="no linear kernel registered"):
        K.Registry().validate()


def test_dispatcher_caches_per_row_bucket_and_mode():
    reg = K.Registry()
    a, b = FakeKernel("a"), FakeKernel("b", capture=False)
    reg.register(b)
    reg.register(a)
    d = K.Dispatcher(reg)
    assert select(d, M=16).name == "b" and select(d, M=31).name == "b"
    assert len(d._cache) == 1                                                        # 16 and 31 share a bucket
    assert select(d, M=32).name == "b" and len(d._cache) == 2
    assert select(d, M=16, capturing=True).name == "a" and len(d._cache) == 3        # capturing is part of the key
    assert select(d, M=0).name == "b"                                                # an empty batch is the one-row bucket
    assert len(d._cache) == 4


def test_forced_kernel_and_its_absence():
    reg = K.Registry()
    reg.register(FakeKernel("a"))
    reg.register(FakeKernel("b", specs=("fp8_per_tensor",)))
    assert select(K.Dispatcher(reg, forced="a")).name == "a"
    with pytest.raises(RuntimeError, match=r"forced='b'"):
        select(K.Dispatcher(reg, forced="b"))          # b exists, but not for bf16
    with pytest.raises(RuntimeError, match="registered: \\['a', 'b'\\]"):
        select(K.Dispatcher(reg, forced="nobody"))


def test_unsupported_spec_is_reported_at_the_first_call_not_at_construction(monkeypatch):
    """A layer with an fp8 spec can be built anywhere; the error comes when a kernel has to be chosen on an SM no
    registered kernel serves, and it names the spec, the SM and the shape."""
    reg = K.Registry()
    reg.register(FakeKernel("new", specs=("fp8_block_128_128",), min_sm=100, devices=("cuda",)))
    d = K.Dispatcher(reg)
    monkeypatch.setattr(K, "sm_arch", lambda: 86)
    with pytest.raises(RuntimeError, match=r"fp8_block_128_128.*sm_86.*M=8"):
        select(d, "fp8_block_128_128", M=8, device="cuda")
    monkeypatch.setattr(K, "sm_arch", lambda: 100)
    assert select(d, "fp8_block_128_128", M=8, device="cuda").name == "new"


def test_init_installs_both_providers_and_honours_the_forced_name():
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config

    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    K._reset_for_test()
    d = K.get_linear_dispatcher()
    assert d.registry.names() == ["b200", "torch"] and d.forced is None
    assert select(d).name == "torch"                    # CPU: the CUDA provider does not apply
    assert K.init(force="torch").forced == "torch"
    K._reset_for_test()


def test_torch_kernel_runs_plain_and_quantised_layers():
    from phyai_b200.engine_config import DeviceConfig, EngineConfig, init_engine_config
    from phyai_b200.layers.linear import ReplicatedLinear

    init_engine_config(EngineConfig(device=DeviceConfig("cpu", torch.float32)))
    K._reset_for_test()
    layer = ReplicatedLinear(32, 16, bias=True, params_dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    layer.weight.data.copy_(torch.randn(16, 32, generator=g))
    layer.bias.data.copy_(torch.randn(16, generator=g))
    x = torch.randn(5, 32, generator=g)
    y, _ = layer(x)
    assert torch.allclose(y, x @ layer.weight.t() + layer.bias, atol=1e-5)
    K._reset_for_test()
