import os
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _engine_config_default(request):
    """CPU fp32 config for plain tests, CUDA bf16 for GPU tests; singletons reset around every test."""
    from phyai_b200 import engine_config as ec
    from phyai_b200.layers.linear import kernels

    if "gpu" in request.keywords:
        ec.set_engine_config(ec.EngineConfig(device=ec.DeviceConfig("cuda", torch.bfloat16)))
    else:
        ec.set_engine_config(ec.EngineConfig(device=ec.DeviceConfig("cpu", torch.float32),
                                             runtime=ec.RuntimeConfig(use_cuda_graph=False)))
    kernels._reset_for_test()
    yield
    ec.reset_engine_config()
    kernels._reset_for_test()
