import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _engine_for_test(request):
    """Tests without the gpu mark run on a CPU fp32 engine even where a GPU is present; gpu tests get the default engine."""
    from oa_b200.runtime import engine as RT

    prev = RT.OaEngine.GetGlobal()
    if "gpu" in request.keywords:
        yield
        return
    cfg = RT.OaEngineConfig()
    cfg.DevicePreference = RT.OaDevicePreference.Cpu
    cfg.Precision = RT.OaPrecision.FP32
    eng = RT.OaEngine.Create(cfg)
    eng.SetAsGlobal()
    try:
        yield
    finally:
        with RT.OaEngine._lock:
            RT.OaEngine._global = prev
