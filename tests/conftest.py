import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
for p in (os.path.join(ROOT, "mlx-swift-lm_b200", "python"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    import kvcache_oracle
    kvcache_oracle.build()
    return kvcache_oracle


@pytest.fixture(scope="session")
def kvc():
    """The ctypes binding of the CUDA library (built on demand, never faked)."""
    lib = os.path.join(ROOT, "mlx-swift-lm_b200", "lib", "libkvcache_b200.so")
    if not os.path.exists(lib):
        import importlib.util
        spec = importlib.util.spec_from_file_location("kvc_build", os.path.join(ROOT, "mlx-swift-lm_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    import kvcache_b200
    return kvcache_b200


@pytest.fixture(scope="session")
def cuda(kvc):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    assert kvc.device_available(), "library does not see an sm_100 device"
    return torch.device("cuda:0")
