import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ggml_golden.npz"))


@pytest.fixture(scope="session")
def cuda_device():
    """An opened device of the CUDA provider; the GPU tests fail (not skip) when the library cannot load."""
    from sharplight_b200 import CudaExecutionProvider
    provider = CudaExecutionProvider()
    availability = provider.check_availability()
    assert availability.available, f"CUDA provider unavailable: {availability.reason}"
    device = provider.open_device(provider.get_devices()[0])
    yield device
    device.dispose()
