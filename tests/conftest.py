import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def rt():
    """The ctypes runtime with device 0 initialised (GPU tests only)."""
    from appy_b200.backends.cuda_sm100 import runtime
    if runtime.device_count() < 1:
        pytest.fail("no CUDA device visible: GPU tests must run on a GPU box")
    runtime.init(0)
    return runtime
