import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "slow: long-running CPU test")
    config.addinivalue_line("markers", "expects_status: the test reads the device status word itself")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True)
def _no_kernel_gave_up(request):
    """After every GPU test: no bounded wait inside a tensor-core kernel ran out (a kernel that gives up returns
    normally with garbage, so a parity failure next to a non-zero status word points at the wait, not the math)."""
    yield
    if request.node.get_closest_marker("gpu") is None or request.node.get_closest_marker("expects_status"):
        return
    import torch

    if not torch.cuda.is_available():
        return
    from jax_linear_attention_b200 import _lib

    assert _lib.device_status() == 0, "a tensor-core kernel's bounded wait gave up during this test"
