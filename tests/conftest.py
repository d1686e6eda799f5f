import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def lib():
    from flydsl_b200 import _lib
    return _lib.load()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test: no kernel may have reported a bounded-wait timeout."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from flydsl_b200 import _lib
            assert _lib.device_status() == 0, "a kernel reported a device-side timeout"
