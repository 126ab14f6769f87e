import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _no_expired_device_waits(request):
    """After every GPU test: no bounded wait inside a tensor-core kernel may have expired."""
    yield
    if "gpu" in request.keywords:
        from mogankda_b200 import _lib
        assert _lib.device_status() == 0, "a bounded wait inside a tensor-core kernel expired (see mkda_device_status)"
