import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """After every GPU test, make sure no kernel reported a wait that gave up."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from omni_infer_b200.ops import _native as nat

            torch.cuda.synchronize()
            nat.check_status()
