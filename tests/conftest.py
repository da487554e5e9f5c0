import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    """Without a CUDA device the gpu tests cannot run: skip them instead of failing."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def device_status_is_clean_after_every_gpu_test(request):
    """No kernel of a GPU test may have given up on a wait, nor (in the checking build) met an index outside its
    bounds, without the test having seen it."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch
    if torch.cuda.is_available():
        from tensorline_b200 import ops
        ops.check_device_status()
