import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
        n_gpu = torch.cuda.device_count() if has_gpu else 0
    except Exception:
        has_gpu, n_gpu = False, 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not has_gpu:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, fail if a bounded wait inside a kernel gave up."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from idrak_b200 import _native
            torch.cuda.synchronize()
            _native.check_status(request.node.name)
