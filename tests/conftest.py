import os
import sys

import pytest

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, _REPO)

# Fixtures written by the reference project's own tools (its tests/Idrak.Tests/data folder) are read through
# IDRAK_REFERENCE_DATA. When the variable is unset, a checkout of the reference beside this repository is used if
# there is one; tests that need the files skip otherwise.
if not os.environ.get("IDRAK_REFERENCE_DATA"):
    _beside = os.path.join(os.path.dirname(_REPO), "reference", "tests", "Idrak.Tests", "data")
    if os.path.isdir(_beside):
        os.environ["IDRAK_REFERENCE_DATA"] = _beside


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
