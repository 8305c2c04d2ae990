import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected by -m 'not gpu'")


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
def _kernel_status_guard(request):
    """After every GPU test: fail if a kernel recorded a bounded-wait timeout."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from machx_inference_engine_b200.ops import cuda as K
            K.check_status()
