import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "slow: long-running")


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
def _check_kernel_status(request):
    """After every GPU test, no kernel may have recorded a timed-out wait or a rejected index."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from antfly_b200 import _native

            st = _native.status(clear=True)
            assert st == 0, f"kernel status word is {st:#x} (a bounded wait gave up or an index was rejected)"
