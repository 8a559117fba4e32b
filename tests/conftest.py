import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built rl_engine._C extension")


@pytest.fixture(autouse=True)
def _device_error_word_is_clean(request):
    """After every GPU test, fail if a kernel recorded a bounded-wait timeout."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if not torch.cuda.is_available():
        return
    from rl_engine.kernels.ops.base import _EXT_AVAILABLE, check_device_errors

    if _EXT_AVAILABLE and request.node.get_closest_marker("expects_device_error") is None:
        check_device_errors(torch.cuda.current_device())
