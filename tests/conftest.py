import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on a GPU box)")


@pytest.fixture(scope="session")
def built():
    """Make sure the native libraries are built (incremental, no-op when fresh)."""
    from aws_ofi_nccl_b200 import build

    build.build_all()
    return build.LIB


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, the status word must still be zero (no bounded wait gave up)."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch

        if torch.cuda.is_available():
            from aws_ofi_nccl_b200.ops import _lib

            assert _lib.read_status() == 0
