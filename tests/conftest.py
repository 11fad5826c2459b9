import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu on a GPU box)")


# Files whose tests run after everything else, in this order: the plugin's device-buffer scenarios
# (two processes per test on the GPU) and then the entry point that allocates nothing, so that a
# run that stops at the first failure has already run every other test.
RUN_LAST = ("test_net_device_gpu.py", "test_zz_no_alloc.py")


def pytest_collection_modifyitems(config, items):
    def rank(item):
        name = os.path.basename(str(item.fspath))
        return RUN_LAST.index(name) + 1 if name in RUN_LAST else 0

    items.sort(key=rank)   # stable: every other test keeps its place


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
