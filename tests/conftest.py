import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
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
def _reset_globals():
    yield
    from minisglang_rdna4_b200.core import set_global_ctx
    from minisglang_rdna4_b200.parallel.info import reset_parallel_info
    from minisglang_rdna4_b200.parallel.comm import reset_comm

    set_global_ctx(None)
    reset_parallel_info()
    reset_comm()
