"""Test configuration: registers the ``gpu`` marker and skips GPU tests when no device exists."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


_MULTI_RANK_FILES = ("test_distributed_gpu.py", "test_distributed_numerics_gpu.py", "test_disagg_gpu.py")


def pytest_collection_modifyitems(config, items):
    # single-GPU tests first: the multi-rank GPU files spawn process groups of 2 to 8 ranks and take most of the
    # suite's time, so a stop at the first failure (-x) there should not hide the kernel and model tests
    items.sort(key=lambda it: 1 if os.path.basename(str(it.fspath)) in _MULTI_RANK_FILES else 0)
    # the randomised GPU schedules judge by token agreement, which fp16 near-ties can dent: they go last
    items.sort(key=lambda it: 1 if os.path.basename(str(it.fspath)) == "test_zzz_engine_fuzz_gpu.py" else 0)
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
