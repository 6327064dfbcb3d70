import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _cuda_present():
    # Device nodes, not the library: with a GPU present a missing or broken CUDA
    # library must fail the GPU tests loudly instead of skipping them.
    return os.path.exists("/dev/nvidiactl") or os.path.exists("/dev/nvidia0")


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with -m gpu; when they are collected on a machine without a
    # device (plain `pytest tests/`), skip them instead of failing.
    if _cuda_present():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
