import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an NVIDIA B200 (sm_100a); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # Files whose name starts with test_zz run last whatever order they were found in.
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"),))
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        skip = pytest.mark.skip(reason="no CUDA device")
        for it in items:
            if "gpu" in it.keywords:
                it.add_marker(skip)
