"""Test configuration: markers and the path set-up shared by every test module."""

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
        n_gpu = torch.cuda.device_count() if have_gpu else 0
    except Exception:  # pragma: no cover
        have_gpu, n_gpu = False, 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device in this process")
    skip_multi = pytest.mark.skip(reason="needs at least two CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not have_gpu:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(skip_multi)
