"""Shared fixtures. Tests marked `gpu` need a B200 and call the CUDA library through
its C ABI; everything else runs on CPU only."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def orc():
    from oracle import binding
    return binding.oracle()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "blocks.npz"))


@pytest.fixture(scope="session")
def cuda():
    """The C ABI, with a device selected. GPU tests fail (not skip) when it is missing."""
    from tensormark_b200 import lib
    L = lib.load()
    assert L.tm_cuda_init(-1), lib.last_error()
    return L


@pytest.fixture(scope="session")
def torch_mod():
    import torch
    assert torch.cuda.is_available(), "a gpu-marked test ran without a CUDA device"
    return torch


@pytest.fixture(autouse=True)
def _fresh_weight_registrations(request):
    """Weight copies on the device are keyed by host address; numpy reuses addresses between tests."""
    yield
    if request.node.get_closest_marker("gpu"):
        from tensormark_b200 import lib
        lib.load().tm_cuda_release_weights()
