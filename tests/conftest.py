"""Pytest configuration: markers, import path, and GPU gating."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _no_kernel_gave_up_a_wait(request):
    """After every GPU test: no tcgen05 kernel may have abandoned one of its bounded barrier waits
    (the device status word stays 0); the word is cleared so that one failure is reported once."""
    yield
    if "gpu" not in request.keywords or not torch.cuda.is_available():
        return
    import ctypes

    from flashqla_b200 import _lib

    torch.cuda.synchronize()
    status = ctypes.c_int(0)
    rc = _lib.load().fqla_device_status(ctypes.byref(status), 1)
    assert rc == 0, f"fqla_device_status failed with {rc}"
    assert status.value == 0, "a kernel abandoned a bounded barrier wait (device status word set)"
