import ctypes
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU machine with -m gpu)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _checked_build_reports_no_violation():
    """Under the checked-access debug build (OZB_LIBRARY points at it and OZB_CHECK_BOUNDS is set, as
    tests/test_gpu_bounds_build.py arranges for its child run) every test must end without a recorded violation."""
    yield
    if os.environ.get("OZB_CHECK_BOUNDS"):
        from ozaki_blackwell_b200._lib import lib
        out = (ctypes.c_ulonglong * 4)()
        rc = lib.ozb_bounds_report(ctypes.byref(out))
        assert rc == 0 and out[0] == 0, f"rc {rc}: {out[0]} out-of-window accesses, first at {out[1]:#x} ({out[3]} bytes) in kernel {out[2]}"
