"""The checked-access debug build (libozaki_blackwell_bounds.so, -DOZ_BOUNDS): every global load and store of the scale /
residue / reconstruction kernels and of the GEMM epilogue is tested against the exact bytes its launch is entitled to, and
the plan's workspaces start out poisoned. The small, odd-shaped and panel tests are run once more against that build in a
child process; each of them must give the checker's bits AND end without a single recorded violation (tests/conftest.py
asks the library after every test). The memory checker of the CUDA toolkit is not used."""
import ctypes
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BOUNDS = os.path.join(ROOT, "ozaki_blackwell_b200", "libozaki_blackwell_bounds.so")


def _env():
    if not os.path.exists(BOUNDS):
        pytest.fail(f"{BOUNDS} is missing: build it with `make -C ozaki_blackwell_b200/csrc bounds`")
    e = dict(os.environ)
    e.update(OZB_LIBRARY=BOUNDS, OZB_CHECK_BOUNDS="1", PYTHONPATH=os.pathsep.join([HERE, ROOT, e.get("PYTHONPATH", "")]))
    return e


def test_the_checker_records_a_violation_without_performing_it():
    code = r"""
import ctypes
from ozaki_blackwell_b200._lib import lib
out = (ctypes.c_ulonglong * 4)()
assert lib.ozb_bounds_report(ctypes.byref(out)) == 0 and out[0] == 0
assert lib.ozb_selftest_bounds() == 0            # four stores inside the window landed, the fifth was skipped
assert lib.ozb_bounds_report(ctypes.byref(out)) == 0 and out[0] == 1 and out[2] == 7 and out[3] == 4, list(out)
assert lib.ozb_bounds_report(ctypes.byref(out)) == 0 and out[0] == 0      # reading cleared the record
print("ok")
"""
    r = subprocess.run([sys.executable, "-c", code], env=_env(), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def test_the_normal_build_says_so():
    from ozaki_blackwell_b200._lib import lib
    if os.environ.get("OZB_CHECK_BOUNDS"):
        pytest.skip("this is the checked build")
    out = (ctypes.c_ulonglong * 4)()
    assert lib.ozb_bounds_report(ctypes.byref(out)) == 10005 and lib.ozb_selftest_bounds() == 10005


def test_stage_odd_shape_and_panel_tests_under_the_checked_build():
    tests = ["tests/test_gpu_stages.py", "tests/test_gpu_panels.py", "tests/test_gpu_norm_scale.py",
             "tests/test_gpu_dgemm.py::test_odd_shapes_bit_exact", "tests/test_gpu_dgemm.py::test_long_k_is_cut_into_chunks_bit_exact",
             "tests/test_gpu_dgemm.py::test_zero_rows_columns_and_special_magnitudes", "tests/test_gpu_dgemm.py::test_host_operands_match_device_operands",
             "tests/test_gpu_api_surface.py::test_plan_interface_with_leading_dimensions_and_a_stream"]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] + tests, cwd=ROOT, env=_env(),
                       capture_output=True, text=True, timeout=1500)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "failed" not in r.stdout.splitlines()[-1], tail
