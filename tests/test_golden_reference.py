"""Outputs of the reference's own GPU code (tests/golden/reference_outputs.npz, made by tests/golden/make_golden.py from
the unmodified reference sources) against the CPU checker (no GPU needed) and against this library (GPU)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import cases  # noqa: E402
import oracle_lib as o  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "reference_outputs.npz")
needs_golden = pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden vectors not generated yet")


def _load(name):
    z = np.load(GOLDEN)
    A, B, nm = cases.inputs(name)
    assert str(z[name + ".inputs_sha256"]) == cases.digest(A, B), "the seeded inputs no longer match the stored digest"
    return A, B, nm, z[name + ".C"]


@needs_golden
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_checker_equals_reference_output(name):
    A, B, nm, want = _load(name)
    got = o.dgemm(A, B, nm).view(np.uint64)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} entries differ from the reference's output"


@needs_golden
@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_library_equals_reference_output(name):
    import gpu_util as g
    A, B, nm, want = _load(name)
    got = g.gpu_dgemm(A, B, nm).view(np.uint64)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} entries differ from the reference's output"


def _load_dd(name):
    z = np.load(GOLDEN)
    if name + ".Ch" not in z:
        pytest.skip("golden file predates the double-double cases")
    parts = cases.dd_inputs(name)
    assert str(z[name + ".inputs_sha256"]) == cases.digest(*parts)
    return parts, z[name + ".Ch"], z[name + ".Cl"]


@needs_golden
@pytest.mark.parametrize("name", sorted(cases.DD_CASES))
def test_dd_checker_equals_reference_output(name):
    (Ah, Al, Bh, Bl), wh, wl = _load_dd(name)
    Ch, Cl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    assert np.array_equal(Ch.view(np.uint64), wh) and np.array_equal(Cl.view(np.uint64), wl)


@needs_golden
@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.DD_CASES))
def test_dd_library_equals_reference_output(name):
    import test_gpu_dd
    (Ah, Al, Bh, Bl), wh, wl = _load_dd(name)
    Ch, Cl = test_gpu_dd._gpu_ddgemm(Ah, Al, Bh, Bl)
    assert np.array_equal(Ch.view(np.uint64), wh) and np.array_equal(Cl.view(np.uint64), wl)
