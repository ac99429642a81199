"""The CPU checker of the double-double product against the reference's known answers (no GPU needed).

bench/dd_test.cu regenerates its inputs from seeds (:25-34) and README.md publishes the errors: the table at :204-209 for
24, 28 and 32 moduli (measured there against the __float128 sum of bench/ref_quad.cpp) and, at :433-435, the 32-moduli
column again against an exact 600-bit sum: 0.71 / 47.1 / 0.41 / 12.6 units of 2^-106. The checker is measured here against
a restatement of ref_quad.cpp (bit-identical to the reference's own compiled ref_quad where that library is present), whose
own error is a few hundredths of a unit, so the 32-moduli column is compared with the exact-reference values.
bench/crt_check.cpp is the reference's known-answer test of the direct-sum CRT tables.
"""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as o

PUBLISHED = {   # (K, spread) -> {moduli: error in units of 2^-106}, M = N = 128
    (256, 0): {24: 6.2e5, 28: 27.1, 32: 0.71},
    (256, 8): {24: 2.0e7, 28: 1160, 32: 47.1},
    (1024, 0): {24: 4.7e5, 28: 31, 32: 0.41},
    (1024, 8): {24: 1.1e7, 28: 713, 32: 12.6},
}


@pytest.mark.parametrize("case", sorted(PUBLISHED))
def test_published_dd_error_table(case):
    K, spread = case
    Ah, Al, Bh, Bl = o.ref_fill_dd(128, 128, K, spread)
    Rh, Rl, Ab = o.ref_quad(Ah, Al, Bh, Bl)
    for nm, want in PUBLISHED[case].items():
        Ch, Cl = o.ddgemm(Ah, Al, Bh, Bl, nm)
        got = o.dd_err_units(Ch, Cl, Rh, Rl, Ab)
        tol = 0.05 * want + (0.06 if nm == 32 else 0.0)   # two printed digits; the quad reference itself is off by ~0.03
        assert abs(got - want) <= tol, (case, nm, got, want)


def test_quad_reference_matches_the_reference_build():
    """Where the reference's own ref_quad.cpp has been compiled (oracle/_ref), the restatement returns the same bits."""
    so = os.path.join(o.ORACLE_DIR, "_ref", "libref_quad.so")
    if not os.path.exists(so):
        pytest.skip("reference build not present")
    f = ctypes.CDLL(so)._Z8ref_quadPKdS0_S0_S0_iiiPdS1_S1_
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3
    f.restype = None
    Ah, Al, Bh, Bl = o.ref_fill_dd(40, 50, 300, 8)
    mine = o.ref_quad(Ah, Al, Bh, Bl)
    theirs = [np.empty((40, 50)) for _ in range(3)]
    f(Ah.ctypes.data, Al.ctypes.data, Bh.ctypes.data, Bl.ctypes.data, 40, 50, 300, *[t.ctypes.data for t in theirs])
    for a, b in zip(mine, theirs):
        assert np.array_equal(a.view(np.uint64), b.view(np.uint64))


def test_direct_sum_crt_known_answers():
    """bench/crt_check.cpp: signed integers of 1..6 limbs come back exactly ("0 of 100000 wrong")."""
    rng = np.random.default_rng(3)
    n = 20000
    V = np.zeros((n, 8), dtype=np.uint32)
    for i in range(n):
        nl = 1 + int(rng.integers(0, 6))
        V[i, :nl] = rng.integers(0, 2**32, nl, dtype=np.uint64).astype(np.uint32)
        if rng.integers(0, 2):
            x = (-int.from_bytes(V[i].tobytes(), "little")) % (1 << 256)
            V[i] = np.frombuffer(x.to_bytes(32, "little"), dtype=np.uint32)
    assert o.dd_crt_kat(V, 32) == 0


def test_dd_modes_and_zero_handling():
    """mode 1 subtracts from C, mode 2 negates; an all-zero row gives exact zeros (src/ozaki_dd.cuh:94-95,121)."""
    rng = np.random.default_rng(4)
    M, N, K = 9, 11, 40
    Ah = rng.normal(size=(M, K)); Al = Ah * 2.0**-55 * rng.uniform(-1, 1, (M, K))
    Bh = rng.normal(size=(K, N)); Bl = Bh * 2.0**-55 * rng.uniform(-1, 1, (K, N))
    Ah[3] = 0; Al[3] = 0
    Ch, Cl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    assert np.all(Ch[3] == 0) and np.all(Cl[3] == 0)
    Nh, Nl = o.ddgemm(Ah, Al, Bh, Bl, 32, mode=2)
    assert np.array_equal(Nh, -Ch) and np.array_equal(Nl, -Cl)
    Sh, Sl = o.ddgemm(Ah, Al, Bh, Bl, 32, mode=1, Ch=Ch, Cl=Cl)     # C - AB with C = AB: zero to double-double accuracy
    assert np.all(np.abs(Sh) <= np.abs(Ch) * 2.0**-100 + 1e-300)
    assert np.allclose(Ch, Ah @ Bh, rtol=1e-12)
