"""Size-independent properties of the Ozaki-II product, on the CPU checker at a small size (the GPU tests use the same
properties at the benchmark's full sizes, where the checker cannot recompute the whole product): powers of two move into
the scales, permutations of rows of A / columns of B commute with the product, a block of rows alone gives the same rows."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import oracle_lib as o


def _bits(x):
    return np.ascontiguousarray(x).view(np.uint64)


@pytest.mark.parametrize("nm", [12, 16])
def test_properties_hold_for_the_checker(nm):
    rng = np.random.default_rng(nm)
    M, N, K = 40, 56, 200
    A = np.ldexp(rng.uniform(-1, 1, (M, K)), rng.integers(-8, 9, (M, K)).astype(np.int32))
    B = np.ldexp(rng.uniform(-1, 1, (K, N)), rng.integers(-8, 9, (K, N)).astype(np.int32))
    C = o.dgemm(A, B, nm)
    assert np.array_equal(_bits(o.dgemm(A * 2.0 ** 7, B * 2.0 ** -11, nm)), _bits(C * 2.0 ** -4))
    pr, pc = rng.permutation(M), rng.permutation(N)
    assert np.array_equal(_bits(o.dgemm(A[pr], B[:, pc], nm)), _bits(C[pr][:, pc]))
    assert np.array_equal(_bits(o.dgemm(A[7:29], B, nm)), _bits(C[7:29]))
