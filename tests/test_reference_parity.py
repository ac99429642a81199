"""This library, the CPU checker and the reference's own kernels side by side on the GPU (skipped where the reference
build oracle/_ref/libozb_ref.so is absent). The reference library is the reference's python/capi.cu compiled unmodified
for sm_100a by `make -C oracle ref`; it runs the reference's mma.sync kernels."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu
REF = os.path.join(o.ORACLE_DIR, "_ref", "libozb_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("reference build not present")
    lib = ctypes.CDLL(REF)
    lib.ozb_dgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2
    lib.ozb_error.restype = ctypes.c_char_p
    yield lib
    lib.ozb_release()


def _ref_dgemm(lib, A, B, nm):
    M, K = A.shape
    N = B.shape[1]
    C = np.full((M, N), np.nan)
    rc = lib.ozb_dgemm(M, N, K, A.ctypes.data, B.ctypes.data, C.ctypes.data, nm, 1)
    assert rc == 0, lib.ozb_error(rc)
    return C


@pytest.mark.parametrize("nm", [8, 11, 14, 16])
@pytest.mark.parametrize("shape", [(256, 256, 512), (200, 300, 500), (384, 512, 1024)])
def test_three_way_bit_parity(ref, shape, nm):
    import gpu_util as g
    M, N, K = shape
    A, B = g.synthetic(M, K, 40 + nm), g.synthetic(K, N, 41 + nm)
    theirs = _ref_dgemm(ref, A, B, nm)
    ours = g.gpu_dgemm(A, B, nm)
    assert g.same_bits(ours, theirs), g.describe_mismatch(ours, theirs)
    assert g.same_bits(o.dgemm(A, B, nm), theirs)


def test_bit_parity_at_n2048_and_reference_accuracy_inputs(ref):
    import gpu_util as g
    n = 2048
    A, B = g.synthetic(n, n, 50), g.synthetic(n, n, 51)
    assert g.same_bits(g.gpu_dgemm(A, B, 16), _ref_dgemm(ref, A, B, 16))
    K = 4096
    A = o.ref_fill(256 * K, 8, 1 + K).reshape(256, K)
    B = o.ref_fill(K * 256, 8, 2 + K).reshape(K, 256)
    theirs = _ref_dgemm(ref, A, B, 16)
    assert g.same_bits(g.gpu_dgemm(A, B, 16), theirs)
    assert abs(o.err_units(A, B, theirs) - 1.87) < 0.05          # README.md:52 of the reference
