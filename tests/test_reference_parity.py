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


def test_norm_scales_against_the_reference_kernel():
    """The optional 2-norm scaling: the reference's own scales_norm kernel (bench/oz_strassen.cu:78-97, launched as the
    reference launches it, one block of 256 threads per contiguous row) against the CPU checker's restatement, scale by
    scale, and through it against this library's product (whose scales the checker reproduces bit for bit)."""
    path = os.path.join(o.ORACLE_DIR, "_ref", "libscales_norm_ref.so")
    if not os.path.exists(path):
        pytest.skip("reference build not present")
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib as ours
    lib = ctypes.CDLL(path)
    lib.ozref_scales_norm.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    rng = np.random.default_rng(7)
    for rows, length, nm in [(300, 500, 16), (64, 4096, 14), (33, 8192, 16), (17, 1, 8), (5, 70000, 12)]:
        X = g.synthetic(rows, length, 400 + rows)
        X[1, :] = 0.0                                        # a zero row
        X[2, :] *= 2.0 ** 500                                # huge entries: the squares are taken after scaling by 2^-e
        X[3, :] = np.ldexp(X[3, :], -1040)                   # a subnormal row
        X[4, :] = rng.standard_normal(length)                # norm well above the largest entry: where the two scalings differ
        beta = o.bits_for_norm(nm)
        Xd = g.dev(X)
        s = torch.full((rows,), -999, dtype=torch.int32, device="cuda")
        assert lib.ozref_scales_norm(g.ptr(Xd), rows, length, beta, g.ptr(s)) == 0
        want = o.scales_norm(X, rows, length, length, 1, beta)
        assert np.array_equal(s.cpu().numpy(), want), (rows, length, np.flatnonzero(s.cpu().numpy() != want)[:8])
        mine = torch.full((rows,), -999, dtype=torch.int32, device="cuda")     # this library's kernel on the same rows
        g.check(ours.ozb_scales_norm(g.ptr(Xd), rows, length, length, 1, nm, g.ptr(mine), None))
        assert torch.equal(mine, s), (rows, length)
    # the same rows as columns of a row-major matrix (how this library reads B): the checker's strided form agrees with
    # the reference kernel on the transposed copy (the reference transposes B first, bench/oz_strassen.cu:258)
    X = g.synthetic(130, 2049, 77)
    beta = o.bits_for_norm(16)
    Xd = g.dev(X)
    s = torch.empty(130, dtype=torch.int32, device="cuda")
    assert lib.ozref_scales_norm(g.ptr(Xd), 130, 2049, beta, g.ptr(s)) == 0
    Xt = np.ascontiguousarray(X.T)                           # 2049 x 130: the rows of X are its columns
    assert np.array_equal(s.cpu().numpy(), o.scales_norm(Xt, 130, 2049, 1, 130, beta))
    mine = torch.empty(130, dtype=torch.int32, device="cuda")
    g.check(ours.ozb_scales_norm(g.ptr(g.dev(Xt)), 130, 2049, 130, 0, 16, g.ptr(mine), None))   # by columns, as B is read
    assert torch.equal(mine, s)
