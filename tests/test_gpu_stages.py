"""Each CUDA stage against the CPU checker on the same inputs, bit for bit (GPU tests; all calls go through the C ABI)."""
import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu


def _gu():
    import gpu_util
    return gpu_util


# ---- INT8 GEMM: the reference's known-answer shapes (bench/gemm_i8_test.cu:35-36) and shapes off every tile boundary ----
KAT_SHAPES = [(128, 128, 64), (256, 384, 512), (512, 256, 1024)]
ODD_SHAPES = [(1, 1, 1), (5, 7, 3), (128, 256, 128), (129, 257, 130), (200, 300, 500), (127, 255, 127), (300, 40, 1000),
              (64, 512, 16), (384, 768, 96)]


@pytest.mark.parametrize("shape", KAT_SHAPES + ODD_SHAPES)
def test_gemm_i8_exact(shape):
    g = _gu()
    M, N, K = shape
    A, Bt = o.fill_i8(M, N, K)
    got = g.gpu_gemm_i8(A[None], Bt[None])[0]
    want = o.gemm_i8(A, Bt)
    assert np.array_equal(got, want), g.describe_mismatch(got, want)


def test_gemm_i8_exact_large_kat():
    """8192 x 8192 x 128, the reference's fourth known-answer case; checked with NumPy's integer product of a row sample
    plus a full check of the first tile rows."""
    g = _gu()
    M, N, K = 8192, 8192, 128
    A, Bt = o.fill_i8(M, N, K)
    got = g.gpu_gemm_i8(A[None], Bt[None])[0]
    rows = np.r_[0:256, np.random.default_rng(0).integers(256, M, 256)]
    want = A[rows].astype(np.int32) @ Bt.astype(np.int32).T
    assert np.array_equal(got[rows], want), g.describe_mismatch(got[rows], want)


def test_gemm_i8_extreme_values_and_planes():
    """All entries -128 (the largest magnitude products, K just under the int32 limit is too slow on the CPU side, so K =
    4096 here), and several planes in one launch with different data per plane."""
    g = _gu()
    M, N, K, Z = 130, 260, 4096, 3
    rng = np.random.default_rng(3)
    A = rng.integers(-128, 128, size=(Z, M, K), dtype=np.int8)
    Bt = rng.integers(-128, 128, size=(Z, N, K), dtype=np.int8)
    A[0] = -128
    Bt[0] = -128
    got = g.gpu_gemm_i8(A, Bt)
    for z in range(Z):
        want = o.gemm_i8(A[z], Bt[z])
        assert np.array_equal(got[z], want), (z, g.describe_mismatch(got[z], want))
    assert got[0, 0, 0] == 128 * 128 * K


def test_gemm_i8_fused_mod_matches_balanced_residue():
    g = _gu()
    Z, M, N, K = 16, 200, 300, 2048
    rng = np.random.default_rng(4)
    A = rng.integers(-128, 128, size=(Z, M, K), dtype=np.int8)
    Bt = rng.integers(-128, 128, size=(Z, N, K), dtype=np.int8)
    A[:, 0, :] = -128
    Bt[:, 0, :] = -128      # element (0,0): +K*2^14, the positive extreme
    Bt[:, 1, :] = 127       # element (0,1): the negative extreme
    got = g.gpu_gemm_i8_mod(A, Bt)
    for z in range(Z):
        m = o.modulus(z)
        raw = o.gemm_i8(A[z], Bt[z]).astype(np.int64)
        r = np.mod(raw, m)
        want = np.where(r >= (m + 1) // 2, r - m, r).astype(np.int8)
        assert np.array_equal(got[z], want), (z, m, g.describe_mismatch(got[z], want))


@pytest.mark.parametrize("busy", [None, 0, 1])
def test_gemm_i8_beside_other_kernels_same_residues(busy):
    """The persistent grid that leaves SMs to other kernels: with the decision on the host (busy None), and on the device
    with the word clear (every CTA pair works) or set (the pairs beyond the kept ones leave when they start). More tiles
    than resident pairs, so the pairs that stay take over what the leavers would have done."""
    import torch
    g = _gu()
    Z, M, N, K = 6, 1100, 2300, 384
    rng = np.random.default_rng(41)
    A = rng.integers(-128, 128, size=(Z, M, K), dtype=np.int8)
    Bt = rng.integers(-128, 128, size=(Z, N, K), dtype=np.int8)
    Kp, Np = g.round_up(K, 16), g.round_up(N, 16)
    Ad = torch.zeros((Z, M, Kp), dtype=torch.int8, device="cuda")
    Bd = torch.zeros((Z, N, Kp), dtype=torch.int8, device="cuda")
    Ad[:, :, :K] = g.dev(A)
    Bd[:, :, :K] = g.dev(Bt)
    word = None if busy is None else torch.tensor([busy], dtype=torch.int32, device="cuda")
    for reserve in (16, 64, 1000):      # 1000: more than the device has -- one pair is always kept
        C = torch.full((Z, M, Np), 99, dtype=torch.int8, device="cuda")
        g.check(g.lib.ozb_gemm_i8_mod_beside(g.ptr(Ad), g.ptr(Bd), g.ptr(C), M, N, K, Z, Kp, Kp, Np, M * Kp, N * Kp, M * Np, 3,
                                             reserve, None if word is None else g.ptr(word), None))
        g.check(g.lib.ozb_status())
        got = C.cpu().numpy()[:, :, :N]
        for z in range(Z):
            m = o.modulus(3 + z)
            r = np.mod(o.gemm_i8(A[z], Bt[z]).astype(np.int64), m)
            want = np.where(r >= (m + 1) // 2, r - m, r).astype(np.int8)
            assert np.array_equal(got[z], want), (busy, reserve, z, g.describe_mismatch(got[z], want))


def test_gemm_mutant_is_detected():
    """The comparison itself must notice a single flipped byte (the reference's mutation check, bench/oz_strassen.cu:299-308)."""
    g = _gu()
    A, Bt = o.fill_i8(128, 256, 128)
    want = o.gemm_i8(A, Bt)
    A2 = A.copy()
    A2[17, 5] ^= 1
    got = g.gpu_gemm_i8(A2[None], Bt[None])[0]
    assert not np.array_equal(got, want)
    assert np.array_equal(got[:17], want[:17]) and np.array_equal(got[18:], want[18:])


# ---- scales + residues ----
def _edge_matrix(rows, cols, seed):
    g = _gu()
    X = g.synthetic(rows, cols, seed, spread=8)
    X[1, :] = 0.0                       # all-zero row: scale 0, residues 0
    X[2, :] = 0.0
    X[2, cols // 2] = 5e-324            # only a subnormal: scale beyond the normal exponent range
    X[3, :] *= 2.0 ** 900               # huge entries: large negative scale
    X[3, 0] = 1.0e-300                  # ... next to one that underflows to zero after scaling
    X[4, :] = np.ldexp(X[4, :], -1060)  # a subnormal row
    X[5, 0] = -X[5, 0]
    X[6, :] = 1.0                       # exact powers of two (ilogb boundaries)
    X[7, :] = -0.5
    X[8, :] = np.nextafter(1.0, 0.0)    # just below a power of two
    return X


@pytest.mark.parametrize("nm", [8, 12, 13, 16])
@pytest.mark.parametrize("shape", [(16, 512), (40, 500), (33, 8192), (12, 9000), (20, 1), (10, 40000)])
def test_scale_residues_rows(shape, nm):
    g = _gu()
    rows, K = shape
    X = _edge_matrix(max(rows, 9), max(K, 2), seed=rows + K)[:rows, :K].copy()
    bits = o.bits_for(nm, K)
    s, R = g.gpu_scale_residues_rows(X, nm, bits)
    s_want = o.scales(X, rows, K, K, 1, bits)
    assert np.array_equal(s, s_want), g.describe_mismatch(s, s_want)
    R_want = o.residues(X, rows, K, K, 1, s_want, nm)
    assert np.array_equal(R[:, :, :K], R_want), g.describe_mismatch(R[:, :, :K], R_want)
    k4 = g.round_up(K, 4)
    assert np.all(R[:, :, K:k4] == 0)           # the tail of the last group of four is written as zeros


def test_scale_residues_rows_strided_unaligned():
    """Row pitch larger than the length and odd, so rows start on 8-byte but not 16-byte boundaries."""
    g = _gu()
    rows, K, nm = 9, 777, 16
    X = g.synthetic(rows, K, 11)
    bits = o.bits_for(nm, K)
    s, R = g.gpu_scale_residues_rows(X, nm, bits, ldx=K + 3)
    s_want = o.scales(X, rows, K, K, 1, bits)
    assert np.array_equal(s, s_want)
    assert np.array_equal(R[:, :, :K], o.residues(X, rows, K, K, 1, s_want, nm))


@pytest.mark.parametrize("nm", [8, 14, 16])
@pytest.mark.parametrize("shape", [(512, 16), (500, 40), (4096, 96), (300, 1), (1, 300), (1000, 515)])
def test_scale_residues_cols(shape, nm):
    g = _gu()
    K, cols = shape
    X = _edge_matrix(max(cols, 9), max(K, 2), seed=K + cols)[:cols, :K].T.copy()   # K x cols, edge cases per column
    bits = o.bits_for(nm, K)
    s, R = g.gpu_scale_residues_cols(X, nm, bits)
    s_want = o.scales(X, cols, K, 1, cols, bits)
    assert np.array_equal(s, s_want), g.describe_mismatch(s, s_want)
    R_want = o.residues(X, cols, K, 1, cols, s_want, nm)
    assert np.array_equal(R[:, :, :K], R_want), g.describe_mismatch(R[:, :, :K], R_want)
    assert np.all(R[:, :, K:g.round_up(K, 16)] == 0)


# ---- CRT ----
@pytest.mark.parametrize("nm", list(range(8, 17)))
def test_crt_from_int32_planes(nm):
    g = _gu()
    M, N, K = 70, 130, 256
    A = g.synthetic(M, K, 21)
    B = g.synthetic(K, N, 22)
    bits = o.bits_for(nm, K)
    sa, sb = o.scales(A, M, K, K, 1, bits), o.scales(B, N, K, 1, N, bits)
    Ar, Br = o.residues(A, M, K, K, 1, sa, nm), o.residues(B, N, K, 1, N, sb, nm)
    Cl = np.stack([o.gemm_i8(Ar[l], Br[l]) for l in range(nm)])
    want = o.crt(Cl, sa, sb)
    got = g.gpu_crt_i32(Cl, sa, sb)
    assert g.same_bits(got, want), g.describe_mismatch(got, want)
    # the int8 route: balanced residues first (what the fused GEMM epilogue stores)
    Cr = np.empty_like(Cl, dtype=np.int8)
    for l in range(nm):
        m = o.modulus(l)
        r = np.mod(Cl[l].astype(np.int64), m)
        Cr[l] = np.where(r >= (m + 1) // 2, r - m, r)
    got8 = g.gpu_crt_i8(Cr, sa, sb)
    assert g.same_bits(got8, want), g.describe_mismatch(got8, want)


def test_crt_random_residues_cover_all_digit_values():
    """Arbitrary residue vectors (not only those of small products): every digit range, including -128 for modulus 256."""
    g = _gu()
    nm, M, N = 16, 64, 257
    rng = np.random.default_rng(9)
    Cl = rng.integers(-2**31, 2**31, size=(nm, M, N), dtype=np.int64).astype(np.int32)
    sa = rng.integers(-30, 30, size=M).astype(np.int32)
    sb = rng.integers(-30, 30, size=N).astype(np.int32)
    want = o.crt(Cl, sa, sb)
    got = g.gpu_crt_i32(Cl, sa, sb)
    assert g.same_bits(got, want), g.describe_mismatch(got, want)


def test_crt_extreme_scales_subnormal_and_huge_results():
    g = _gu()
    nm, M, N = 16, 8, 64
    rng = np.random.default_rng(10)
    Cl = rng.integers(-2**20, 2**20, size=(nm, M, N), dtype=np.int64).astype(np.int32)
    sa = np.array([0, 500, 1000, 1100, -400, -900, 1150, 40], dtype=np.int32)
    sb = rng.integers(-60, 60, size=N).astype(np.int32)
    want = o.crt(Cl, sa, sb)
    got = g.gpu_crt_i32(Cl, sa, sb)
    assert g.same_bits(got, want), g.describe_mismatch(got, want)
