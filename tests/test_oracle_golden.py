"""The CPU checker against the reference's own known answers (no GPU needed).

The reference stores no binary fixtures: its accuracy test regenerates its inputs from seeds (bench/ozaki_test.cu:27-41)
and its README publishes the resulting error table (README.md:47-52 for 12/14/16 moduli at K = 512 and 4096, spreads 0
and 8; README.md:257-259 for spreads 16 and 32 at K = 4096). Reproducing those numbers from the same inputs pins the
checker's scaling, rounding, residues, Garner digits and FP64 Horner to the reference's.
"""
import numpy as np
import pytest

import oracle_lib as o

# (K, spread) -> {moduli: published max error in units of 2^-53 of |A||B|}, M = N = 256
PUBLISHED = {
    (512, 0): {12: 2660, 14: 10.9, 16: 0.99},
    (512, 8): {12: 94600, 14: 395, 16: 3.1},
    (4096, 0): {12: 2400, 14: 10.5, 16: 0.24},
    (4096, 8): {12: 42200, 14: 203, 16: 1.87},
    (4096, 16): {14: 800, 16: 4.7},
    (4096, 32): {14: 3680, 16: 31.5},
}
# bits_for as the reference prints it next to each column (bench/ozaki_test.cu:70) for these K
BITS = {(12, 512): 41, (14, 512): 49, (16, 512): 57, (12, 4096): 40, (14, 4096): 48, (16, 4096): 55,
        (16, 8192): 55, (16, 32768): 54}


def _inputs(K, spread, M=256, N=256):
    A = o.ref_fill(M * K, spread, 1 + K).reshape(M, K)
    B = o.ref_fill(K * N, spread, 2 + K).reshape(K, N)
    return A, B


@pytest.mark.parametrize("case", sorted(PUBLISHED))
def test_published_error_table(case):
    K, spread = case
    A, B = _inputs(K, spread)
    for nm, want in PUBLISHED[case].items():
        C = o.dgemm(A, B, nm)
        got = o.err_units(A, B, C, which=0)
        # the README rounds to two or three significant digits
        assert abs(got - want) <= 0.02 * want + 0.006, (case, nm, got, want)


def test_bits_for():
    for (nm, K), want in BITS.items():
        assert o.bits_for(nm, K) == want
    assert o.bits_for(16, 131072) == -1          # the reference aborts here; the C ABI reports an error instead
    assert o.bits_for(16, 512, 40) == 40         # the cap (the double-double path passes its own)


def test_moduli_pairwise_coprime_and_inverses():
    m = [o.modulus(l) for l in range(49)]
    assert m[:16] == [256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193]
    for a in range(49):
        for b in range(a + 1, 49):
            assert np.gcd(m[a], m[b]) == 1
            inv = o.lib.oz_oracle_inv_mod(m[a] % m[b], m[b])
            assert 0 < inv < m[b] and (m[a] * inv) % m[b] == 1


def test_int8_gemm_known_answer_small():
    """bench/gemm_i8_test.cu's three small shapes: the checker's GEMM against NumPy's int64 product."""
    for M, N, K in ((128, 128, 64), (256, 384, 512), (512, 256, 1024)):
        A, Bt = o.fill_i8(M, N, K)
        assert A.min() >= -127 and A.max() <= 127
        want = A.astype(np.int64) @ Bt.astype(np.int64).T
        assert np.array_equal(o.gemm_i8(A, Bt), want.astype(np.int32))


def test_garner_digits_reconstruct_the_integer():
    """Mixed-radix digits are balanced and sum_l x_l * prod_{t<l} m_t is the integer the residues came from."""
    rng = np.random.default_rng(5)
    m = [o.modulus(l) for l in range(16)]
    for nm in (8, 12, 16):
        P = 1
        for l in range(nm):
            P *= m[l]
        for _ in range(200):
            v = int(rng.integers(-2**62, 2**62)) * int(rng.integers(1, 2**40)) % P
            if v >= (P + 1) // 2:
                v -= P
            res = np.array([((v % mm) + mm) % mm for mm in m[:nm]], dtype=np.int32)
            x = o.garner_digits(res)
            acc, w = 0, 1
            for l in range(nm):
                assert -(m[l] // 2) <= x[l] < (m[l] + 1) // 2
                acc += int(x[l]) * w
                w *= m[l]
            assert acc == v


def test_non_tile_multiple_shape_and_zero_rows():
    """200 x 300 x 500 (bench/ozaki_test.cu:39) plus an all-zero row and column: scale 0, exact zeros out."""
    M, N, K = 200, 300, 500
    A, B = _inputs(K, 0, M, N)
    A[7, :] = 0
    B[:, 11] = 0
    C = o.dgemm(A, B, 16)
    assert np.all(C[7, :] == 0) and np.all(C[:, 11] == 0)
    keep = np.ones(N, bool); keep[11] = False
    Ak = np.delete(A, 7, axis=0); Bk = B[:, keep]
    Ck = np.ascontiguousarray(np.delete(C, 7, axis=0)[:, keep])
    assert o.err_units(Ak, Bk, Ck) < 2.0
