"""ctypes view of the CPU checker (oracle/liboz_oracle.so). Test infrastructure: imported only by tests, the smoke check
and the benchmark's CPU-baseline leg, never by the library."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_DIR = os.path.join(os.path.dirname(_HERE), "oracle")
_SO = os.path.join(ORACLE_DIR, "liboz_oracle.so")


def build():
    """(Re)build the checker with its Makefile; a no-op when it is up to date."""
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)


def _load():
    if not os.path.exists(_SO):
        build()
    lib = ctypes.CDLL(_SO)
    i, ll, d, p, sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t
    lib.oz_oracle_modulus.argtypes = [i]
    lib.oz_oracle_set_threads.argtypes = [i]
    lib.oz_oracle_inv_mod.argtypes = [i, i]
    lib.oz_oracle_bits_for.argtypes = [i, i, i]
    lib.oz_oracle_scales.argtypes = [p, i, i, ll, ll, i, p]
    lib.oz_oracle_scales.restype = None
    lib.oz_oracle_residues.argtypes = [p, i, i, ll, ll, p, i, p, i, sz]
    lib.oz_oracle_residues.restype = None
    lib.oz_oracle_gemm_i8.argtypes = [p, p, p, i, i, i, i, i, i]
    lib.oz_oracle_gemm_i8.restype = None
    lib.oz_oracle_crt.argtypes = [p, sz, i, i, i, p, p, i, p, i]
    lib.oz_oracle_crt.restype = None
    lib.oz_oracle_garner_digits.argtypes = [p, i, p]
    lib.oz_oracle_garner_digits.restype = None
    lib.oz_oracle_dgemm.argtypes = [i, i, i, p, p, p, i]
    lib.oz_oracle_err_units.argtypes = [i, i, i, p, p, p, i, i, i]
    lib.oz_oracle_err_units.restype = d
    lib.oz_oracle_err_units_sampled.argtypes = [i, i, i, p, p, p, p, i]
    lib.oz_oracle_err_units_sampled.restype = d
    lib.oz_oracle_fill_i8.argtypes = [i, i, i, p, p]
    lib.oz_oracle_fill_i8.restype = None
    lib.oz_ref_fill.argtypes = [p, sz, d, ctypes.c_uint]
    lib.oz_ref_fill.restype = None
    return lib


lib = _load()


def _ptr(a):
    return a.ctypes.data


def set_threads(n=0):
    """OpenMP threads of the checker (n = 0: only report). Needed under launchers that export OMP_NUM_THREADS=1."""
    return lib.oz_oracle_set_threads(n)


def modulus(l):
    return lib.oz_oracle_modulus(l)


def bits_for(nm, K, maxbits=62):
    return lib.oz_oracle_bits_for(nm, K, maxbits)


def scales(X, rows, length, s_row, s_col, bits):
    X = np.ascontiguousarray(X, dtype=np.float64)
    s = np.empty(rows, dtype=np.int32)
    lib.oz_oracle_scales(_ptr(X), rows, length, s_row, s_col, bits, _ptr(s))
    return s


def residues(X, rows, length, s_row, s_col, s, nm, ld=None):
    """int8 planes [nm][rows][ld] (zero beyond `length`)."""
    X = np.ascontiguousarray(X, dtype=np.float64)
    s = np.ascontiguousarray(s, dtype=np.int32)
    ld = length if ld is None else ld
    R = np.zeros((nm, rows, ld), dtype=np.int8)
    lib.oz_oracle_residues(_ptr(X), rows, length, s_row, s_col, _ptr(s), nm, _ptr(R), ld, rows * ld)
    return R


def gemm_i8(A, Bt):
    """A [M][K] int8, Bt [N][K] int8 -> int32 [M][N]."""
    A = np.ascontiguousarray(A, dtype=np.int8)
    Bt = np.ascontiguousarray(Bt, dtype=np.int8)
    M, K = A.shape
    N = Bt.shape[0]
    C = np.empty((M, N), dtype=np.int32)
    lib.oz_oracle_gemm_i8(_ptr(A), _ptr(Bt), _ptr(C), M, N, K, K, K, N)
    return C


def crt(Cl, sa, sb):
    """Cl int32 [nm][M][N] -> float64 [M][N]."""
    Cl = np.ascontiguousarray(Cl, dtype=np.int32)
    nm, M, N = Cl.shape
    sa = np.ascontiguousarray(sa, dtype=np.int32)
    sb = np.ascontiguousarray(sb, dtype=np.int32)
    C = np.empty((M, N), dtype=np.float64)
    lib.oz_oracle_crt(_ptr(Cl), M * N, M, N, N, _ptr(sa), _ptr(sb), nm, _ptr(C), N)
    return C


def garner_digits(res):
    res = np.ascontiguousarray(res, dtype=np.int32)
    x = np.empty(res.shape[0], dtype=np.int32)
    lib.oz_oracle_garner_digits(_ptr(res), res.shape[0], _ptr(x))
    return x


def dgemm(A, B, nm=16):
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), dtype=np.float64)
    rc = lib.oz_oracle_dgemm(M, N, K, _ptr(A), _ptr(B), _ptr(C), nm)
    if rc:
        raise RuntimeError(f"oracle dgemm failed: {rc}")
    return C


def err_units(A, B, C, which=0, rows0=0, rows=None):
    """max |C - ref| / (|A||B|) in units of 2^-53 (which: 0 Dot2 reference, 1 80-bit reference, 2 ref80 vs Dot2)."""
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    C = np.ascontiguousarray(C, dtype=np.float64)
    M, K = A.shape
    N = B.shape[1]
    rows = M - rows0 if rows is None else rows
    return lib.oz_oracle_err_units(M, N, K, _ptr(A), _ptr(B), _ptr(C), which, rows0, rows)


def err_units_sampled(A, B, C, idx):
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    C = np.ascontiguousarray(C, dtype=np.float64)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    M, K = A.shape
    N = B.shape[1]
    return lib.oz_oracle_err_units_sampled(M, N, K, _ptr(A), _ptr(B), _ptr(C), _ptr(idx), idx.size)


def fill_i8(M, N, K):
    A = np.empty((M, K), dtype=np.int8)
    Bt = np.empty((N, K), dtype=np.int8)
    lib.oz_oracle_fill_i8(M, N, K, _ptr(A), _ptr(Bt))
    return A, Bt


def ref_fill(n, spread, seed):
    v = np.empty(n, dtype=np.float64)
    lib.oz_ref_fill(_ptr(v), n, float(spread), seed)
    return v


# ---- double-double path (oracle/ozaki_dd_oracle.c) ----
_i, _ll, _d, _p, _sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t
lib.oz_oracle_residues_dd.argtypes = [_p, _p, _i, _i, _ll, _ll, _p, _i, _p, _i, _sz]
lib.oz_oracle_residues_dd.restype = None
lib.oz_oracle_crt_dd.argtypes = [_p, _sz, _i, _i, _i, _p, _p, _i, _p, _p, _i, _i]
lib.oz_oracle_crt_dd.restype = None
lib.oz_oracle_ddgemm.argtypes = [_i, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i]
lib.oz_oracle_ref_quad.argtypes = [_p, _p, _p, _p, _i, _i, _i, _p, _p, _p]
lib.oz_oracle_ref_quad.restype = None
lib.oz_oracle_dd_err_units.argtypes = [_p, _p, _p, _p, _p, _sz]
lib.oz_oracle_dd_err_units.restype = _d
lib.oz_oracle_dd_crt_kat.argtypes = [_p, _i, _i]
lib.oz_ref_fill_dd.argtypes = [_p, _p, _sz, _p, _p, _sz, _d, ctypes.c_uint]
lib.oz_ref_fill_dd.restype = None


def _c(a, dt=np.float64):
    return np.ascontiguousarray(a, dtype=dt)


def residues_dd(Xh, Xl, rows, length, s_row, s_col, s, nm, ld=None):
    Xh, Xl, s = _c(Xh), _c(Xl), _c(s, np.int32)
    ld = length if ld is None else ld
    R = np.zeros((nm, rows, ld), dtype=np.int8)
    lib.oz_oracle_residues_dd(_ptr(Xh), _ptr(Xl), rows, length, s_row, s_col, _ptr(s), nm, _ptr(R), ld, rows * ld)
    return R


def crt_dd(Cl, sa, sb, mode=0, Ch=None, Cl_=None):
    Cl = _c(Cl, np.int32)
    nm, M, N = Cl.shape
    sa, sb = _c(sa, np.int32), _c(sb, np.int32)
    Ch = np.zeros((M, N)) if Ch is None else _c(Ch).copy()
    Cl_ = np.zeros((M, N)) if Cl_ is None else _c(Cl_).copy()
    lib.oz_oracle_crt_dd(_ptr(Cl), M * N, M, N, N, _ptr(sa), _ptr(sb), nm, _ptr(Ch), _ptr(Cl_), N, mode)
    return Ch, Cl_


def ddgemm(Ah, Al, Bh, Bl, nm=32, mode=0, Ch=None, Cl=None):
    Ah, Al, Bh, Bl = _c(Ah), _c(Al), _c(Bh), _c(Bl)
    M, K = Ah.shape
    N = Bh.shape[1]
    Ch = np.zeros((M, N)) if Ch is None else _c(Ch).copy()
    Cl = np.zeros((M, N)) if Cl is None else _c(Cl).copy()
    rc = lib.oz_oracle_ddgemm(M, N, K, _ptr(Ah), _ptr(Al), _ptr(Bh), _ptr(Bl), _ptr(Ch), _ptr(Cl), nm, mode)
    if rc:
        raise RuntimeError(f"oracle ddgemm failed: {rc}")
    return Ch, Cl


def ref_quad(Ah, Al, Bh, Bl):
    Ah, Al, Bh, Bl = _c(Ah), _c(Al), _c(Bh), _c(Bl)
    M, K = Ah.shape
    N = Bh.shape[1]
    Rh, Rl, Ab = np.empty((M, N)), np.empty((M, N)), np.empty((M, N))
    lib.oz_oracle_ref_quad(_ptr(Ah), _ptr(Al), _ptr(Bh), _ptr(Bl), M, N, K, _ptr(Rh), _ptr(Rl), _ptr(Ab))
    return Rh, Rl, Ab


def dd_err_units(Ch, Cl, Rh, Rl, Ab):
    Ch, Cl, Rh, Rl, Ab = _c(Ch), _c(Cl), _c(Rh), _c(Rl), _c(Ab)
    return lib.oz_oracle_dd_err_units(_ptr(Ch), _ptr(Cl), _ptr(Rh), _ptr(Rl), _ptr(Ab), Ch.size)


def dd_crt_kat(V, nm=32):
    V = np.ascontiguousarray(V, dtype=np.uint32)
    return lib.oz_oracle_dd_crt_kat(_ptr(V), V.shape[0], nm)


def ref_fill_dd(M, N, K, spread):
    Ah, Al = np.empty(M * K), np.empty(M * K)
    Bh, Bl = np.empty(K * N), np.empty(K * N)
    lib.oz_ref_fill_dd(_ptr(Ah), _ptr(Al), M * K, _ptr(Bh), _ptr(Bl), K * N, float(spread), K + int(spread))
    return Ah.reshape(M, K), Al.reshape(M, K), Bh.reshape(K, N), Bl.reshape(K, N)


# ---- optional 2-norm scaling (bench/oz_strassen.cu:74-97 of the reference) ----
lib.oz_oracle_scales_norm.argtypes = [_p, _i, _i, _ll, _ll, _i, _p]
lib.oz_oracle_scales_norm.restype = None
lib.oz_oracle_bits_for_norm.argtypes = [_i]
lib.oz_oracle_dgemm_norm.argtypes = [_i, _i, _i, _p, _p, _p, _i]


def scales_norm(X, rows, length, s_row, s_col, beta):
    X = _c(X)
    s = np.empty(rows, dtype=np.int32)
    lib.oz_oracle_scales_norm(_ptr(X), rows, length, s_row, s_col, beta, _ptr(s))
    return s


def bits_for_norm(nm):
    return lib.oz_oracle_bits_for_norm(nm)


def dgemm_norm(A, B, nm=16):
    A, B = _c(A), _c(B)
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N))
    rc = lib.oz_oracle_dgemm_norm(M, N, K, _ptr(A), _ptr(B), _ptr(C), nm)
    if rc:
        raise RuntimeError(f"oracle dgemm_norm failed: {rc}")
    return C
