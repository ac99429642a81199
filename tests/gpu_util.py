"""Helpers for the GPU tests: device buffers through torch, calls through the C ABI (ctypes), checks against the oracle."""
import ctypes

import numpy as np
import torch

from ozaki_blackwell_b200._lib import lib


def check(code):
    assert code == 0, lib.ozb_error(code).decode()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def round_up(x, to):
    return (x + to - 1) // to * to


def synthetic(rows, cols, seed, spread=8):
    """The benchmark family: U[-1,1) * 2^e, e uniform integer in [-spread, spread] (spread 0: plain U[-1,1))."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, size=(rows, cols))
    if spread:
        x = np.ldexp(x, rng.integers(-spread, spread + 1, size=(rows, cols)).astype(np.int32))
    return x


def gpu_scale_residues_rows(X, nm, bits, ld=None, ldx=None):
    rows, length = X.shape
    ld = round_up(length, 16) if ld is None else ld
    Xd = dev(X) if ldx is None else None
    if ldx is not None:
        buf = torch.zeros((rows, ldx), dtype=torch.float64, device="cuda")
        buf[:, :length] = dev(X)
        Xd = buf
    s = torch.full((rows,), -12345, dtype=torch.int32, device="cuda")
    R = torch.full((nm, rows, ld), 77, dtype=torch.int8, device="cuda")
    check(lib.ozb_scale_residues_rows(nm, ptr(Xd), rows, length, Xd.stride(0), bits, ptr(s), ptr(R), ld, rows * ld, None))
    check(lib.ozb_status())
    return s.cpu().numpy(), R.cpu().numpy()


def gpu_scale_residues_cols(X, nm, bits, ld=None):
    rows, cols = X.shape   # rows = K
    ld = round_up(rows, 16) if ld is None else ld
    Xd = dev(X)
    s = torch.full((cols,), -12345, dtype=torch.int32, device="cuda")
    R = torch.full((nm, cols, ld), 77, dtype=torch.int8, device="cuda")
    cm = torch.zeros((cols,), dtype=torch.int64, device="cuda")
    check(lib.ozb_scale_residues_cols(nm, ptr(Xd), rows, cols, cols, bits, ptr(cm), ptr(s), ptr(R), ld, cols * ld, None))
    check(lib.ozb_status())
    return s.cpu().numpy(), R.cpu().numpy()


def gpu_gemm_i8(A, Bt):
    """A [Z][M][K] int8, Bt [Z][N][K] int8 (K padded to 16 here) -> int32 [Z][M][N]."""
    Z, M, K = A.shape
    N = Bt.shape[1]
    Kp = round_up(K, 16)
    Ad = torch.zeros((Z, M, Kp), dtype=torch.int8, device="cuda")
    Bd = torch.zeros((Z, N, Kp), dtype=torch.int8, device="cuda")
    Ad[:, :, :K] = dev(A)
    Bd[:, :, :K] = dev(Bt)
    C = torch.full((Z, M, N), 0x55555555, dtype=torch.int32, device="cuda")
    check(lib.ozb_gemm_i8(ptr(Ad), ptr(Bd), ptr(C), M, N, K, Z, Kp, Kp, N, M * Kp, N * Kp, M * N, None))
    check(lib.ozb_status())
    return C.cpu().numpy()


def gpu_gemm_i8_mod(A, Bt, first_modulus=0):
    Z, M, K = A.shape
    N = Bt.shape[1]
    Kp, Np = round_up(K, 16), round_up(N, 16)
    Ad = torch.zeros((Z, M, Kp), dtype=torch.int8, device="cuda")
    Bd = torch.zeros((Z, N, Kp), dtype=torch.int8, device="cuda")
    Ad[:, :, :K] = dev(A)
    Bd[:, :, :K] = dev(Bt)
    C = torch.full((Z, M, Np), 99, dtype=torch.int8, device="cuda")
    check(lib.ozb_gemm_i8_mod(ptr(Ad), ptr(Bd), ptr(C), M, N, K, Z, Kp, Kp, Np, M * Kp, N * Kp, M * Np, first_modulus, None))
    check(lib.ozb_status())
    return C.cpu().numpy()[:, :, :N]


def gpu_crt_i32(Cl, sa, sb):
    nm, M, N = Cl.shape
    Cd, sad, sbd = dev(Cl.astype(np.int32)), dev(sa.astype(np.int32)), dev(sb.astype(np.int32))
    C = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    check(lib.ozb_crt_i32(nm, ptr(Cd), M * N, M, N, N, ptr(sad), ptr(sbd), ptr(C), N, None))
    check(lib.ozb_status())
    return C.cpu().numpy()


def gpu_crt_i8(Cr, sa, sb):
    nm, M, N = Cr.shape
    Np = round_up(N, 16)
    Cd = torch.zeros((nm, M, Np), dtype=torch.int8, device="cuda")
    Cd[:, :, :N] = dev(Cr.astype(np.int8))
    sad, sbd = dev(sa.astype(np.int32)), dev(sb.astype(np.int32))
    C = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    check(lib.ozb_crt_i8(nm, ptr(Cd), M * Np, M, N, Np, ptr(sad), ptr(sbd), ptr(C), N, None))
    check(lib.ozb_status())
    return C.cpu().numpy()


def gpu_dgemm(A, B, nm=16, on_host=False):
    M, K = A.shape
    N = B.shape[1]
    if on_host:
        A = np.ascontiguousarray(A, dtype=np.float64)
        B = np.ascontiguousarray(B, dtype=np.float64)
        C = np.full((M, N), np.nan)
        check(lib.ozb_dgemm(M, N, K, A.ctypes.data, B.ctypes.data, C.ctypes.data, nm, 1))
        return C
    Ad, Bd = dev(A), dev(B)
    C = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    check(lib.ozb_dgemm(M, N, K, ptr(Ad), ptr(Bd), ptr(C), nm, 0))
    return C.cpu().numpy()


def same_bits(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint64), np.ascontiguousarray(b).view(np.uint64))


def describe_mismatch(got, want, limit=8):
    bad = np.argwhere(got != want)
    head = ", ".join(f"{tuple(int(v) for v in ix)}: got {got[tuple(ix)]} want {want[tuple(ix)]}" for ix in bad[:limit])
    return f"{len(bad)} of {got.size} differ; first: {head}"
