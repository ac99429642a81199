"""The double-double product on the GPU: ozb_ddgemm / ozb_ddgemm_ex bit for bit against the CPU checker, and against the
reference's own ozb_ddgemm where its build is present (GPU tests; all calls go through the C ABI)."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu
REF = os.path.join(o.ORACLE_DIR, "_ref", "libozb_ref.so")


def _dd_inputs(M, N, K, seed, spread=8):
    import gpu_util as g
    Ah, Bh = g.synthetic(M, K, seed, spread), g.synthetic(K, N, seed + 1, spread)
    rng = np.random.default_rng(seed + 2)
    Al = Ah * 2.0**-53 * rng.uniform(-1, 1, (M, K))      # lo = hi * U[-1,1) * 2^-53
    Bl = Bh * 2.0**-53 * rng.uniform(-1, 1, (K, N))
    return Ah, Al, Bh, Bl


def _gpu_ddgemm(Ah, Al, Bh, Bl, on_host=False):
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, K = Ah.shape
    N = Bh.shape[1]
    if on_host:
        arrs = [np.ascontiguousarray(x) for x in (Ah, Al, Bh, Bl)]
        Ch, Cl = np.full((M, N), np.nan), np.full((M, N), np.nan)
        g.check(lib.ozb_ddgemm(M, N, K, *[a.ctypes.data for a in arrs], Ch.ctypes.data, Cl.ctypes.data, 1))
        return Ch, Cl
    d = [g.dev(x) for x in (Ah, Al, Bh, Bl)]
    Ch = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    Cl = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    g.check(lib.ozb_ddgemm(M, N, K, *[g.ptr(x) for x in d], g.ptr(Ch), g.ptr(Cl), 0))
    return Ch.cpu().numpy(), Cl.cpu().numpy()


@pytest.mark.parametrize("shape", [(128, 128, 256), (64, 96, 1024), (200, 300, 500), (1, 1, 1), (3, 5, 7), (130, 260, 129), (257, 40, 2050)])
def test_ddgemm_bit_exact(shape):
    import gpu_util as g
    M, N, K = shape
    Ah, Al, Bh, Bl = _dd_inputs(M, N, K, 70)
    Ch, Cl = _gpu_ddgemm(Ah, Al, Bh, Bl)
    Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    assert g.same_bits(Ch, Wh), g.describe_mismatch(Ch, Wh)
    assert g.same_bits(Cl, Wl), g.describe_mismatch(Cl, Wl)


@pytest.mark.parametrize("case", [(256, 0, 0.71), (256, 8, 47.1), (1024, 0, 0.41), (1024, 8, 12.6)])
def test_reference_dd_accuracy_cases(case):
    """bench/dd_test.cu's inputs at 32 moduli: the checker's bits and the published error (README.md:433-435)."""
    import gpu_util as g
    K, spread, published = case
    Ah, Al, Bh, Bl = o.ref_fill_dd(128, 128, K, spread)
    Ch, Cl = _gpu_ddgemm(Ah, Al, Bh, Bl)
    Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    assert g.same_bits(Ch, Wh) and g.same_bits(Cl, Wl)
    err = o.dd_err_units(Ch, Cl, *o.ref_quad(Ah, Al, Bh, Bl))
    assert abs(err - published) <= 0.05 * published + 0.06, (err, published)


def test_dd_host_operands_special_rows_and_long_k():
    import gpu_util as g
    Ah, Al, Bh, Bl = _dd_inputs(70, 90, 12400, 73)          # K above 12288: the GEMMs run in two chunks
    Ah[2] = 0; Al[2] = 0
    Bh[:, 4] = 0; Bl[:, 4] = 0
    Ah[3] *= 2.0**500; Al[3] *= 2.0**500
    Bh[:, 5] *= 2.0**-600; Bl[:, 5] *= 2.0**-600
    Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    for on_host in (False, True):
        Ch, Cl = _gpu_ddgemm(Ah, Al, Bh, Bl, on_host)
        assert g.same_bits(Ch, Wh), g.describe_mismatch(Ch, Wh)
        assert g.same_bits(Cl, Wl), g.describe_mismatch(Cl, Wl)
    assert np.all(Wh[2] == 0) and np.all(Wh[:, 4] == 0)


@pytest.mark.parametrize("nm", [24, 28, 32])
def test_ddgemm_ex_modes_strides_and_modulus_counts(nm):
    """Leading dimensions larger than the matrices, and the reference's modes: 1 updates C in place, 2 negates."""
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, N, K = 150, 140, 333
    Ah, Al, Bh, Bl = _dd_inputs(M, N, K, 75)
    lda, ldb, ldo = K + 5, N + 3, N + 8

    def padded(x, ld):
        t = torch.zeros((x.shape[0], ld), dtype=torch.float64, device="cuda")
        t[:, :x.shape[1]] = g.dev(x)
        return t
    dAh, dAl, dBh, dBl = padded(Ah, lda), padded(Al, lda), padded(Bh, ldb), padded(Bl, ldb)
    C0h, C0l = g.synthetic(M, N, 77), np.zeros((M, N))
    for mode in (0, 2, 1):
        Ch, Cl = padded(C0h, ldo), padded(C0l, ldo)
        g.check(lib.ozb_ddgemm_ex(M, N, K, g.ptr(dAh), g.ptr(dAl), lda, g.ptr(dBh), g.ptr(dBl), ldb, g.ptr(Ch), g.ptr(Cl), ldo, nm, mode, None))
        torch.cuda.synchronize()
        Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, nm, mode=mode, Ch=C0h, Cl=C0l)
        assert g.same_bits(Ch[:, :N].cpu().numpy(), Wh) and g.same_bits(Cl[:, :N].cpu().numpy(), Wl), (nm, mode)
        assert torch.all(Ch[:, N:] == 0)                 # nothing written beyond the N columns


def test_dd_three_way_with_the_reference_build():
    import gpu_util as g
    if not os.path.exists(REF):
        pytest.skip("reference build not present")
    ref = ctypes.CDLL(REF)
    ref.ozb_ddgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 6 + [ctypes.c_int]
    for shape in ((128, 128, 256), (200, 300, 500), (384, 256, 1024)):
        M, N, K = shape
        Ah, Al, Bh, Bl = _dd_inputs(M, N, K, 79)
        Th, Tl = np.full((M, N), np.nan), np.full((M, N), np.nan)
        arrs = [np.ascontiguousarray(x) for x in (Ah, Al, Bh, Bl)]
        assert ref.ozb_ddgemm(M, N, K, *[a.ctypes.data for a in arrs], Th.ctypes.data, Tl.ctypes.data, 1) == 0
        Ch, Cl = _gpu_ddgemm(Ah, Al, Bh, Bl)
        assert g.same_bits(Ch, Th), g.describe_mismatch(Ch, Th)
        assert g.same_bits(Cl, Tl), g.describe_mismatch(Cl, Tl)
        Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, 32)
        assert g.same_bits(Wh, Th) and g.same_bits(Wl, Tl)
    ref.ozb_release()


def test_python_wrapper_matmul_dd():
    import ozaki_blackwell_b200 as ob
    import gpu_util as g
    Ah, Al, Bh, Bl = _dd_inputs(40, 30, 64, 81)
    Ch, Cl = ob.matmul_dd((Ah, Al), (Bh, Bl))
    Wh, Wl = o.ddgemm(Ah, Al, Bh, Bl, 32)
    assert g.same_bits(Ch, Wh) and g.same_bits(Cl, Wl)
    ms, tf = ob.bench(512, "dd", reps=2)
    assert ms > 0 and tf > 0
