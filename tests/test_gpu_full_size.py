"""The benchmark's full sizes (n = 8192 with 16 moduli; n = 4096 with 12, 14, 16), where the CPU checker cannot recompute
the whole product inside a test: properties that hold at any size, checked bit for bit on the device, plus a band of rows
against the checker.

  * scaling by powers of two: C(2^a A, 2^b B) = 2^(a+b) C(A, B) exactly (the row and column scales absorb the factors
    and the integers, residues, products and digits stay the same);
  * row and column permutations commute with the product (row scales are per row of A, column scales per column of B);
  * a block of rows of A alone gives the same rows of C (what the multi-GPU partition rests on);
  * a band of rows equals the checker's, and the sampled error stays within the target.
"""
import ctypes
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as o

pytestmark = pytest.mark.gpu


def _device_inputs(n, seed, spread=8):
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    x = torch.rand((n, n), generator=gen, dtype=torch.float64, device="cuda") * 2 - 1
    if spread:
        x = x * torch.exp2(torch.randint(-spread, spread + 1, (n, n), generator=gen, device="cuda").double())
    return x


def _product(A, B, nm):
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, K = A.shape
    N = B.shape[1]
    A, B = A.contiguous(), B.contiguous()
    C = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    g.check(lib.ozb_dgemm(M, N, K, g.ptr(A), g.ptr(B), g.ptr(C), nm, 0))
    return C


def _same(x, y):
    import torch
    return bool(torch.equal(x.view(torch.int64), y.view(torch.int64)))


@pytest.mark.parametrize("n,nm", [(8192, 16), (4096, 12), (4096, 14), (4096, 16)])
def test_full_size_properties(n, nm):
    import torch
    A, B = _device_inputs(n, 100 + nm), _device_inputs(n, 200 + nm)
    C = _product(A, B, nm)
    assert bool(torch.isfinite(C).all())
    # powers of two move into the scales
    C2 = _product(A * 2.0 ** 7, B * 2.0 ** -11, nm)
    assert _same(C2, C * 2.0 ** -4)
    # permutations of the rows of A and of the columns of B
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    pr, pc = torch.randperm(n, generator=gen, device="cuda"), torch.randperm(n, generator=gen, device="cuda")
    assert _same(_product(A[pr], B[:, pc], nm), C[pr][:, pc])
    # a block of rows alone (not aligned to any tile)
    lo, hi = n // 3 + 5, n // 3 + 5 + 777
    assert _same(_product(A[lo:hi], B, nm), C[lo:hi])
    # a band of rows against the checker, and the error on a sample
    rows = slice(n // 2 - 3, n // 2 + 5)
    Ah, Bh = A[rows].cpu().numpy(), B.cpu().numpy()
    want = o.dgemm(Ah, Bh, nm)
    got = C[rows].cpu().numpy()
    assert np.array_equal(got.view(np.uint64), want.view(np.uint64))
    if nm == 16:
        idx = np.random.default_rng(2).integers(0, got.size, 512)
        assert o.err_units_sampled(Ah, Bh, got, idx) <= 2.0     # the target at n = 8192, 16 moduli


def test_double_double_at_n4096():
    """Configuration 3: hi = U[-1,1) 2^e, lo = hi U[-1,1) 2^-53, n = 4096, 32 moduli. Powers of two move into the scales
    (hi and lo parts both), a block of rows alone gives the same rows, a band of rows equals the checker's, and a 64 x 64
    sample stays within the reference's published error against the quad-precision product."""
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    n = 4096
    Ah, Bh = _device_inputs(n, 301), _device_inputs(n, 302)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(303)
    Al = Ah * 2.0 ** -53 * (torch.rand((n, n), generator=gen, dtype=torch.float64, device="cuda") * 2 - 1)
    Bl = Bh * 2.0 ** -53 * (torch.rand((n, n), generator=gen, dtype=torch.float64, device="cuda") * 2 - 1)

    def dd(ah, al, bh, bl):
        m, k = ah.shape
        ch = torch.full((m, bh.shape[1]), float("nan"), dtype=torch.float64, device="cuda")
        cl = torch.full_like(ch, float("nan"))
        ops = [x.contiguous() for x in (ah, al, bh, bl)]
        torch.cuda.synchronize()
        g.check(lib.ozb_ddgemm(m, bh.shape[1], k, *[g.ptr(x) for x in ops], g.ptr(ch), g.ptr(cl), 0))
        return ch, cl

    Ch, Cl = dd(Ah, Al, Bh, Bl)
    assert bool(torch.isfinite(Ch).all()) and bool(torch.isfinite(Cl).all())
    Ch2, Cl2 = dd(Ah * 2.0 ** 5, Al * 2.0 ** 5, Bh * 2.0 ** -9, Bl * 2.0 ** -9)
    assert _same(Ch2, Ch * 2.0 ** -4) and _same(Cl2, Cl * 2.0 ** -4)
    lo, hi = 1234, 1234 + 333
    Ch3, Cl3 = dd(Ah[lo:hi], Al[lo:hi], Bh, Bl)
    assert _same(Ch3, Ch[lo:hi]) and _same(Cl3, Cl[lo:hi])
    rows = slice(2000, 2004)
    host = [x.cpu().numpy() for x in (Ah[rows], Al[rows], Bh, Bl)]
    Wh, Wl = o.ddgemm(*host, 32)
    assert np.array_equal(Ch[rows].cpu().numpy().view(np.uint64), Wh.view(np.uint64))
    assert np.array_equal(Cl[rows].cpu().numpy().view(np.uint64), Wl.view(np.uint64))
    # 64 x 64 sample against the quad-precision product (bench/dd_test.cu measures the same; it publishes 12.6 units of
    # 2^-106 at K = 1024 for this input family, and the error grows slowly with K)
    r, c = slice(512, 576), slice(3000, 3064)
    sub = [Ah[r].cpu().numpy(), Al[r].cpu().numpy(), Bh[:, c].cpu().numpy(), Bl[:, c].cpu().numpy()]
    err = o.dd_err_units(Ch[r, c].cpu().numpy(), Cl[r, c].cpu().numpy(), *o.ref_quad(*sub))
    assert err <= 64.0, err
