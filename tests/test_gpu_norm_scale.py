"""The optional 2-norm scaling (ozb_dgemm_norm; the reference's scales_norm, bench/oz_strassen.cu:74-97) on the GPU against
the CPU checker, which sums in the reference's order (GPU tests)."""
import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu


def _run(A, B, nm):
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, K = A.shape
    N = B.shape[1]
    Ad, Bd = g.dev(A), g.dev(B)
    C = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    g.check(lib.ozb_dgemm_norm(M, N, K, g.ptr(Ad), K, g.ptr(Bd), N, g.ptr(C), N, nm, None))
    torch.cuda.synchronize()
    g.check(lib.ozb_status())
    return C.cpu().numpy()


@pytest.mark.parametrize("nm", [8, 14, 16])
@pytest.mark.parametrize("shape", [(256, 256, 512), (200, 300, 500), (64, 130, 4096), (3, 5, 7)])
def test_norm_scaled_product_bit_exact(shape, nm):
    import gpu_util as g
    M, N, K = shape
    A, B = g.synthetic(M, K, 90), g.synthetic(K, N, 91)
    A[1 % M, :] = 0                       # a zero row: scale 0, zeros out
    got = _run(A, B, nm)
    want = o.dgemm_norm(A, B, nm)
    assert g.same_bits(got, want), g.describe_mismatch(got, want)


def test_norm_scale_keeps_more_bits_at_large_k():
    """The reference's claim (README.md:160-162): at large K the 2-norm scale buys about a modulus; here 14 moduli, K = 4096."""
    A = o.ref_fill(256 * 4096, 0, 1 + 4096).reshape(256, 4096)
    B = o.ref_fill(4096 * 256, 0, 2 + 4096).reshape(4096, 256)
    e_norm = o.err_units(A, B, _run(A, B, 14))
    e_max = o.err_units(A, B, o.dgemm(A, B, 14))
    assert e_norm < 0.5 * e_max and e_norm < 4.0
