"""Column windows of the product planes: the fused GEMM epilogue writing into a window of wider planes, the split
interface (ozb_plan_set_a + ozb_plan_panel) with panels given in order, and the internal multi-panel path of a plan
(environment variable OZ_PANELS), all against the CPU checker bit for bit (GPU tests, through the C ABI)."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu


def _balanced(raw, m):
    r = np.mod(raw.astype(np.int64), m)
    return np.where(r >= (m + 1) // 2, r - m, r).astype(np.int8)


@pytest.mark.parametrize("tail", [1, 14, 16, 17, 31, 32])
@pytest.mark.parametrize("M", [130, 300])
def test_fused_epilogue_touches_nothing_outside_its_window(tail, M):
    """C points at column 256 of planes that are exactly as wide as the window needs (256 + N rounded up to 16), so a
    piece written past the window would land in the next row (or, for the last row of the last plane, in the guard
    block after the buffer). Everything outside [0, round_up(N, 16)) of every row must keep its sentinel."""
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    Z, K, j0 = 3, 200, 256
    N = 32 + tail
    W = j0 + g.round_up(N, 16)
    rng = np.random.default_rng(100 + tail)
    A = rng.integers(-128, 128, size=(Z, M, K), dtype=np.int8)
    Bt = rng.integers(-128, 128, size=(Z, N, K), dtype=np.int8)
    Kp = g.round_up(K, 16)
    Ad = torch.zeros((Z, M, Kp), dtype=torch.int8, device="cuda"); Ad[:, :, :K] = g.dev(A)
    Bd = torch.zeros((Z, N, Kp), dtype=torch.int8, device="cuda"); Bd[:, :, :K] = g.dev(Bt)
    guard = 4096
    flat = torch.full((Z * M * W + guard,), 99, dtype=torch.int8, device="cuda")
    Cw = flat[:Z * M * W].view(Z, M, W)
    first = 2                                                 # planes reduce mod moduli 2, 3, 4 of the table
    cptr = ctypes.c_void_p(flat.data_ptr() + j0)
    g.check(lib.ozb_gemm_i8_mod(g.ptr(Ad), g.ptr(Bd), cptr, M, N, K, Z, Kp, Kp, W, M * Kp, N * Kp, M * W, first, None))
    g.check(lib.ozb_status())
    got = Cw.cpu().numpy()
    for z in range(Z):
        want = _balanced(o.gemm_i8(A[z], Bt[z]), o.modulus(first + z))
        assert np.array_equal(got[z, :, j0:j0 + N], want), (z, g.describe_mismatch(got[z, :, j0:j0 + N], want))
    assert np.all(got[:, :, :j0] == 99), "bytes before the window were written"
    assert np.all(got[:, :, j0 + g.round_up(N, 16):] == 99), "bytes after the window were written"
    assert np.all(flat[Z * M * W:].cpu().numpy() == 99), "bytes after the planes were written"


@pytest.mark.parametrize("shape", [(150, 270, 333, 15), (350, 1000, 520, 16)])
def test_panels_in_order_through_the_split_interface(shape):
    """ozb_plan_set_a, then the column panels left to right (the order a broadcast delivers them in). With N % 32 in
    1..16 the last panel's last piece used to reach into the first columns of the next row, which panel 0 had already
    produced."""
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, N, K, nm = shape
    A, B = g.synthetic(M, K, 201), g.synthetic(K, N, 202)
    Ad, Bd = g.dev(A), g.dev(B)
    Cd = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    plan = ctypes.c_void_p()
    g.check(lib.ozb_plan_create(M, N, K, nm, 62, ctypes.byref(plan)))
    want = o.dgemm(A, B, nm)
    for width in (256, 512):
        Cd.fill_(float("nan"))
        g.check(lib.ozb_plan_set_a(plan, g.ptr(Ad), K, None))
        for j0 in range(0, N, width):
            n = min(width, N - j0)
            g.check(lib.ozb_plan_panel(plan, ctypes.c_void_p(Bd.data_ptr() + 8 * j0), N, ctypes.c_void_p(Cd.data_ptr() + 8 * j0), N, j0, n, None))
        g.check(lib.ozb_plan_status(plan))
        got = Cd.cpu().numpy()
        assert g.same_bits(got, want), (width, g.describe_mismatch(got, want))
    lib.ozb_plan_destroy(plan)


@pytest.mark.parametrize("panels", [2, 4])
@pytest.mark.parametrize("shape", [(150, 270, 333), (350, 1000, 520), (200, 2049, 260)])
def test_internal_panels_overlapping_on_three_streams(shape, panels):
    """OZ_PANELS > 1 (read when a plan is made): B's residues, the GEMMs and the reconstruction of different column
    panels run on three streams. Same bits as one panel, repeated so that a product meets the previous one's tail."""
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, N, K = shape
    nm = 16
    A, B = g.synthetic(M, K, 211), g.synthetic(K, N, 212)
    Ad, Bd = g.dev(A), g.dev(B)
    Cd = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    plan = ctypes.c_void_p()
    old = os.environ.get("OZ_PANELS")
    os.environ["OZ_PANELS"] = str(panels)
    try:
        g.check(lib.ozb_plan_create(M, N, K, nm, 62, ctypes.byref(plan)))
    finally:
        if old is None:
            del os.environ["OZ_PANELS"]
        else:
            os.environ["OZ_PANELS"] = old
    g.check(lib.ozb_plan_profile(plan, 3))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            g.check(lib.ozb_plan_dgemm(plan, g.ptr(Ad), K, g.ptr(Bd), N, g.ptr(Cd), N, ctypes.c_void_p(stream.cuda_stream)))
    g.check(lib.ozb_plan_status(plan))
    got = Cd.cpu().numpy()
    want = o.dgemm(A, B, nm)
    assert g.same_bits(got, want), g.describe_mismatch(got, want)
    ms = (ctypes.c_float * 4)()
    for slot in range(3):
        g.check(lib.ozb_plan_phase_ms(plan, slot, ctypes.byref(ms)))
        assert 0 < ms[1] <= ms[3] * 1.01 + 0.01         # the panels' GEMMs follow one another on the caller's stream
    lib.ozb_plan_destroy(plan)
