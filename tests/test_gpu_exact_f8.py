"""The correctly rounded BF16 x block-scaled FP8 product on the GPU (ozb_bf16_fp8_gemm) against the exact CPU checker:
every compared output must have the checker's bits (GPU tests)."""
import ctypes
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import exact_f8_oracle as x  # noqa: E402

pytestmark = pytest.mark.gpu


def _run(X, W, S):
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, K = X.shape
    N = W.shape[1]
    Xd = torch.from_numpy(X.view(np.int16)).cuda()
    Wd, Sd = torch.from_numpy(W).cuda(), torch.from_numpy(S).cuda()
    Y = torch.full((M, N), 12345.0, dtype=torch.float32, device="cuda")
    opn, nm = ctypes.c_int(-1), ctypes.c_int(-1)
    rc = lib.ozb_bf16_fp8_gemm(M, N, K, g.ptr(Xd), g.ptr(Wd), g.ptr(Sd), g.ptr(Y), ctypes.byref(opn), ctypes.byref(nm), None)
    return rc, Y.cpu().numpy(), opn.value, nm.value


def _same(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


@pytest.mark.parametrize("shape", [(16, 24, 256), (33, 130, 300), (5, 7, 128), (1, 1, 1), (130, 260, 129), (64, 96, 1024)])
def test_every_output_is_the_rounded_exact_sum(shape):
    M, N, K = shape
    X, W, S = x.synthetic(M, N, K, 11 + M)
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0 and opn == 0 and 8 <= nm <= 19
    want = x.product(X, W, S)
    assert _same(Y, want), f"{(Y.view(np.uint32) != want.view(np.uint32)).sum()} of {Y.size} outputs differ"


def test_config4_family_sampled():
    """K = 7168 as in the benchmark configuration, a slice of its M and N; a sample of outputs against the exact sums."""
    M, N, K = 256, 640, 7168
    X, W, S = x.synthetic(M, N, K, 3)
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0 and opn == 0
    rng = np.random.default_rng(0)
    entries = [(int(i), int(j)) for i, j in zip(rng.integers(0, M, 200), rng.integers(0, N, 200))]
    want = x.product(X, W, S, entries)
    got = np.array([Y[i, j] for i, j in entries], dtype=np.float32)
    assert _same(got, want)


@pytest.mark.parametrize("name", ["normal_k256", "normal_k7168", "wide_k384", "tiny_k128"])
def test_kernel_reproduces_the_reference_superaccumulator(name):
    """The stored outputs of the reference's own exact_dot (llm/ultra.cu:336-369 of the reference; BF16-valued scales, which
    both definitions share): the kernel must return the same bits."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import f8_cases
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "exact_f8_reference.npz"))
    X, W, S = f8_cases.inputs(name)
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0
    nan = np.isnan(Y)
    assert opn == int(nan.sum())
    want = golden[name].view(np.float32)
    assert _same(Y[~nan], want[~nan])
    if name != "wide_k384":                       # 60 binades inside one row exceed the window: some outputs may stay open there
        assert opn == 0


def test_config4_full_size_sampled():
    """BASELINE's rectangular configuration at its stated size: 2048 x 7168 times 7168 x 18432 with one FP32 scale per
    128 x 128 block. Nothing may be left open, and a few hundred sampled outputs must be the exactly rounded sums."""
    M, N, K = 2048, 18432, 7168
    X, W, S = x.synthetic(M, N, K, 4)
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0 and opn == 0 and 8 <= nm <= 19
    assert not np.isnan(Y).any()
    rng = np.random.default_rng(1)
    entries = [(int(i), int(j)) for i, j in zip(rng.integers(0, M, 300), rng.integers(0, N, 300))]
    entries += [(0, 0), (M - 1, N - 1), (0, N - 1), (M - 1, 0)]
    want = x.product(X, W, S, entries)
    got = np.array([Y[i, j] for i, j in entries], dtype=np.float32)
    assert _same(got, want), f"{(got.view(np.uint32) != want.view(np.uint32)).sum()} of {len(entries)} sampled outputs differ"


def test_signs_zeros_subnormals_and_wide_scales():
    M, N, K = 12, 260, 384
    X, W, S = x.synthetic(M, N, K, 5)
    X[1, :] = 0                                  # zero row
    X[2, :] = 0x0001                             # smallest bf16 subnormal everywhere
    X[3, ::2] = 0x8000                           # negative zeros
    X[4, :] = x.to_bf16_bits(np.full(K, 3.0e38, dtype=np.float32))   # near the top of the range: FP32 overflow in the sum
    W[:, 5] = 0
    S[0, 0] = -S[0, 0]                           # a negative scale
    S[1, 1] = 0.0                                # a zero scale
    S[2, 0] = np.float32(2.0**-18)               # 18 binades below the largest scale: still inside the 44-bit scale window
    S[0, 2] = np.float32(1e-41)                  # a subnormal scale, 130 binades below its column block's other scales:
                                                 # beyond the 44-bit scale window, so that block's multiplier is truncated
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0
    want = x.product(X, W, S)
    nan = np.isnan(Y)
    assert opn == int(nan.sum()) and not nan[:, :256].any()      # only the third column block may be left open
    assert not nan[1].any()                                      # ... and never against an all-zero row
    assert _same(Y[~nan], want[~nan])
    assert np.all(Y[1] == 0) and np.all(np.isinf(Y[4, :5]) | (np.abs(Y[4, :5]) > 1e30))


def test_truncated_operands_are_certified_or_reported():
    """A row whose exponents span more than the 62-bit window: entries below it are truncated. Outputs the bound cannot
    decide come back as NaN and are counted; every other output must still be the exactly rounded sum."""
    M, N, K = 8, 128, 256
    X, W, S = x.synthetic(M, N, K, 7)
    big = x.to_bf16_bits(np.array([2.0**60], dtype=np.float32))[0]
    tiny = x.to_bf16_bits(np.array([2.0**-40], dtype=np.float32))[0]
    X[0, :] = tiny
    X[0, 0] = big                                 # 100 binades apart
    X[1, :] = tiny
    X[1, 3] = big
    W[0, :] = 0x38                                # 1.0: the big entry contributes 2^60 * scale exactly
    rc, Y, opn, nm = _run(X, W, S)
    assert rc == 0
    want = x.product(X, W, S)
    nan = np.isnan(Y)
    assert opn == int(nan.sum())
    assert _same(Y[~nan], want[~nan])
    assert not nan[2:].any()                      # rows without truncation are never left open


def test_non_finite_inputs_are_rejected():
    X, W, S = x.synthetic(4, 8, 128, 9)
    X[1, 2] = 0x7F80                              # +inf
    assert _run(X, W, S)[0] == 10001
    X, W, S = x.synthetic(4, 8, 128, 9)
    S[0, 0] = np.float32(np.inf)
    assert _run(X, W, S)[0] == 10001
