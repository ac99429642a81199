"""The CPU checker of the correctly rounded BF16 x FP8 product (oracle/exact_f8_oracle.py) against independent
conversions: torch's bf16 / float8_e4m3fn decoding and numpy's float64 -> float32 rounding (no GPU needed)."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import exact_f8_oracle as x  # noqa: E402


def test_decoders_match_torch():
    u = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    fin = ((u >> 7) & 255) != 255
    m, e = x.decode_bf16(u[fin])
    ref = torch.from_numpy(u[fin].view(np.int16)).view(torch.bfloat16).to(torch.float64).numpy()
    assert np.array_equal(np.ldexp(m.astype(np.float64), e.astype(np.int32)), ref)
    b = np.arange(256, dtype=np.uint16).astype(np.uint8)
    ok = (b & 0x7F) != 0x7F
    v = x.decode_e4m3_times_512(b[ok])
    ref = torch.from_numpy(b[ok]).view(torch.float8_e4m3fn).to(torch.float64).numpy()
    assert np.array_equal(v / 512.0, ref)
    s = np.array([1.0, 0.37, 2.0**-8, 1e-40, -3.5, 0.0], dtype=np.float32)
    sm, se = x.decode_f32(s)
    assert np.array_equal(np.ldexp(sm.astype(np.float64), se.astype(np.int32)), s.astype(np.float64))


def test_rounding_matches_numpy_and_handles_ties_subnormals_overflow():
    rng = np.random.default_rng(0)
    with np.errstate(over="ignore"):
        for _ in range(5000):
            i, ex = int(rng.integers(-2**52, 2**52)), int(rng.integers(-210, 90))
            want, got = np.float32(np.ldexp(np.float64(i), ex)), x.round_to_f32(i, ex)
            assert got == want or (np.isinf(got) and np.isinf(want)), (i, ex)
    assert x.round_to_f32((1 << 24) + 1, 0) == np.float32(2**24)          # tie to even, down
    assert x.round_to_f32((1 << 24) + 3, 0) == np.float32(2**24 + 4)      # tie to even, up
    assert x.round_to_f32(((1 << 24) + 1) << 100 | 1, -100) == np.float32(2**24 + 2)   # one bit beyond a tie decides
    assert x.round_to_f32(1, -150) == 0 and x.round_to_f32(3, -151) == np.float32(2.0**-149)
    assert np.isinf(x.round_to_f32((1 << 24) - 1, 105)) and x.round_to_f32(-1, -149) == -np.float32(2.0**-149)


def test_small_product_against_float64():
    X, W, S = x.synthetic(6, 9, 256, 1)
    Y = x.product(X, W, S)
    xf = torch.from_numpy(X.view(np.int16)).view(torch.bfloat16).to(torch.float64).numpy()
    wf = torch.from_numpy(W).view(torch.float8_e4m3fn).to(torch.float64).numpy()
    approx = sum(xf[:, kb * 128:(kb + 1) * 128] @ wf[kb * 128:(kb + 1) * 128] * S[kb, 0].astype(np.float64) for kb in range(2))
    assert np.all(np.abs(Y - approx) <= np.abs(approx) * 2.0**-23 + 1e-30)
