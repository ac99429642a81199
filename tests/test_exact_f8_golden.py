"""The CPU checker of the correctly rounded BF16 x block-scaled FP8 product against the REFERENCE'S OWN host
superaccumulator (llm/ultra.cu:336-369 of the reference): stored outputs of that code (tests/golden/exact_f8_reference.npz,
made by tests/golden/make_golden_f8.py) and, where the reference build is present (oracle/_ref/libultra_ref.so), the code
itself on fresh inputs. No GPU needed."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))
sys.path.insert(0, os.path.join(HERE, "golden"))
import exact_f8_oracle as x  # noqa: E402
import f8_cases  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "exact_f8_reference.npz"))


@pytest.mark.parametrize("name", list(f8_cases.CASES))
def test_checker_reproduces_the_reference_superaccumulator(name):
    X, W, S = f8_cases.inputs(name)
    want = GOLDEN[name]
    assert want.shape == (X.shape[0], W.shape[1])
    got = x.product(X, W, S).view(np.uint32)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} outputs differ from the reference's exact_dot"


def test_stored_cases_are_not_trivial():
    Y = GOLDEN["tiny_k128"].view(np.float32)
    assert np.any((np.abs(Y) < 1.17e-38) & (Y != 0)) and np.abs(Y).max() < 1e-37   # subnormal outputs: the rounding position is clamped
    Y = GOLDEN["wide_k384"].view(np.float32)
    assert np.all(Y[1] == 0) and np.abs(Y).max() > 1e9               # a zero row, large magnitudes


def test_against_the_reference_code_itself_when_it_is_built():
    path = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libultra_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libultra_ref.so is built only where the reference sources are")
    import make_golden_f8
    ref = make_golden_f8.load_reference()
    rng = np.random.default_rng(99)
    M, N, K = 5, 130, 512
    X = f8_cases.bf16_bits(np.ldexp(rng.standard_normal((M, K)), rng.integers(-12, 13, (M, K)).astype(np.int32)).astype(np.float32))
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    W = codes[rng.integers(0, codes.size, (K, N))]
    S = f8_cases.bf16_to_f32(f8_cases.bf16_bits(np.exp2(rng.uniform(-8, 0, (K // 128, 2))).astype(np.float32)))
    want = make_golden_f8.reference_product(ref, X, W, S).view(np.uint32)
    got = x.product(X, W, S).view(np.uint32)
    assert np.array_equal(got, want)
