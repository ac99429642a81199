"""Seeded cases of the correctly rounded BF16 x block-scaled FP8 product whose outputs from the reference's own host
superaccumulator are stored in exact_f8_reference.npz (shared by the generator and the tests).

The reference's block scale is BF16 (llm/ultra.cu:57-60), so every scale here is a BF16-representable FP32 value; the
activations are BF16 and the weights finite E4M3 codes, as in the benchmark configuration."""
import numpy as np

# name -> (M, N, K, seed, family)
CASES = {
    "normal_k256": (12, 40, 256, 21, "normal"),
    "normal_k7168": (3, 24, 7168, 22, "normal"),      # the benchmark configuration's inner length
    "wide_k384": (8, 260, 384, 23, "wide"),           # exponents spread over many binades, zeros, a zero and a small scale
    "tiny_k128": (4, 8, 128, 24, "tiny"),             # subnormal outputs
}


def bf16_bits(x):
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def inputs(name):
    """X uint16 [M][K] (bf16 bits), W uint8 [K][N] (e4m3 codes), S float32 [K/128][ceil(N/128)] holding BF16 values."""
    M, N, K, seed, family = CASES[name]
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if family == "wide":
        x = np.ldexp(x, rng.integers(-30, 31, (M, K)).astype(np.int32)).astype(np.float32)
        x[1, :] = 0.0
        x[2, ::3] = -0.0
    if family == "tiny":
        x = np.ldexp(x, -60).astype(np.float32)
    X = bf16_bits(x)
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    W = codes[rng.integers(0, codes.size, (K, N))]
    s = np.exp2(rng.uniform(-8.0, 0.0, (K // 128, (N + 127) // 128))).astype(np.float32)
    if family == "wide":                              # (no negative scale: the reference's decoder drops a scale's sign bit)
        s[1, 1] = 0.0
        s[2, 0] = np.float32(2.0 ** -18)
    if family == "tiny":
        s = (s * np.float32(2.0 ** -70)).astype(np.float32)
    S = bf16_to_f32(bf16_bits(s))
    return X, W, S
