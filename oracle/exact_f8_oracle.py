"""CPU checker of the correctly rounded BF16 x block-scaled FP8 product.

TEST INFRASTRUCTURE ONLY (imported by tests/ and nothing else): exact integer arithmetic with Python integers, so sized for
small matrices and for samples of large ones.

The contract is the one the reference's exact products are tested against (reference paths): every output is the
round-to-nearest-even FP32 value of the EXACT real sum, as the reference's host superaccumulator computes it
(llm/ultra.cu:336-369: exact_dot / big_round, p = 24 bits, FP32 exponent range with subnormals). The operand decodings follow
llm/ultra.cu:45-62 (wdec): BF16 value = m 2^e with m = 128 + f (or f for exponent field 0), e = ex - 134 (or -133);
E4M3 value = m 2^e with m = 8 + f (or f), e = ex - 10 (or -9), i.e. an integer v = E4M3 * 2^9 as in llm/tgemm.cu:37-40;
a block scale multiplies the 128 x 128 block of W it belongs to (llm/ultra.cu:57-60 uses a BF16 scale; here it is FP32,
decoded as m = 2^23 + f (or f), e = ex - 150 (or -149), llm/ultra.cu:51-53).
    Y[i][j] = RN_fp32( sum_k X[i][k] * W[k][j] * S[k // 128][j // 128] ),   X: M x K bf16,  W: K x N e4m3,  S: fp32 blocks
"""
import numpy as np


def decode_bf16(u):
    u = np.asarray(u, dtype=np.uint16).astype(np.int64)
    ex, f = (u >> 7) & 255, u & 127
    m = np.where(ex != 0, 128 + f, f)
    e = np.where(ex != 0, ex - 134, -133)
    return np.where(u >> 15 != 0, -m, m), e


def decode_e4m3_times_512(b):
    b = np.asarray(b, dtype=np.uint8).astype(np.int64)
    ex, f = (b >> 3) & 15, b & 7
    v = np.where(ex != 0, (8 + f) << np.maximum(ex - 1, 0), f)
    return np.where(b >> 7 != 0, -v, v)


def decode_f32(s):
    u = np.asarray(s, dtype=np.float32).view(np.uint32).astype(np.int64)
    ex, f = (u >> 23) & 255, u & 0x7FFFFF
    m = np.where(ex != 0, (1 << 23) + f, f)
    e = np.where(ex != 0, ex - 150, -149)
    return np.where(u >> 31 != 0, -m, m), e


def round_to_f32(i, e):
    """The FP32 nearest (ties to even) to the integer i times 2^e, as a numpy float32 (inf on overflow)."""
    if i == 0:
        return np.float32(0.0)
    neg, a = i < 0, abs(i)
    msb = a.bit_length() - 1 + e                  # exponent of the leading bit
    lsb = max(msb - 23, -149)                     # exponent of the last kept bit (subnormals stop at 2^-149)
    r = lsb - e
    if r > 0:
        q, rem, half = a >> r, a & ((1 << r) - 1), 1 << (r - 1)
        if rem > half or (rem == half and (q & 1)):
            q += 1
    else:
        q, lsb = a, e
    if q.bit_length() - 1 + lsb > 127:
        val = np.float32(np.inf)
    else:
        val = np.float32(np.ldexp(np.float64(q), lsb))   # q has at most 25 bits and the result is representable
    return -val if neg else val


def exact_entry(xm, xe, v, sm, se, i, j):
    """Exact sum of output (i, j) as (integer, exponent)."""
    K = xm.shape[1]
    emin = int(xe[i].min()) + int(se[:, j // 128].min()) - 9
    total = 0
    for k in range(K):
        m = int(xm[i, k]) * int(v[k, j]) * int(sm[k // 128, j // 128])
        if m:
            total += m << (int(xe[i, k]) + int(se[k // 128, j // 128]) - 9 - emin)
    return total, emin


def product(X, W, S, entries=None):
    """X uint16 [M][K] (bf16 bits), W uint8 [K][N] (e4m3 bits), S float32 [ceil(K/128)][ceil(N/128)].
    entries = None: the full M x N result; else a list of (i, j): the values at those positions."""
    xm, xe = decode_bf16(X)
    v = decode_e4m3_times_512(W)
    sm, se = decode_f32(S)
    M, N = X.shape[0], W.shape[1]
    if entries is None:
        Y = np.empty((M, N), dtype=np.float32)
        for i in range(M):
            for j in range(N):
                Y[i, j] = round_to_f32(*exact_entry(xm, xe, v, sm, se, i, j))
        return Y
    return np.array([round_to_f32(*exact_entry(xm, xe, v, sm, se, i, j)) for i, j in entries], dtype=np.float32)


def to_bf16_bits(x):
    """float32 array -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def synthetic(M, N, K, seed):
    """BASELINE config 4's family: X bf16 N(0,1); W uniform over the finite E4M3 codes; S = 2^U[-8,0] in FP32."""
    rng = np.random.default_rng(seed)
    X = to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    W = codes[rng.integers(0, codes.size, (K, N))]
    S = np.exp2(rng.uniform(-8.0, 0.0, ((K + 127) // 128, (N + 127) // 128))).astype(np.float32)
    return X, W, S
