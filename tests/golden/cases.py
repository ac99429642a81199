"""The seeded cases whose reference outputs are stored under tests/golden/ (shared by the generator and the tests)."""
import hashlib

import numpy as np

# name -> (M, N, K, moduli, family, seed)
CASES = {
    "cfg1_nm16": (256, 256, 512, 16, "pow2", 0),
    "cfg1_nm12": (256, 256, 512, 12, "pow2", 0),
    "cfg1_nm8": (256, 256, 512, 8, "pow2", 0),
    "odd_nm16": (200, 300, 500, 16, "pow2", 3),
    "odd_nm13": (77, 129, 1031, 13, "uniform", 4),
    "wide_nm16": (96, 160, 384, 16, "wide", 5),
    "tiny_nm16": (3, 5, 7, 16, "pow2", 6),
}


def inputs(name):
    M, N, K, nm, family, seed = CASES[name]
    rng = np.random.default_rng(1000 + seed)
    A = rng.uniform(-1.0, 1.0, (M, K))
    B = rng.uniform(-1.0, 1.0, (K, N))
    if family == "pow2":          # U[-1,1) * 2^e, e uniform integer in [-8, 8]
        A = np.ldexp(A, rng.integers(-8, 9, (M, K)).astype(np.int32))
        B = np.ldexp(B, rng.integers(-8, 9, (K, N)).astype(np.int32))
    elif family == "wide":        # rows / columns of very different magnitude, a zero row and a zero column
        A = np.ldexp(A, rng.integers(-40, 41, (M, 1)).astype(np.int32) + rng.integers(-8, 9, (M, K)).astype(np.int32))
        B = np.ldexp(B, rng.integers(-40, 41, (1, N)).astype(np.int32) + rng.integers(-8, 9, (K, N)).astype(np.int32))
        A[5, :] = 0.0
        B[:, 9] = 0.0
    return np.ascontiguousarray(A), np.ascontiguousarray(B), nm


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


# double-double cases: name -> (M, N, K, seed); 32 moduli (the reference's C ABI fixes that count)
DD_CASES = {"dd_cfg": (128, 128, 256, 20), "dd_odd": (77, 130, 515, 21)}


def dd_inputs(name):
    M, N, K, seed = DD_CASES[name]
    rng = np.random.default_rng(2000 + seed)
    Ah = np.ldexp(rng.uniform(-1.0, 1.0, (M, K)), rng.integers(-8, 9, (M, K)).astype(np.int32))
    Bh = np.ldexp(rng.uniform(-1.0, 1.0, (K, N)), rng.integers(-8, 9, (K, N)).astype(np.int32))
    Al = Ah * 2.0**-53 * rng.uniform(-1.0, 1.0, (M, K))
    Bl = Bh * 2.0**-53 * rng.uniform(-1.0, 1.0, (K, N))
    return [np.ascontiguousarray(x) for x in (Ah, Al, Bh, Bl)]
