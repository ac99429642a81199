"""Generates tests/golden/exact_f8_reference.npz from the REFERENCE'S OWN host superaccumulator.

Run where the reference sources are present, after `make -C oracle ref` has built oracle/_ref/libultra_ref.so (the
reference's llm/ultra.cu compiled where it lies, with one exported function around its exact_dot, llm/ultra.cu:336-369).
For every case in f8_cases.py each output is computed by the reference's code -- every product added exactly into its
2560-bit accumulator, rounded once to 24 bits -- and the FP32 bit patterns are stored, so that the CPU tests can compare
the checker (oracle/exact_f8_oracle.py) with the reference without its sources, and the GPU tests the kernel with both.

    python tests/golden/make_golden_f8.py [output.npz]
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import f8_cases  # noqa: E402


def load_reference():
    ref = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle", "_ref", "libultra_ref.so"))
    ref.ozref_exact_dot_e4m3b.restype = ctypes.c_float
    ref.ozref_exact_dot_e4m3b.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    return ref


def reference_product(ref, X, W, S):
    """Y[i][j] through the reference's exact_dot: its weight matrix is stored by output (row j of W^T), with the BF16
    scales of that row's blocks beside it."""
    M, K = X.shape
    N = W.shape[1]
    xf = f8_cases.bf16_to_f32(X)
    Wt = np.ascontiguousarray(W.T)
    Sb = f8_cases.bf16_bits(S)                                  # exact: the scales are BF16 values
    Y = np.empty((M, N), dtype=np.float32)
    for j in range(N):
        w = np.ascontiguousarray(Wt[j])
        s = np.ascontiguousarray(Sb[:, j // 128])
        for i in range(M):
            x = np.ascontiguousarray(xf[i])
            Y[i, j] = ref.ozref_exact_dot_e4m3b(w.ctypes.data, s.ctypes.data, K, x.ctypes.data, 24)
    return Y


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "exact_f8_reference.npz")
    ref = load_reference()
    store = {}
    for name in f8_cases.CASES:
        X, W, S = f8_cases.inputs(name)
        store[name] = reference_product(ref, X, W, S).view(np.uint32)
        print(name, store[name].shape)
    np.savez_compressed(out, **store)


if __name__ == "__main__":
    main()
