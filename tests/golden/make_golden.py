"""Generates tests/golden/reference_outputs.npz from the REFERENCE ITSELF.

Run on a machine with a GPU after `make -C oracle ref` has built the reference's own C ABI (its python/capi.cu, compiled
unmodified from the reference sources into oracle/_ref/libozb_ref.so). For every case in cases.py it calls the reference's
ozb_dgemm on host arrays and stores the 64-bit patterns of C together with a digest of the inputs, so that the CPU tests
can compare the checker with the reference's real output without a GPU and without the reference sources.

    python tests/golden/make_golden.py [output.npz]
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_outputs.npz")
    ref = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle", "_ref", "libozb_ref.so"))
    ref.ozb_dgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2
    ref.ozb_error.restype = ctypes.c_char_p
    store = {}
    for name in cases.CASES:
        A, B, nm = cases.inputs(name)
        M, K = A.shape
        N = B.shape[1]
        C = np.full((M, N), np.nan)
        rc = ref.ozb_dgemm(M, N, K, A.ctypes.data, B.ctypes.data, C.ctypes.data, nm, 1)
        if rc:
            raise RuntimeError(f"{name}: reference ozb_dgemm returned {rc}: {ref.ozb_error(rc).decode()}")
        store[name + ".C"] = C.view(np.uint64)
        store[name + ".inputs_sha256"] = np.array(cases.digest(A, B))
        print(name, C.shape, "ok")
    ref.ozb_ddgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 6 + [ctypes.c_int]
    for name in cases.DD_CASES:
        Ah, Al, Bh, Bl = cases.dd_inputs(name)
        M, K = Ah.shape
        N = Bh.shape[1]
        Ch, Cl = np.full((M, N), np.nan), np.full((M, N), np.nan)
        rc = ref.ozb_ddgemm(M, N, K, Ah.ctypes.data, Al.ctypes.data, Bh.ctypes.data, Bl.ctypes.data, Ch.ctypes.data, Cl.ctypes.data, 1)
        if rc:
            raise RuntimeError(f"{name}: reference ozb_ddgemm returned {rc}: {ref.ozb_error(rc).decode()}")
        store[name + ".Ch"], store[name + ".Cl"] = Ch.view(np.uint64), Cl.view(np.uint64)
        store[name + ".inputs_sha256"] = np.array(cases.digest(Ah, Al, Bh, Bl))
        print(name, Ch.shape, "ok")
    ref.ozb_release()
    np.savez_compressed(out, **store)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
