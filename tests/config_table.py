"""Prints the accuracy / speed table of the benchmark configurations on one GPU (a script, not a test):

    python tests/config_table.py [--sizes 4096 8192] > config_table.md

For every size, modulus count (12, 14, 16 at n = 4096; 16 at the other sizes) and input family (U[-1,1) and U[-1,1) * 2^e,
e in [-8, 8]): this library's time (median of 5 after a warm-up, CUDA events around the synchronous ozb_dgemm, as the
reference's bench/ozaki_test.cu:94-102 measures), FP64-equivalent TFLOP/s, the componentwise error on 1024 sampled
entries against the exact Dot2 sum (bench/ozaki_test.cu:42-63) in units of 2^-53, the reference's own kernels rebuilt for
sm_100a (oracle/_ref/libozb_ref.so, when present) timed the same way with a bit-for-bit comparison of C, and cuBLAS DGEMM
(torch.matmul in float64) with its error. Uses the CPU checker for the errors, so it lives under tests/.
"""
import argparse
import ctypes
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import oracle_lib as o  # noqa: E402
from ozaki_blackwell_b200._lib import lib  # noqa: E402


def timed(fn, reps=5):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st = torch.cuda.default_stream()
    ts = []
    for _ in range(reps):
        e0.record(st)
        fn()
        e1.record(st)
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[4096, 8192])
    a = ap.parse_args()
    ref_path = os.path.join(o.ORACLE_DIR, "_ref", "libozb_ref.so")
    ref = ctypes.CDLL(ref_path) if os.path.exists(ref_path) else None
    if ref:
        ref.ozb_dgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2
    print("| n | moduli | inputs | this library ms | TFLOP/s | max err (2^-53, 1024 entries) | reference kernels on this GPU ms | TFLOP/s | same bits | cuBLAS DGEMM ms | TFLOP/s | err |")
    print("|---|---|---|---|---|---|---|---|---|---|---|---|")
    for n in a.sizes:
        for spread in (0, 8):
            g = torch.Generator(device="cuda")
            g.manual_seed(n + spread)
            A = torch.rand((n, n), dtype=torch.float64, device="cuda", generator=g) * 2 - 1
            B = torch.rand((n, n), dtype=torch.float64, device="cuda", generator=g) * 2 - 1
            if spread:
                A = torch.ldexp(A, torch.randint(-spread, spread + 1, (n, n), device="cuda", generator=g, dtype=torch.int32))
                B = torch.ldexp(B, torch.randint(-spread, spread + 1, (n, n), device="cuda", generator=g, dtype=torch.int32))
            C, R = torch.empty_like(A), torch.empty_like(A)
            Ah, Bh = A.cpu().numpy(), B.cpu().numpy()
            idx = np.random.default_rng(1).integers(0, n * n, 1024)
            t_cb = timed(lambda: torch.matmul(A, B, out=R))
            e_cb = o.err_units_sampled(Ah, Bh, R.cpu().numpy(), idx)
            for nm in ((12, 14, 16) if n == 4096 else (16,)):
                def ours():
                    rc = lib.ozb_dgemm(n, n, n, A.data_ptr(), B.data_ptr(), C.data_ptr(), nm, 0)
                    assert rc == 0, lib.ozb_error(rc)
                t = timed(ours)
                err = o.err_units_sampled(Ah, Bh, C.cpu().numpy(), idx)
                t_ref, same = float("nan"), "n/a"
                if ref:
                    def theirs():
                        assert ref.ozb_dgemm(n, n, n, A.data_ptr(), B.data_ptr(), R.data_ptr(), nm, 0) == 0
                    t_ref = timed(theirs)
                    same = "yes" if torch.equal(C.view(torch.int64), R.view(torch.int64)) else "NO"
                fl = 2.0 * n ** 3 / 1e9
                print(f"| {n} | {nm} | 2^±{spread} | {t:.3f} | {fl / t:.1f} | {err:.3g} | {t_ref:.2f} | {fl / t_ref:.1f} | {same} | {t_cb:.2f} | {fl / t_cb:.1f} | {e_cb:.3g} |", flush=True)
            if ref:
                ref.ozb_release()
            lib.ozb_release()


if __name__ == "__main__":
    main()
