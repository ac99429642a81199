"""Speed of the INT8 GEMM stage alone (the counterpart of the timing half of the reference's bench/gemm_i8_test.cu:38-51).

    python -m ozaki_blackwell_b200.gemm_bench [--m 8192 --n 8192 --k 8192 --planes 16 --reps 5 --fused 1]

Random int8 planes on the device, one warm-up, `reps` timed launches of ozb_gemm_i8_mod (fused residue output) or
ozb_gemm_i8 (int32 output) with CUDA events; prints ms and INT8 TOP/s per launch.
"""
import argparse
import ctypes

import torch

from ._lib import lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--planes", type=int, default=16)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--fused", type=int, default=1)
    a = ap.parse_args()
    M, N, K, Z = a.m, a.n, a.k, a.planes
    Kp, Np = (K + 127) // 128 * 128, (N + 15) // 16 * 16
    A = torch.randint(-128, 128, (Z, M, Kp), dtype=torch.int8, device="cuda")
    B = torch.randint(-128, 128, (Z, N, Kp), dtype=torch.int8, device="cuda")
    C = torch.empty((Z, M, Np), dtype=torch.int8 if a.fused else torch.int32, device="cuda")

    def launch():
        if a.fused:
            rc = lib.ozb_gemm_i8_mod(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, Z, Kp, Kp, Np, M * Kp, N * Kp, M * Np, 0, None)
        else:
            rc = lib.ozb_gemm_i8(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, Z, Kp, Kp, Np, M * Kp, N * Kp, M * Np, None)
        if rc:
            raise RuntimeError(lib.ozb_error(rc).decode())

    launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = torch.cuda.default_stream()   # the library launches on the legacy default stream when given NULL
    times = []
    for _ in range(a.reps):
        e0.record(stream)
        launch()
        e1.record(stream)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    rc = lib.ozb_status()
    if rc:
        raise RuntimeError(lib.ozb_error(rc).decode())
    times.sort()
    ms = times[len(times) // 2]
    print(f"M={M} N={N} K={K} planes={Z} fused={a.fused}: {ms:.3f} ms  {2.0 * Z * M * N * K / (ms * 1e-3) / 1e12:.0f} INT8 TOP/s "
          f"(min {times[0]:.3f}, max {times[-1]:.3f})")


if __name__ == "__main__":
    main()
