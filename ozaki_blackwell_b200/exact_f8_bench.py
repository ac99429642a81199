"""Speed of the correctly rounded BF16 x block-scaled FP8 product at an LLM-shaped size.

    python -m ozaki_blackwell_b200.exact_f8_bench [--m 2048 --k 7168 --n 18432 --reps 5]

X: bf16 N(0,1); W: uniform over the finite E4M3 codes; one FP32 scale per 128 x 128 block, 2^U[-8,0]; all generated on the
device from a seed. Prints the median wall time of ozb_bf16_fp8_gemm (which is synchronous), the correctly rounded
TFLOP/s (2 M N K / time), the number of INT8 planes the data needed and the number of outputs left open (0 expected).
"""
import argparse
import ctypes
import time

import torch

from ._lib import lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=7168)
    ap.add_argument("--n", type=int, default=18432)
    ap.add_argument("--reps", type=int, default=5)
    a = ap.parse_args()
    M, K, N = a.m, a.k, a.n
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    X = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
    codes = torch.tensor([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=torch.uint8, device="cuda")
    W = codes[torch.randint(0, codes.numel(), (K, N), device="cuda", generator=g)]
    S = torch.exp2(torch.rand(((K + 127) // 128, (N + 127) // 128), device="cuda", generator=g) * -8.0).to(torch.float32)
    Y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    opn, nm = ctypes.c_int(), ctypes.c_int()

    def run():
        rc = lib.ozb_bf16_fp8_gemm(M, N, K, X.data_ptr(), W.data_ptr(), S.data_ptr(), Y.data_ptr(), ctypes.byref(opn), ctypes.byref(nm), None)
        if rc:
            raise RuntimeError(lib.ozb_error(rc).decode())

    run()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.reps):
        t = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t)
    ts.sort()
    t = ts[len(ts) // 2]
    print(f"{M}x{K} bf16 times {K}x{N} e4m3 (FP32 block scales): {t * 1e3:.2f} ms, {2.0 * M * N * K / t / 1e12:.1f} correctly rounded TFLOP/s, "
          f"{nm.value} planes, {opn.value} open")


if __name__ == "__main__":
    main()
