"""Speed of the scale / residue / reconstruction stages alone, one stage call at a time (what the reference's phase
benchmark does with its own kernels, bench/phases.cu:21-30).

    python -m ozaki_blackwell_b200.stage_bench [--n 8192 --moduli 16 --reps 10]
    OZB_LIBRARY=/path/to/another/build.so python -m ozaki_blackwell_b200.stage_bench      # the same for another build of the ABI

Synthetic entries U[-1,1) * 2^e, e in [-8, 8], on the device; one warm-up call, then `reps` calls of
ozb_scale_residues_rows, ozb_scale_residues_cols (both passes over B) and ozb_crt_i8 between CUDA events; prints the
mean ms per call and the achieved GB/s of the stage's algorithmic bytes.
"""
import argparse

import torch

from ._lib import lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--moduli", type=int, default=16)
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    n, nm = a.n, a.moduli
    dev = "cuda"
    X = (torch.rand((n, n), dtype=torch.float64, device=dev) * 2 - 1) * torch.exp2(torch.randint(-8, 9, (n, n), device=dev).double())
    bits = lib.ozb_bits_for(nm, n, 62)
    s = torch.empty(n, dtype=torch.int32, device=dev)
    R = torch.empty((nm, n, n), dtype=torch.int8, device=dev)
    cm = torch.zeros(n, dtype=torch.int64, device=dev)
    C = torch.empty((n, n), dtype=torch.float64, device=dev)
    Rr = torch.randint(-90, 90, (nm, n, n), dtype=torch.int8, device=dev)
    zero = torch.zeros(n, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream()

    def check(code):
        if code:
            raise RuntimeError(lib.ozb_error(code).decode())

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(a.reps):
            fn()
        e1.record(st)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.reps

    stages = [
        ("scales + residues of the rows of A", (8 + nm) * n * n,
         lambda: check(lib.ozb_scale_residues_rows(nm, X.data_ptr(), n, n, n, bits, s.data_ptr(), R.data_ptr(), n, n * n, st.cuda_stream))),
        ("scales + residues of the columns of B", (16 + nm) * n * n,
         lambda: check(lib.ozb_scale_residues_cols(nm, X.data_ptr(), n, n, n, bits, cm.data_ptr(), s.data_ptr(), R.data_ptr(), n, n * n, st.cuda_stream))),
        ("reconstruction from int8 residues", (8 + nm) * n * n,
         lambda: check(lib.ozb_crt_i8(nm, Rr.data_ptr(), n * n, n, n, n, zero.data_ptr(), zero.data_ptr(), C.data_ptr(), n, st.cuda_stream))),
    ]
    for name, nbytes, fn in stages:
        ms = timed(fn)
        print(f"{name:40s} {ms:7.3f} ms  {nbytes / ms / 1e6:7.0f} GB/s")
    check(lib.ozb_status())


if __name__ == "__main__":
    main()
