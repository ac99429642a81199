"""python -m ozaki_blackwell_b200 [n] [--kinds fp64,dd]: a self-test against exact rational arithmetic, then speed at n.

The counterpart of the reference package's `python -m ozaki_blackwell` (python/ozaki_blackwell/__main__.py): sampled
entries of small products are compared with exact sums of Python fractions, with the reference's pass thresholds (FP64:
8 units of 2^-53 for exponent spreads 2^+-0 and 2^+-8 at K = 256; double-double: 16 units of 2^-106); the triple-double
product is not built in this library and is reported as such. Then the median device time of an n x n x n product.
"""
import argparse
import sys
import time
from fractions import Fraction

import numpy as np

import ozaki_blackwell_b200 as ob


def sampled_error(a_parts, b_parts, c_parts, unit, samples, rng):
    """Largest |C - AB| / (|A||B|) over `samples` random entries, in units of `unit`, in exact rationals."""
    rows, cols = c_parts[0].shape
    inner = a_parts[0].shape[1]
    worst = Fraction(0)
    for _ in range(samples):
        i, j = int(rng.integers(rows)), int(rng.integers(cols))
        exact, mag = Fraction(0), Fraction(0)
        for t in range(inner):
            x = sum(Fraction(float(p[i, t])) for p in a_parts)
            y = sum(Fraction(float(p[t, j])) for p in b_parts)
            exact += x * y
            mag += abs(x * y)
        got = sum(Fraction(float(p[i, j])) for p in c_parts)
        if mag:
            worst = max(worst, abs(got - exact) / mag / Fraction(unit))
    return float(worst)


def main():
    ap = argparse.ArgumentParser(prog="python -m ozaki_blackwell_b200")
    ap.add_argument("n", nargs="?", type=int, default=4096)
    ap.add_argument("--kinds", default="fp64,dd")
    ap.add_argument("--no-selftest", action="store_true")
    args = ap.parse_args()
    info = ob.device()
    print(f"ozaki_blackwell_b200 {ob.__version__} on {info['name']} (sm_{info['sm']}, {info['sms']} SMs, L2 {info['l2_kib'] // 1024} MiB)")
    ok = True
    if not args.no_selftest:
        rng = np.random.default_rng(2026)
        size = 256

        def draw(spread, scale=1.0):
            return rng.standard_normal((size, size)) * np.exp2(rng.integers(-spread, spread + 1, (size, size))) * scale

        for spread in (0, 8):
            a, b = draw(spread), draw(spread)
            err = sampled_error([a], [b], [ob.matmul(a, b)], 2.0 ** -53, 32, rng)
            good = err <= 8
            ok &= good
            print(f"  FP64, K={size}, spread 2^+-{spread}: {err:.3g} units of 2^-53  {'ok' if good else 'FAIL'}")
        a, b = (draw(0), draw(0, 2.0 ** -53)), (draw(0), draw(0, 2.0 ** -53))
        err = sampled_error(a, b, ob.matmul_dd(a, b), 2.0 ** -106, 16, rng)
        good = err <= 16
        ok &= good
        print(f"  double-double, K={size}: {err:.3g} units of 2^-106  {'ok' if good else 'FAIL'}")
        print("  triple-double: not built in this library (ozb_tdgemm returns its 'not built' code)")
    n = args.n
    print(f"speed at n={n}, operands on the device, median of 5 (FP64-equivalent TFLOP/s):")
    for kind in [k for k in args.kinds.split(",") if k]:
        ms, tf = ob.bench(n, kind)
        print(f"  {kind:5s} {ms:9.3f} ms  {tf:7.2f} TFLOP/s")
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((n, n)), rng.standard_normal((n, n))
    t = time.perf_counter()
    ob.matmul(a, b)
    print(f"  fp64 from NumPy arrays, transfers included: {(time.perf_counter() - t) * 1e3:.1f} ms")
    ob.release()
    print("self-test", "skipped" if args.no_selftest else ("passed" if ok else "FAILED"))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
