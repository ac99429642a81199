#!/usr/bin/env python
"""Benchmark of the Ozaki-II FP64 product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--n 8192] [--moduli 16]

One step = one FP64-accurate product C = A B with 16 moduli on seeded synthetic matrices (entries U[-1,1) * 2^e, e a
uniform integer in [-8, 8]). At N = 1 the workload is n = 8192 (M = N = K = n). At N > 1 (one process per GPU, launched
by torch.distributed.run) rank g owns n rows of A and of C, B lives on rank 0 and is broadcast over NCCL inside every
step (weak scaling: M = n * N in total). Rank 0 prints one JSON line.

  value     FP64-equivalent TFLOP/s (2 M N K / time), operands resident in HBM, CUDA events, max over ranks
  e2e       the same through the reference's entry point ozb_dgemm(on_host = 1): pinned host operands, H2D and D2H inside
  roofline  the INT8 GEMM kernel: 2 nm M N K integer operations / its event-timed duration inside the same timed region,
            against twice the measured dense bf16 rate (the tensor cores run INT8 at twice the bf16 rate)
  cpu_baseline  the CPU restatement of the reference's pipeline (oracle/) on the host cores, on a bounded sample
--impl reference times that CPU restatement alone (the reference has no CPU implementation of the Ozaki pipeline of its
own: its device code is restated in oracle/ozaki2_oracle.c), rank 0 only.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SPREAD = 8
PEAKS_FILE = os.path.join(ROOT, "MEASURED_PEAKS.json")
FALLBACK_BF16_TFLOPS, FALLBACK_HBM_GBS = 1590.0, 6650.0


def peaks():
    try:
        with open(PEAKS_FILE) as f:
            p = json.load(f)
        return {"bf16": float(p["bf16_tflops_sustained"]), "bf16_burst": float(p["bf16_tflops"]), "hbm": float(p["hbm_gbs"]),
                "source": "measured"}
    except Exception:
        return {"bf16": 1400.0, "bf16_burst": FALLBACK_BF16_TFLOPS, "hbm": FALLBACK_HBM_GBS, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 20 ms. The sampler is started early (nvidia-smi
    takes a moment to come up) and every sample carries a time stamp; only the samples that fall inside the timed region
    [mark_start(), mark_end()] are summarised."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path, self.t0, self.t1 = index, None, None, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            for _ in range(100):                      # wait (at most 5 s) for the first sample
                if os.path.getsize(self.path) > 0:
                    break
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "power_w": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 8:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    c, m, p = float(f[1]), float(f[2]), float(f[3])
                except ValueError:
                    continue
                if self.t0 is not None and not (self.t0 <= ts <= self.t1 + 0.02):
                    continue
                sm.append(c); mx.append(m); pw.append(p)
                for nme, v in zip(names, f[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), power_w=statistics.median(pw), reasons=sorted(reasons), samples=len(sm))
        return out


def synthetic(rows, cols, seed, device):
    """U[-1,1) * 2^e, e uniform integer in [-SPREAD, SPREAD], generated on the device from a seed."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.rand((rows, cols), dtype=torch.float64, device=device, generator=g) * 2.0 - 1.0
    e = torch.randint(-SPREAD, SPREAD + 1, (rows, cols), device=device, generator=g, dtype=torch.int32)
    return torch.ldexp(x, e)


# ---------------------------------------------------------------------------------------------------------------
# CPU leg: the checker's pipeline on the host cores (bounded sample), also the accuracy / parity check of the GPU result
# ---------------------------------------------------------------------------------------------------------------
def cpu_pipeline_sample(A_rows, B, nm):
    """Times the CPU restatement on `rows` rows of the product. B's scale/residue pass is timed on its own and charged
    once for the whole product, the per-row work is scaled to all M rows. Returns (C_rows, t_b, t_rows)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import oracle_lib as o   # the checker: used here as the timed CPU baseline, never by the GPU path
    rows, K = A_rows.shape
    N = B.shape[1]
    bits = o.bits_for(nm, K)
    t0 = time.perf_counter()
    sb = o.scales(B, N, K, 1, N, bits)
    Br = o.residues(B, N, K, 1, N, sb, nm)
    t1 = time.perf_counter()
    sa = o.scales(A_rows, rows, K, K, 1, bits)
    Ar = o.residues(A_rows, rows, K, K, 1, sa, nm)
    Cl = np.stack([o.gemm_i8(Ar[l], Br[l]) for l in range(nm)])
    C = o.crt(Cl, sa, sb)
    t2 = time.perf_counter()
    return C, t1 - t0, t2 - t1


def run_reference(args):
    import numpy as np
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n, nm, rows = args.n, args.moduli, args.cpu_rows
    rng = np.random.default_rng(0)
    B = np.ldexp(rng.uniform(-1, 1, (n, n)), rng.integers(-SPREAD, SPREAD + 1, (n, n)).astype(np.int32))
    A = np.ldexp(rng.uniform(-1, 1, (rows, n)), rng.integers(-SPREAD, SPREAD + 1, (rows, n)).astype(np.int32))
    cores = os.cpu_count()
    times = []
    for s in range(args.warmup + args.steps):
        _, tb, tr = cpu_pipeline_sample(A, B, nm)
        if s >= args.warmup:
            times.append(tb + tr * (n / rows))
    t = sum(times) / len(times)
    val = 2.0 * n ** 3 / t / 1e12
    sample = (f"{rows} of {n} rows per step; B's scale/residue pass charged once per product, the per-row work scaled to {n} rows")
    print(json.dumps({
        "impl": "reference", "metric": "fp64_equiv_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 residues / int32 accumulate / f64 in-out", "data": "synthetic",
        "config": {"workload": f"FP64 GEMM n={n}, {nm} moduli (Ozaki-II), entries U[-1,1)*2^e, e in [-8,8]", "moduli": nm, "n": n},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from ozaki_blackwell_b200._lib import lib
    from ozaki_blackwell_b200.dist import RowShardedGemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU path"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def check(code):
        if code:
            raise RuntimeError(lib.ozb_error(code).decode())

    n, nm = args.n, args.moduli
    N = K = n                                       # B is n x n
    M = n // world if args.strong else n            # rows of A and C per rank (weak: n each; strong: n in total)
    A = synthetic(M, K, 1000 + rank, dev)
    B = synthetic(K, N, 7, dev) if rank == 0 else None
    C = torch.empty((M, N), dtype=torch.float64, device=dev)
    stream = torch.cuda.current_stream()
    op = RowShardedGemm(M, N, K, nm, panels=args.panels, layout=args.layout)
    plan = op.engine._plan
    steps, warm = args.steps, args.warmup
    check(lib.ozb_plan_profile(plan, steps if world == 1 else 0))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(warm):
        op(A, B, C)
    barrier()
    if world == 1:
        check(lib.ozb_plan_profile(plan, steps))      # restart the slot counter after the warm-up
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.mark_start()
    e0.record(stream)
    for _ in range(steps):
        op(A, B, C)
    e1.record(stream)
    barrier()
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    op.engine.status()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / steps
    flops_step = 2.0 * M * N * K * world
    value = flops_step / (ms_step * 1e-3) / 1e12

    # phases of the same timed steps (single GPU: events recorded inside the library on the same stream)
    pk = peaks()
    roof = None
    phases = None
    if world == 1:
        ph = np.zeros((steps, 4))
        buf = (ctypes.c_float * 4)()
        for s in range(steps):
            check(lib.ozb_plan_phase_ms(plan, s, ctypes.byref(buf)))
            ph[s] = list(buf)
        phases = ph.mean(axis=0)
        ops = 2.0 * nm * M * N * K
        achieved = ops / (phases[1] * 1e-3) / 1e12
        # the denominator: this GPU's own INT8 tensor rate, measured now by the library's probe (tcgen05.mma alone on
        # random bytes, the GEMM kernel's instruction shape). Two figures, as for any kernel on a power-capped part: a burst
        # of about a millisecond, and a run of about 0.1 s, after which the power limit has pulled the clock down. The GEMM
        # kernel is timed inside steps that keep the GPU busy for far longer than that, so the sustained figure is its
        # peak; the burst figure is reported beside it.
        ms_p, tops_p = ctypes.c_float(), ctypes.c_double()
        probe = {"burst_one_cta": 0.0, "burst_cta_pair": 0.0}
        for pair in (0, 1):
            for _ in range(3):
                check(lib.ozb_int8_peak(2000, pair, ctypes.byref(ms_p), ctypes.byref(tops_p)))
                key = "burst_cta_pair" if pair else "burst_one_cta"
                probe[key] = max(probe[key], tops_p.value)
        for _ in range(2):                      # the second run starts with the limit already active
            check(lib.ozb_int8_peak(160000, 1, ctypes.byref(ms_p), ctypes.byref(tops_p)))
        probe["sustained_cta_pair"] = tops_p.value
        probe["sustained_ms"] = ms_p.value
        peak = probe["sustained_cta_pair"]
        burst = max(probe["burst_one_cta"], probe["burst_cta_pair"])
        # DRAM bytes of one GEMM launch: the ncu capture at n = 4096 (profiles/gemm_i8_tc2_n4096_16moduli.md) measured
        # 784.0 MB against 805.3 MB of algorithmic bytes (every residue byte read once, every product byte written once);
        # traffic is proportional to those bytes, so it is scaled to this launch by them
        traffic = 784.0 / 805.3 * nm * (M * K + N * K + M * N)
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
                "kernel": "gemm_i8_tc2<fused mod> (cta_group::2)", "peak_burst": burst, "frac_of_burst": achieved / burst,
                "peak_probe_int8_tops": probe,
                "note": "INT8 tera-operations/s. peak = sustained tensor-pipe probe (0.1 s of tcgen05.mma alone) measured in this run on "
                "this GPU, the kernel being timed inside long steps; peak_burst = the same probe for 1 ms (MEASURED_PEAKS.json holds "
                f"no INT8 figure); for comparison 2 x measured dense bf16: sustained {2 * pk['bf16']:.0f}, burst {2 * pk['bf16_burst']:.0f} "
                f"({pk['source']}); nominal dense INT8 4500"}

    # end to end through the reference's entry point, host operands in pinned memory
    e2e = None
    if args.e2e_steps > 0:
        Ah = torch.empty((M, K), dtype=torch.float64, pin_memory=True); Ah.copy_(A)
        if rank == 0:
            Bh = torch.empty((K, N), dtype=torch.float64, pin_memory=True); Bh.copy_(B)
        Ch = torch.empty((M, N), dtype=torch.float64, pin_memory=True)
        if world == 1:
            def e2e_step():
                check(lib.ozb_dgemm(M, N, K, Ah.data_ptr(), Bh.data_ptr(), Ch.data_ptr(), nm, 1))
            h2d, d2h = (M * K + K * N) * 8, M * N * 8
        else:
            Ad = torch.empty_like(A); Bd = torch.empty((K, N), dtype=torch.float64, device=dev) if rank == 0 else None

            def e2e_step():
                Ad.copy_(Ah, non_blocking=True)
                if rank == 0:
                    Bd.copy_(Bh, non_blocking=True)
                op(Ad, Bd, C)
                Ch.copy_(C, non_blocking=True)
                torch.cuda.synchronize()
            h2d, d2h = (M * K * world + K * N) * 8, M * N * 8 * world
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / args.e2e_steps
        if world > 1:
            t = torch.tensor([dt], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        if world == 1 and not torch.equal(Ch.to(dev), C):
            raise RuntimeError("host-staged result differs from the device-resident result")
        e2e = {"value": flops_step / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": dt * 1e3, "steps": args.e2e_steps}

    # CPU leg (rank 0, one GPU only): baseline timing on a bounded sample, bit parity and error of the GPU result
    cpu = None
    if world == 1 and args.cpu_rows > 0:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as o
        rows = args.cpu_rows
        Bn = B.cpu().numpy()
        An = A[:rows].cpu().numpy()
        Cs, tb, tr = cpu_pipeline_sample(An, Bn, nm)
        t_full = tb + tr * (M / rows)
        same = bool(np.array_equal(Cs.view(np.uint64), C[:rows].cpu().numpy().view(np.uint64)))
        er = min(rows, 32)
        err = o.err_units(An[:er], Bn, Cs[:er])   # Dot2 reference, every entry of the first rows of the sample
        cpu = {"value": 2.0 * M * N * K / t_full / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
               "sample": f"rows 0..{rows - 1} of the product ({tb + tr:.1f} s of CPU work); B's scale/residue pass charged once, "
                         f"per-row work scaled to {M} rows",
               "gpu_rows_bit_identical": same, "bit_checked_entries": rows * N, "max_err_units_2^-53": err, "err_entries": er * N}
        if not same:
            raise RuntimeError("GPU result differs from the CPU checker on the sampled rows")

    if rank == 0:
        line = {
            "metric": "fp64_equiv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if args.strong else "weak", "vs_baseline": None,
            "dtype": "int8 residues / int32 accumulate / f64 in-out", "data": "synthetic",
            "config": {"workload": f"FP64 GEMM n={n}, {nm} moduli (Ozaki-II), entries U[-1,1)*2^e, e in [-8,8]"
                                   + ("" if world == 1 else f"; {world} row blocks of {M} rows (M={M * world}), B broadcast from rank 0 every step"),
                       "moduli": nm, "n": n, "M_total": M * world, "l2": "operands (512 MiB each at n=8192) exceed L2; no flush needed",
                       "parallelism": f"row-block x{world}", "panels": len(op.ranges), "broadcast_layout": op.layout if world > 1 else None},
            "gpu_launches": steps * (5 if world == 1 else (4 + len(op.ranges) if op.layout == "rows" else 2 + 4 * len(op.ranges))),
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "power_w", "reasons", "samples")} if clocks else None,
        }
        if e2e:
            line["e2e"] = e2e
        if roof:
            line["roofline"] = roof
            line["phases_ms"] = {"before_first_gemm": float(phases[0]), "gemm_i8_kernels": float(phases[1]),
                                 "after_last_gemm": float(phases[2]), "product": float(phases[3]),
                                 "note": "CUDA events recorded by the library on the launching stream inside the timed steps (mean over the steps)"}
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", "--n", dest="n", type=int, default=8192, help="n of the n x n x n product (use --size under torchrun)")
    ap.add_argument("--moduli", type=int, default=16)
    ap.add_argument("--panels", type=int, default=None, help="pieces B is broadcast in (N > 1; default: by the size of B)")
    ap.add_argument("--layout", choices=("auto", "rows", "panels"), default="auto", help="broadcast B in row chunks or in column panels (N > 1)")
    ap.add_argument("--strong", action="store_true", help="strong scaling: the n x n x n product is split over the ranks")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-rows", type=int, default=256)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
