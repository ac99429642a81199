#!/usr/bin/env python
"""Benchmark of the Ozaki-II FP64 product on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size 8192] [--moduli 16]

One step = one FP64-accurate product C = A B with 16 moduli on seeded synthetic matrices (entries U[-1,1) * 2^e, e a
uniform integer in [-8, 8]). At N = 1 the workload is n = 8192 (M = N = K = n). At N > 1 (one process per GPU, launched
by torch.distributed.run) rank g owns n rows of A and of C, B lives on rank 0 and is broadcast over NCCL inside every
step (weak scaling: M = n * N in total). Rank 0 prints one JSON line.

  value        FP64-equivalent TFLOP/s (2 M N K / time), operands resident in HBM, CUDA events, max over ranks
  e2e          the same from pinned host operands, host<->device copies inside the timed region: through the reference's
               entry point ozb_dgemm(on_host = 1) at N = 1, through the sharded host-operand path at N > 1
  roofline     the INT8 GEMM kernel: 2 nm M N K integer operations / its event-timed duration inside the same timed steps,
               against twice the measured dense bf16 rate (the tensor cores run INT8 at twice the bf16 rate)
  roofline_hbm the scale / residue / reconstruction kernels: algorithmic bytes / event-timed duration in the same steps,
               against the measured copy bandwidth
  baselines    outside the timed region, same operands: the reference's own kernels compiled for this GPU, and cuBLAS DGEMM
  cpu_baseline the CPU restatement of the reference's pipeline on the host cores, on a bounded sample; the same leg
               bit-compares the GPU result with it
  strong_n32768  BASELINE's large configuration: one n = 32768 product split by row blocks over the N ranks
  ranks_bit_identical  (N > 1) every rank's band of C against the CPU restatement
--rows R gives every rank R rows of A and C whatever N is (with --strong --size 32768 --rows 4096: the share a rank of
eight holds, run on fewer GPUs); e2e.ms_last_step_per_rank shows which rank the host link holds up.
--impl reference times that CPU restatement alone (the reference has no CPU implementation of the Ozaki pipeline of its
own: its device code is restated in oracle/ozaki2_oracle.c), rank 0 only, on a block sample of the product per step.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SPREAD = 8
PEAKS_FILE = os.path.join(ROOT, "MEASURED_PEAKS.json")
FALLBACK = {"bf16": 1400.0, "bf16_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}
NOMINAL_INT8_TOPS = 4500.0
DTYPE = "int8 residues / int32 accumulate / f64 in-out"


def peaks():
    try:
        with open(PEAKS_FILE) as f:
            p = json.load(f)
        return {"bf16": float(p["bf16_tflops_sustained"]), "bf16_burst": float(p["bf16_tflops"]), "hbm": float(p["hbm_gbs"]),
                "source": "measured"}
    except Exception:
        return dict(FALLBACK)


def workload_config(n, nm, world):
    """The `config` object: the same in both arms for the same flags."""
    return {"workload": f"FP64 GEMM n={n}, {nm} moduli (Ozaki-II), entries U[-1,1)*2^e, e in [-{SPREAD},{SPREAD}], seeded; "
                        f"{world} row block(s) of {n} rows, B on rank 0",
            "moduli": nm, "n": n, "M_total": n * world, "parallelism": f"row-block x{world}",
            "l2": "operands (512 MiB each at n=8192) exceed L2; no flush needed"}


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
    x = torch.rand((rows, cols), dtype=torch.float64, device=device, generator=g)
    x.mul_(2.0).sub_(1.0)
    e = torch.randint(-SPREAD, SPREAD + 1, (rows, cols), device=device, generator=g, dtype=torch.int32)
    return torch.ldexp(x, e, out=x)


def oracle():
    """The CPU checker (test infrastructure): imported only by the legs that time it or check against it."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as o
    return o


# ---------------------------------------------------------------------------------------------------------------
# CPU legs: the checker's pipeline on the host cores (bounded samples)
# ---------------------------------------------------------------------------------------------------------------
def cpu_block_sample(A_rows, B_cols, nm):
    """The CPU restatement on a rows x cols block of the product (all of K). Returns (C_block, t_b, t_a, t_gemm_crt): the
    scale/residue pass over the sampled columns of B, over the sampled rows of A, and the INT8 GEMMs + reconstruction."""
    import numpy as np
    o = oracle()
    rows, K = A_rows.shape
    cols = B_cols.shape[1]
    bits = o.bits_for(nm, K)
    t0 = time.perf_counter()
    sb = o.scales(B_cols, cols, K, 1, cols, bits)
    Br = o.residues(B_cols, cols, K, 1, cols, sb, nm)
    t1 = time.perf_counter()
    sa = o.scales(A_rows, rows, K, K, 1, bits)
    Ar = o.residues(A_rows, rows, K, K, 1, sa, nm)
    t2 = time.perf_counter()
    Cl = np.stack([o.gemm_i8(Ar[l], Br[l]) for l in range(nm)])
    C = o.crt(Cl, sa, sb)
    t3 = time.perf_counter()
    return C, t1 - t0, t2 - t1, t3 - t2


def full_product_seconds(tb, ta, tg, rows, cols, M, N):
    """Block timings scaled to the whole M x N product: B's pass once over all N columns, A's over all M rows, the GEMMs
    and the reconstruction over all M N outputs."""
    return tb * (N / cols) + ta * (M / rows) + tg * (M / rows) * (N / cols)


def run_reference(args):
    """The reference arm: the CPU restatement of the pipeline with every host thread, rank 0 only. A step is one block of
    the product (rows x cols outputs over the whole of K), sized during the warm-up so that a step takes about a second;
    the value is the block's time scaled to the whole product, and the line says so."""
    import numpy as np
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, args.gpus)
    n, nm = args.n, args.moduli
    o = oracle()
    cores = o.set_threads(os.cpu_count() or 1)      # launchers export OMP_NUM_THREADS=1 to their children
    rng = np.random.default_rng(0)
    rows, cols = 16, min(n, 512)

    def operands(r, c):
        A = np.ldexp(rng.uniform(-1, 1, (r, n)), rng.integers(-SPREAD, SPREAD + 1, (r, n)).astype(np.int32))
        B = np.ldexp(rng.uniform(-1, 1, (n, c)), rng.integers(-SPREAD, SPREAD + 1, (n, c)).astype(np.int32))
        return A, B

    A, B = operands(rows, cols)
    target, t_wall0 = 1.0, time.perf_counter()
    for _ in range(6):                               # size the sample: grow until a step takes about `target` seconds
        t0 = time.perf_counter()
        cpu_block_sample(A, B, nm)
        dt = time.perf_counter() - t0
        if dt >= 0.6 * target or (rows >= 256 and cols >= n):
            break
        grow = min(4.0, target / max(dt, 1e-3))
        if rows < 256 and grow >= 2:
            rows = min(256, rows * 2)
            grow /= 2
        if grow >= 2 and cols < n:
            cols = min(n, cols * (4 if grow >= 4 else 2))
        A, B = operands(rows, cols)
    times, sample_s = [], []
    for s in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        _, tb, ta, tg = cpu_block_sample(A, B, nm)
        if s >= args.warmup:
            times.append(full_product_seconds(tb, ta, tg, rows, cols, n * world, n))
            sample_s.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    val = 2.0 * n * n * n * world / t / 1e12
    sample = (f"a {rows} x {cols} block of the {n * world} x {n} product over all of K per step ({statistics.mean(sample_s):.2f} s of CPU work); "
              f"scaled to the whole product: B's pass by N/{cols}, A's by M/{rows}, GEMMs + reconstruction by both")
    print(json.dumps({
        "impl": "reference", "metric": "fp64_equiv_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": workload_config(n, nm, world),
        "extrapolated": True, "sample_ms_per_step": statistics.mean(sample_s) * 1e3, "rows_timed": rows, "cols_timed": cols,
        "wall_s": time.perf_counter() - t_wall0,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------
class Bench:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from ozaki_blackwell_b200._lib import lib
        self.torch, self.dist, self.lib, self.args = torch, dist, lib, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU path"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream()

    def check(self, code):
        if code:
            raise RuntimeError(self.lib.ozb_error(code).decode())

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, step, steps, warm, sampler=None):
        """`warm` untimed steps, then exactly `steps` steps between barriers, CUDA events on the launching stream, the
        maximum over the ranks. Returns ms per step."""
        torch = self.torch
        for _ in range(warm):
            step()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.mark_start()
        e0.record(self.stream)
        for _ in range(steps):
            step()
        e1.record(self.stream)
        self.barrier()
        if sampler:
            sampler.mark_end()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    # -- bit parity of a band of every rank's rows against the CPU restatement ---------------------------------
    def ranks_bit_identical(self, A, B, C, nm, rows=16, cols=512):
        """Every rank recomputes rows [r0, r0 + rows) x columns [c0, c0 + cols) of its block of C with the CPU restatement
        (an output column needs only its own column of B, an output row only its own row of A) and compares bit for bit.
        The bands differ from rank to rank. B's columns come from rank 0's own tensor, not from the product's staging."""
        import numpy as np
        torch, dist = self.torch, self.dist
        o = oracle()
        o.set_threads(max(1, (os.cpu_count() or 1) // self.world))
        M, K = A.shape
        N = C.shape[1]
        rows, cols = min(rows, M), min(cols, N)
        c0s = [((7 * r + 3) * cols) % max(1, N - cols + 1) for r in range(self.world)]
        r0 = (37 * self.rank + 11) % max(1, M - rows + 1)
        if self.world > 1:
            slab = torch.empty((self.world, K, cols), dtype=torch.float64, device=self.dev)
            if self.rank == 0:
                for r, c0 in enumerate(c0s):
                    slab[r].copy_(B[:, c0:c0 + cols])
            dist.broadcast(slab, src=0)
            Bn = slab[self.rank].cpu().numpy()
        else:
            Bn = B[:, c0s[0]:c0s[0] + cols].cpu().numpy()
        c0 = c0s[self.rank]
        An = A[r0:r0 + rows].cpu().numpy()
        want = o.dgemm(An, Bn, nm)
        got = C[r0:r0 + rows, c0:c0 + cols].cpu().numpy()
        same = bool(np.array_equal(want.view(np.uint64), got.view(np.uint64)))
        err = float(o.err_units(An, Bn, got)) if same else float("nan")
        if self.world == 1:
            return [same], [err], rows * cols
        flags = torch.tensor([1.0 if same else 0.0, err], dtype=torch.float64, device=self.dev)
        allf = [torch.empty_like(flags) for _ in range(self.world)]
        dist.all_gather(allf, flags)
        return [bool(f[0].item() == 1.0) for f in allf], [float(f[1].item()) for f in allf], rows * cols

    # -- the sharded product of this build ----------------------------------------------------------------------
    def sharded(self, M, N, K, nm):
        from ozaki_blackwell_b200.dist import RowShardedGemm
        return RowShardedGemm(M, N, K, nm, panels=self.args.panels, layout=self.args.layout)

    # -- BASELINE's large configuration: one n x n x n product split by row blocks --------------------------------
    def strong_case(self, n, nm, steps, warm):
        torch = self.torch
        from ozaki_blackwell_b200.dist import row_block
        lo, hi = row_block(n, self.rank, self.world)
        M = hi - lo
        A = synthetic(M, n, 5000 + self.rank, self.dev)
        B = synthetic(n, n, 77, self.dev) if self.rank == 0 else None
        C = torch.empty((M, n), dtype=torch.float64, device=self.dev)
        op = self.sharded(M, n, n, nm)
        ms = self.timed(lambda: op(A, B, C), steps, warm)
        op.engine.status()
        same, errs, entries = self.ranks_bit_identical(A, B, C, nm, rows=8, cols=256)
        out = {"n": n, "moduli": nm, "n_gpus": self.world, "rows_per_rank": M, "ms_per_step": ms, "steps": steps, "warmup": warm,
               "value": 2.0 * n * n * n / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "scaling": "strong",
               "broadcast": None if self.world == 1 else {"layout": op.layout, "pieces": len(op.ranges)},
               "ranks_bit_identical": same, "bit_checked_entries_per_rank": entries, "max_err_units_2^-53": max(errs),
               "note": "one n x n x n product, rank g owns rows [g n/N, (g+1) n/N) of A and C, B on rank 0 and broadcast inside every "
                       "step; CUDA events, max over ranks; the speed-up over one GPU is this value over the same key of the N = 1 line"}
        op.close()
        del A, B, C, op
        torch.cuda.empty_cache()
        return out

    # -- the headline run --------------------------------------------------------------------------------------
    def run(self):
        import numpy as np
        torch, lib, args = self.torch, self.lib, self.args
        world, rank, dev, check = self.world, self.rank, self.dev, self.check
        n, nm = args.n, args.moduli
        N = K = n
        M = n // world if args.strong else n            # rows of A and C per rank (weak: n each; --strong: n in total)
        if args.rows > 0:
            M = args.rows                               # a chosen share per rank: what a rank of a larger job would hold
        A = synthetic(M, K, 1000 + rank, dev)
        B = synthetic(K, N, 7, dev) if rank == 0 else None
        C = torch.empty((M, N), dtype=torch.float64, device=dev)
        steps, warm = args.steps, args.warmup
        pk = peaks()
        sampler = ClockSampler(self.local)
        if rank == 0:
            sampler.start()

        plan, op = None, None
        if world == 1:
            plan = ctypes.c_void_p()
            check(lib.ozb_plan_create(M, N, K, nm, 62, ctypes.byref(plan)))
            check(lib.ozb_plan_profile(plan, steps))
            sp = ctypes.c_void_p(self.stream.cuda_stream)

            def step():
                check(lib.ozb_plan_dgemm(plan, A.data_ptr(), K, B.data_ptr(), N, C.data_ptr(), N, sp))
            for _ in range(warm):
                step()
            self.barrier()
            check(lib.ozb_plan_profile(plan, steps))      # restart the slot counter after the warm-up
            ms_step = self.timed(step, steps, 0, sampler)
            check(lib.ozb_plan_status(plan))
            launches = steps * 5
        else:
            op = self.sharded(M, N, K, nm)

            def step():
                op(A, B, C)
            ms_step = self.timed(step, steps, warm, sampler)
            op.engine.status()
            if op.native:
                launches = steps * op.native.kernels          # rank 0's kernels per product, counted by the library
            else:
                launches = steps * (4 + len(op.ranges) if op.layout == "rows" else 2 + 4 * len(op.ranges))
        clocks = sampler.stop() if rank == 0 else None
        flops_step = 2.0 * M * N * K * world
        value = flops_step / (ms_step * 1e-3) / 1e12

        # kernels of the same timed steps (single GPU: events recorded inside the library on the launching stream)
        roof = hbm = kernels_ms = None
        if world == 1:
            ph = np.zeros((steps, 5))
            buf = (ctypes.c_float * 5)()
            for s in range(steps):
                check(lib.ozb_plan_kernel_ms(plan, s, ctypes.byref(buf)))
                ph[s] = list(buf)
            t_rows, t_absmax, t_cols, t_gemm, t_crt = ph.mean(axis=0)
            kernels_ms = {"row_scale_residues": t_rows, "col_absmax": t_absmax, "col_residues_t": t_cols, "gemm_i8_tc2": t_gemm,
                          "crt_kernel": t_crt, "sum": float(ph.mean(axis=0).sum()), "product": ms_step,
                          "note": "CUDA events recorded by the library on the launching stream around each kernel inside the timed steps (mean)"}
            ops = 2.0 * nm * M * N * K
            achieved = ops / (t_gemm * 1e-3) / 1e12
            # An INT8 figure this GPU reaches with nothing but tcgen05.mma running (the library's probe), reported beside the
            # roofline: a burst of about a millisecond and a run of about 0.1 s, after which the power limit has pulled the clock down.
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
            alg_bytes = nm * (M * K + N * K + M * N)
            traffic, traffic_how = gemm_traffic(n, nm, alg_bytes)
            peak = 2.0 * pk["bf16"]
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": traffic, "traffic_how": traffic_how, "algorithmic_bytes": alg_bytes,
                    "kernel": "gemm_i8_tc2<fused mod> (tcgen05.mma cta_group::2 kind::i8)",
                    "peak_how": f"2 x dense bf16 sustained of MEASURED_PEAKS.json ({pk['source']}): the kernel is timed inside long steps",
                    "peak_burst": 2.0 * pk["bf16_burst"], "frac_of_burst": achieved / (2.0 * pk["bf16_burst"]),
                    "peak_nominal": NOMINAL_INT8_TOPS, "frac_of_nominal": achieved / NOMINAL_INT8_TOPS,
                    "int8_probe_tops": probe,
                    "frac_of_probe_sustained": achieved / probe["sustained_cta_pair"],
                    "note": "INT8 tera-operations/s (2 per multiply-add). cuBLAS bf16 itself runs below the tensor pipe's limit, so a "
                            "fraction above 1 of twice its rate is expected; int8_probe_tops is this GPU's tcgen05.mma-only rate "
                            "(1 ms burst and 0.1 s sustained under the power limit), measured in this run"}
            gb = 1e-9
            def entry(name, t_ms, nbytes, what):
                a = nbytes * gb / (t_ms * 1e-3)
                return {"kernel": name, "bound": "hbm", "achieved": a, "peak": pk["hbm"], "unit": "GB/s", "frac": a / pk["hbm"],
                        "ms": float(t_ms), "algorithmic_bytes": nbytes, "bytes": what}
            hbm = [entry("row_scale_residues<16>", t_rows, (8 + nm) * M * K, "8 M K read + nm M K written"),
                   entry("col_absmax", t_absmax, 8 * K * N, "8 K N read"),
                   entry("col_residues_t<16>", t_cols, (8 + nm) * K * N, "8 K N read + nm K N written"),
                   entry("crt_kernel<16,int8>", t_crt, (nm + 8) * M * N, "nm M N read + 8 M N written")]

        # the same operands through the reference's own kernels and through cuBLAS DGEMM, outside the timed region
        baselines = self.baselines(A, B, C, nm) if world == 1 and not args.no_baselines else None

        # end to end from pinned host memory
        e2e = None
        if args.e2e_steps > 0:
            e2e = self.e2e(A, B, C, M, N, K, nm, op, flops_step)

        # parity: every rank's band against the CPU restatement (N > 1); the CPU baseline leg does it at N = 1
        parity = None
        if world > 1:
            same, errs, entries = self.ranks_bit_identical(A, B, C, nm)
            parity = {"ranks_bit_identical": same, "bit_checked_entries_per_rank": entries, "max_err_units_2^-53": max(errs)}
            if not all(same):
                raise RuntimeError(f"rows of C differ from the CPU checker on ranks {[r for r, s in enumerate(same) if not s]}")

        # CPU leg (one GPU only): baseline timing on a bounded sample, bit parity and error of the GPU result
        cpu = None
        if world == 1 and args.cpu_rows > 0:
            o = oracle()
            cores = o.set_threads(os.cpu_count() or 1)
            rows, cols = args.cpu_rows, min(N, args.cpu_cols)
            Bn = B[:, :cols].cpu().numpy()
            An = A[:rows].cpu().numpy()
            Cs, tb, ta, tg = cpu_block_sample(An, Bn, nm)
            t_full = full_product_seconds(tb, ta, tg, rows, cols, M, N)
            same = bool(np.array_equal(Cs.view(np.uint64), C[:rows, :cols].cpu().numpy().view(np.uint64)))
            er = min(rows, 32)
            err = o.err_units(An[:er], Bn, Cs[:er])   # Dot2 reference, every entry of the first rows of the sample
            if baselines and getattr(self, "cublas_rows", None) is not None:
                baselines["cublas_dgemm"]["max_err_units_2^-53"] = o.err_units(An[:er], Bn, np.ascontiguousarray(self.cublas_rows[:er, :cols]))
            cpu = {"value": 2.0 * M * N * K / t_full / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                   "sample": f"the {rows} x {cols} block of the product at the origin, all of K ({tb + ta + tg:.1f} s of CPU work); scaled to "
                             f"the whole product: B's pass by N/{cols}, A's by M/{rows}, GEMMs + reconstruction by both",
                   "gpu_block_bit_identical": same, "bit_checked_entries": rows * cols, "max_err_units_2^-53": err, "err_entries": er * cols}
            if not same:
                raise RuntimeError("GPU result differs from the CPU checker on the sampled block")

        config = workload_config(n, nm, world)
        if M != n:
            config["workload"] = config["workload"].replace(f"{world} row block(s) of {n} rows", f"{world} row block(s) of {M} rows")
            config["M_total"] = M * world
        dist_info = None if world == 1 else {"broadcast_layout": op.layout, "pieces": len(op.ranges)}
        if plan is not None:
            lib.ozb_plan_destroy(plan)
        if op is not None:
            op.close()
        del A, B, C
        lib.ozb_release()
        torch.cuda.empty_cache()

        strong = None
        if args.strong_size > 0 and not args.strong:
            try:
                strong = self.strong_case(args.strong_size, nm, args.strong_steps, 1)
            except Exception as exc:       # the headline line is still printed; the key then says what went wrong
                strong = {"n": args.strong_size, "n_gpus": world, "error": f"{type(exc).__name__}: {exc}"[:300]}

        if rank == 0:
            line = {
                "metric": "fp64_equiv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warm,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if args.strong else "weak", "vs_baseline": None,
                "dtype": DTYPE, "data": "synthetic", "config": config, "gpu_launches": launches,
                "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "power_w", "reasons", "samples")} if clocks else None,
            }
            if dist_info:
                line["broadcast"] = dist_info
            if e2e:
                line["e2e"] = e2e
            if roof:
                line["roofline"] = roof
                line["roofline_hbm"] = hbm
                line["kernels_ms"] = {k: (float(v) if not isinstance(v, str) else v) for k, v in kernels_ms.items()}
            if baselines:
                line["baselines"] = baselines
            if cpu:
                line["cpu_baseline"] = cpu
            if parity:
                line.update(parity)
            if strong:
                line[f"strong_n{args.strong_size}"] = strong
            print(json.dumps(line))
        if world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()

    def baselines(self, A, B, C, nm):
        """The reference's own device code (python/capi.cu of the reference compiled unmodified for sm_100a, when that
        build is present) and cuBLAS DGEMM (torch.matmul in float64) on the same operands: median of 5 after a warm-up."""
        torch, lib = self.torch, self.lib
        n = A.shape[0]
        R = torch.empty_like(C)

        def med(fn, reps=5):
            fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                fn()
                e1.record(self.stream)
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts)
        fl = 2.0 * n ** 3 / 1e9
        out = {}
        t = med(lambda: torch.matmul(A, B, out=R))
        out["cublas_dgemm"] = {"ms": t, "tflops": fl / t, "what": "torch.matmul in float64 (cuBLAS DGEMM, native FP64)"}
        self.cublas_rows = R[:32].cpu().numpy()          # its error is measured by the CPU leg on the same block as this library's
        ref_path = os.path.join(ROOT, "oracle", "_ref", "libozb_ref.so")
        if os.path.exists(ref_path):
            ref = ctypes.CDLL(ref_path)
            ref.ozb_dgemm.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2

            def theirs():
                rc = ref.ozb_dgemm(n, n, n, A.data_ptr(), B.data_ptr(), R.data_ptr(), nm, 0)
                if rc:
                    raise RuntimeError(f"the reference's ozb_dgemm returned {rc}")
            t = med(theirs)
            same = bool(torch.equal(C.view(torch.int64), R.view(torch.int64)))
            ref.ozb_release()
            out["reference_kernels_sm100a"] = {"ms": t, "tflops": fl / t, "same_bits_as_this_library": same,
                                               "what": "the reference's python/capi.cu (mma.sync GEMM and its own scale/residue/CRT kernels) "
                                                       "compiled unmodified for sm_100a, ozb_dgemm on the same device operands"}
        else:
            out["reference_kernels_sm100a"] = {"unavailable": "oracle/_ref/libozb_ref.so is not built on this machine"}
        del R
        return out

    def e2e(self, A, B, C, M, N, K, nm, op, flops_step):
        torch, lib, world, rank, dev = self.torch, self.lib, self.world, self.rank, self.dev
        steps = self.args.e2e_steps
        Ah = torch.empty((M, K), dtype=torch.float64, pin_memory=True); Ah.copy_(A)
        Bh = None
        if rank == 0:
            Bh = torch.empty((K, N), dtype=torch.float64, pin_memory=True); Bh.copy_(B)
        Ch = torch.empty((M, N), dtype=torch.float64, pin_memory=True)
        if world == 1:
            def e2e_step():
                self.check(lib.ozb_dgemm(M, N, K, Ah.data_ptr(), Bh.data_ptr(), Ch.data_ptr(), nm, 1))
            h2d, d2h = (M * K + K * N) * 8, M * N * 8
            how = "ozb_dgemm(on_host=1): the reference's entry point, pinned host operands, block-pipelined copies inside"
        else:
            if not op.native:
                return None                       # host operands go through the library's own multi-GPU layer only

            def e2e_step():
                op.host(Ah, Bh, Ch)               # synchronous: returns when this rank's rows of C are back in host memory
            h2d, d2h = (M * K * world + K * N) * 8, M * N * 8 * world
            how = ("ozb_mg_dgemm(on_host=1) on every rank: B goes to rank 0's GPU in pieces that are broadcast as they land, every "
                   "rank's rows of A and C travel in blocks beside the computation")
        e2e_step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        self.barrier()
        own = (time.perf_counter() - t0) / steps
        dt = self.max_over_ranks(own)
        # each rank's own time per step, without the closing barrier of the other ranks: shows which rank the host link holds up
        t1 = time.perf_counter()
        e2e_step()
        alone = torch.tensor([(time.perf_counter() - t1) * 1e3], dtype=torch.float64, device=dev)
        per_rank = [alone.clone() for _ in range(world)]
        if world > 1:
            self.dist.all_gather(per_rank, alone)
        if not torch.equal(Ch.to(dev), C):
            raise RuntimeError(f"rank {rank}: the host-staged result differs from the device-resident result")
        return {"value": flops_step / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": dt * 1e3, "steps": steps, "ms_last_step_per_rank": [round(float(t.item()), 3) for t in per_rank],
                "how": how}


def gemm_traffic(n, nm, alg_bytes):
    """DRAM bytes of one GEMM launch from the profiler capture recorded with the package (one launch of this kernel under
    ncu: dram__bytes_read.sum + dram__bytes_write.sum). The capture of this very workload is used as it is; for another
    size the captured ratio of DRAM bytes to algorithmic bytes is applied, and the line says so."""
    try:
        with open(os.path.join(ROOT, "ozaki_blackwell_b200", "ncu_captures.json")) as f:
            caps = json.load(f)["gemm_i8_tc2"]
    except Exception:
        return None, "no capture recorded"
    for c in caps:
        if c["n"] == n and c["moduli"] == nm:
            return float(c["dram_bytes"]), f"measured: one ncu capture of this kernel at this workload ({c['when']})"
    c = max(caps, key=lambda c: c["n"])
    ratio = c["dram_bytes"] / (c["moduli"] * 3.0 * c["n"] ** 2)
    return ratio * alg_bytes, f"estimated: scaled by algorithmic bytes from the ncu capture at n={c['n']}, {c['moduli']} moduli"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", "--n", dest="n", type=int, default=8192, help="n of the n x n x n product (use --size under torchrun)")
    ap.add_argument("--moduli", type=int, default=16)
    ap.add_argument("--spread", type=int, default=8, help="entries U[-1,1) * 2^e with e uniform in [-spread, spread] (0: plain U[-1,1))")
    ap.add_argument("--panels", type=int, default=None, help="pieces B is broadcast in (N > 1; default: by the size of B)")
    ap.add_argument("--layout", choices=("auto", "rows", "panels"), default="auto", help="broadcast B in row chunks or in column panels (N > 1)")
    ap.add_argument("--strong", action="store_true", help="make the headline run itself a strong split of the n x n x n product")
    ap.add_argument("--rows", type=int, default=0, help="rows of A and C per rank, whatever N is (e.g. 4096 with --size 32768: a rank's share at eight GPUs)")
    ap.add_argument("--strong-size", type=int, default=32768, help="n of the strong-scaling case reported beside the headline (0: skip)")
    ap.add_argument("--strong-steps", type=int, default=3)
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--cpu-rows", type=int, default=256, help="rows of the CPU baseline's block sample (0: skip the leg)")
    ap.add_argument("--cpu-cols", type=int, default=4096, help="columns of the CPU baseline's block sample")
    ap.add_argument("--no-baselines", action="store_true", help="skip the reference-kernels and cuBLAS legs")
    args = ap.parse_args()
    global SPREAD
    SPREAD = args.spread
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)
    if args.impl == "reference":
        run_reference(args)
    else:
        Bench(args).run()


if __name__ == "__main__":
    main()
