"""The rest of the C ABI on the GPU: the plan interface (the reference's oz::plan / oz::dgemm / oz::release), leading
dimensions and streams, phase timing, the built-in benchmark, the tensor-pipe probe, concurrent callers, and a C++ program
written against include/ozaki2.hpp the way the reference's programs use src/ozaki2.cuh (GPU tests)."""
import ctypes
import os
import subprocess
import threading

import numpy as np
import pytest

import oracle_lib as o

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_interface_with_leading_dimensions_and_a_stream():
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, N, K, nm = 150, 270, 333, 15
    A, B = g.synthetic(M, K, 101), g.synthetic(K, N, 102)
    lda, ldb, ldc = K + 7, N + 2, N + 6
    Ad = torch.zeros((M, lda), dtype=torch.float64, device="cuda"); Ad[:, :K] = g.dev(A)
    Bd = torch.zeros((K, ldb), dtype=torch.float64, device="cuda"); Bd[:, :N] = g.dev(B)
    Cd = torch.full((M, ldc), 7.0, dtype=torch.float64, device="cuda")
    plan = ctypes.c_void_p()
    g.check(lib.ozb_plan_create(M, N, K, nm, 62, ctypes.byref(plan)))
    bits, kp, np_ = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    ptrs = [ctypes.c_void_p() for _ in range(5)]
    g.check(lib.ozb_plan_view(plan, ctypes.byref(bits), ctypes.byref(kp), ctypes.byref(np_), *[ctypes.byref(p) for p in ptrs]))
    assert bits.value == o.bits_for(nm, K) and kp.value >= K and np_.value >= N and all(p.value for p in ptrs)
    stream = torch.cuda.Stream()
    g.check(lib.ozb_plan_profile(plan, 2))
    with torch.cuda.stream(stream):
        for _ in range(3):
            g.check(lib.ozb_plan_dgemm(plan, g.ptr(Ad), lda, g.ptr(Bd), ldb, g.ptr(Cd), ldc, ctypes.c_void_p(stream.cuda_stream)))
    g.check(lib.ozb_plan_status(plan))                      # synchronises the stream
    want = o.dgemm(A, B, nm)
    assert g.same_bits(Cd[:, :N].cpu().numpy(), want)
    assert torch.all(Cd[:, N:] == 7.0)                      # nothing written past column N
    ms = (ctypes.c_float * 4)()
    g.check(lib.ozb_plan_phase_ms(plan, 0, ctypes.byref(ms)))
    assert ms[3] > 0 and abs(ms[0] + ms[1] + ms[2] - ms[3]) <= 0.05 * ms[3] + 0.02
    assert lib.ozb_plan_phase_ms(plan, 5, ctypes.byref(ms)) == 10001
    km = (ctypes.c_float * 5)()                            # the same product kernel by kernel: the five parts add up to it
    g.check(lib.ozb_plan_kernel_ms(plan, 0, ctypes.byref(km)))
    assert all(t > 0 for t in km) and abs(sum(km) - ms[3]) <= 0.02 * ms[3] + 0.02
    assert abs(km[0] + km[1] + km[2] - ms[0]) <= 0.02 and abs(km[3] - ms[1]) <= 0.02 and abs(km[4] - ms[2]) <= 0.02
    assert lib.ozb_plan_kernel_ms(plan, 5, ctypes.byref(km)) == 10001
    # the split form: residues of A once, then two column panels
    Cd.fill_(0)
    g.check(lib.ozb_plan_set_a(plan, g.ptr(Ad), lda, None))
    g.check(lib.ozb_plan_panel(plan, ctypes.c_void_p(Bd.data_ptr() + 8 * 256), ldb, ctypes.c_void_p(Cd.data_ptr() + 8 * 256), ldc, 256, N - 256, None))
    g.check(lib.ozb_plan_panel(plan, g.ptr(Bd), ldb, g.ptr(Cd), ldc, 0, 256, None))
    g.check(lib.ozb_plan_status(plan))
    assert g.same_bits(Cd[:, :N].cpu().numpy(), want)
    assert lib.ozb_plan_panel(plan, g.ptr(Bd), ldb, g.ptr(Cd), ldc, 100, 50, None) == 10001    # panels start on multiples of 256
    # B in chunks of rows, delivered out of order; then the prepared B with a second A
    Cd.fill_(0)
    g.check(lib.ozb_plan_b_begin(plan, None))
    for k0, rows in ((200, K - 200), (0, 77), (77, 123)):
        g.check(lib.ozb_plan_b_rows(plan, ctypes.c_void_p(Bd.data_ptr() + 8 * ldb * k0), ldb, rows, None))
    g.check(lib.ozb_plan_b_finish(plan, g.ptr(Bd), ldb, None))
    g.check(lib.ozb_plan_multiply(plan, g.ptr(Cd), ldc, None))
    g.check(lib.ozb_plan_status(plan))
    assert g.same_bits(Cd[:, :N].cpu().numpy(), want)
    A2 = g.synthetic(M, K, 103)
    Ad[:, :K] = g.dev(A2)
    g.check(lib.ozb_plan_set_a(plan, g.ptr(Ad), lda, None))
    g.check(lib.ozb_plan_multiply(plan, g.ptr(Cd), ldc, None))
    g.check(lib.ozb_plan_status(plan))
    assert g.same_bits(Cd[:, :N].cpu().numpy(), o.dgemm(A2, B, nm))
    assert lib.ozb_plan_b_rows(plan, g.ptr(Bd), ldb, K + 1, None) == 10001
    # the column maxima first (as their holder would send them ahead), then B in chunks of rows starting on multiples of 128
    Cd.fill_(0)
    colmax = torch.zeros(N, dtype=torch.int64, device="cuda")
    g.check(lib.ozb_cols_absmax(g.ptr(Bd), K, N, ldb, g.ptr(colmax), None))
    assert np.array_equal(colmax.cpu().numpy(), np.abs(B).max(axis=0).view(np.int64))
    for k0, rows in ((256, K - 256), (0, 128), (128, 128)):
        g.check(lib.ozb_plan_b_rows_residues(plan, ctypes.c_void_p(Bd.data_ptr() + 8 * ldb * k0), ldb, k0, rows, g.ptr(colmax), None))
    g.check(lib.ozb_plan_multiply(plan, g.ptr(Cd), ldc, None))
    g.check(lib.ozb_plan_status(plan))
    assert g.same_bits(Cd[:, :N].cpu().numpy(), o.dgemm(A2, B, nm))
    assert lib.ozb_plan_b_rows_residues(plan, g.ptr(Bd), ldb, 100, 28, g.ptr(colmax), None) == 10001
    lib.ozb_plan_destroy(plan)


def test_dgemm_ex_and_builtin_benchmark_and_probe():
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    M, N, K = 96, 128, 200
    A, B = g.synthetic(M, K, 103), g.synthetic(K, N, 104)
    Ad, Bd = g.dev(A), g.dev(B)
    Cd = torch.empty((M, N), dtype=torch.float64, device="cuda")
    g.check(lib.ozb_dgemm_ex(M, N, K, g.ptr(Ad), K, g.ptr(Bd), N, g.ptr(Cd), N, 16, None))
    torch.cuda.synchronize()
    assert g.same_bits(Cd.cpu().numpy(), o.dgemm(A, B, 16))
    ms = ctypes.c_double()
    g.check(lib.ozb_bench(1024, 0, 3, ctypes.byref(ms)))
    assert 0 < ms.value < 1000
    assert lib.ozb_bench(1024, 0, 0, ctypes.byref(ms)) == 10001 and lib.ozb_bench(1024, 3, 1, ctypes.byref(ms)) == 10001
    assert lib.ozb_bench(1024, 2, 1, ctypes.byref(ms)) == 10005          # triple-double: exported, not built
    t, tops = ctypes.c_float(), ctypes.c_double()
    for pair in (0, 1):
        g.check(lib.ozb_int8_peak(2000, pair, ctypes.byref(t), ctypes.byref(tops)))
        assert 500 < tops.value < 6000                                    # an INT8 tensor rate, in TOP/s
    name = ctypes.create_string_buffer(64)
    sm, l2, sms = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    g.check(lib.ozb_device(name, 64, ctypes.byref(sm), ctypes.byref(l2), ctypes.byref(sms)))
    assert sm.value // 10 == 10 and l2.value > 0 and sms.value > 0
    g.check(lib.ozb_device(None, 0, None, None, None))                    # NULL-tolerant, as the reference's


def test_two_threads_call_at_once():
    """ctypes releases the GIL; the library serialises callers with one mutex (python/capi.cu:19 of the reference)."""
    import gpu_util as g
    shapes = [(120, 90, 300, 16), (64, 200, 129, 12)]
    data = [(g.synthetic(M, K, 110 + i), g.synthetic(K, N, 120 + i), nm) for i, (M, N, K, nm) in enumerate(shapes)]
    out = [None, None]

    def work(i):
        A, B, nm = data[i]
        for _ in range(5):
            out[i] = g.gpu_dgemm(A, B, nm, on_host=True)

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in th]
    [t.join() for t in th]
    for i, (A, B, nm) in enumerate(data):
        assert g.same_bits(out[i], o.dgemm(A, B, nm))


def test_cpp_program_against_the_header(tmp_path):
    import gpu_util as g
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "cpp_caller")
    libdir = os.path.join(ROOT, "ozaki_blackwell_b200")
    subprocess.run(["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
                    os.path.join(ROOT, "tests", "cpp_caller.cpp"), "-o", exe, "-L", libdir, "-l:libozaki_blackwell.so",
                    "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"],
                   check=True)
    M, N, K, nm = 130, 70, 260, 14
    A, B = g.synthetic(M, K, 130), g.synthetic(K, N, 131)
    A.tofile(tmp_path / "a.bin"); B.tofile(tmp_path / "b.bin")
    r = subprocess.run([exe, str(M), str(N), str(K), str(nm), str(tmp_path / "a.bin"), str(tmp_path / "b.bin"), str(tmp_path / "c.bin")],
                       capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stdout + r.stderr
    C = np.fromfile(tmp_path / "c.bin").reshape(M, N)
    assert g.same_bits(C, o.dgemm(A, B, nm))


def test_an_expired_wait_is_reported_and_the_context_survives():
    """The failure path of the GEMM kernel's bounded waits, without any fault: a wait that nothing will satisfy runs out of
    its (short) budget, the status word is raised, the call returns OZB_ETIMEOUT, and the next product is correct."""
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    assert lib.ozb_selftest_wait_expiry(50) == 10004
    assert b"wait" in lib.ozb_error(10004)
    assert lib.ozb_status() == 0                                  # reading the status cleared it
    assert lib.ozb_selftest_wait_expiry(0) == 10001
    A, B = g.synthetic(64, 96, 140), g.synthetic(96, 80, 141)
    assert g.same_bits(g.gpu_dgemm(A, B, 16), o.dgemm(A, B, 16))
