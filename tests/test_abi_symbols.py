"""The shared library loads without a GPU and exports every function include/ozb.h declares; the calls that can answer
without a device answer as the reference's do (no compute is attempted here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ozb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ozb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    from ozaki_blackwell_b200._lib import lib, SYMBOLS
    names = _declared()
    assert len(names) >= 30 and {"ozb_version", "ozb_error", "ozb_device", "ozb_dgemm", "ozb_ddgemm", "ozb_tdgemm", "ozb_release",
                                 "ozb_bench"} <= set(names)          # the reference's eight (python/capi.cu:52-164)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert set(SYMBOLS) == set(names), set(SYMBOLS) ^ set(names)     # the binding lists exactly what the header declares


def test_calls_that_need_no_device():
    from ozaki_blackwell_b200._lib import lib
    assert lib.ozb_version().decode().startswith("0.")
    assert lib.ozb_error(0) == b"ok"
    assert b"131072" in lib.ozb_error(10002) and b"positive" in lib.ozb_error(10001)
    assert lib.ozb_modulus(0) == 256 and lib.ozb_modulus(15) == 193 and lib.ozb_modulus(48) == 29 and lib.ozb_modulus(49) == 0
    assert lib.ozb_bits_for(16, 512, 62) == 57 and lib.ozb_bits_for(16, 8192, 62) == 55 and lib.ozb_bits_for(16, 131072, 62) == -1
    z = ctypes.c_void_p(0)
    assert lib.ozb_dgemm(0, 1, 1, z, z, z, 16, 0) == 10001            # argument checks come before any device work
    assert lib.ozb_dgemm(4, 4, 131072, z, z, z, 16, 0) == 10002


def test_multi_gpu_entry_points_check_their_arguments_first():
    """The argument checks of the multi-GPU layer come before any device or NCCL work, as the reference's do
    (python/capi.cu:23-29,79 for ozb_dgemm, whose shape ozb_dgemm_mg extends)."""
    from ozaki_blackwell_b200._lib import lib
    one = ctypes.c_void_p(16)                                         # never dereferenced
    h = ctypes.c_void_p()
    assert lib.ozb_dgemm_mg(0, 4, 4, one, one, one, 16, 1, 2) == 10001
    assert lib.ozb_dgemm_mg(4, 4, 4, one, one, one, 7, 1, 2) == 10001
    assert lib.ozb_dgemm_mg(4, 4, 4, one, one, one, 16, 1, 0) == 10001   # device count 1..16
    assert lib.ozb_dgemm_mg(4, 4, 4, one, None, one, 16, 1, 2) == 10001
    assert lib.ozb_dgemm_mg(4, 4, 131072, one, one, one, 16, 1, 2) == 10002
    assert lib.ozb_mg_create(0, 0, one, 0, ctypes.byref(h)) == 10001
    assert lib.ozb_mg_create(2, 2, one, 0, ctypes.byref(h)) == 10001     # rank outside the world
    assert lib.ozb_mg_create(2, 0, None, 0, ctypes.byref(h)) == 10001    # more than one rank needs the rendezvous id
    assert lib.ozb_mg_create(2, 0, one, -1, ctypes.byref(h)) == 10001
    assert lib.ozb_mg_dgemm(None, 4, 4, 4, one, 4, one, 4, one, 4, 16, 0, 0, None) == 10001
    assert lib.ozb_mg_wait(None) == 10001 and lib.ozb_mg_info(None, None, None, None) == 10001
    assert lib.ozb_gemm_i8_mod_beside(one, one, one, 0, 4, 4, 1, 16, 16, 16, 64, 64, 64, 0, 16, None, None) == 10001
    lib.ozb_mg_destroy(None)                                             # tolerated
    assert b"communicator" in lib.ozb_error(10007) and b"NCCL" in lib.ozb_error(10008)
    ident = ctypes.create_string_buffer(128)
    rc = lib.ozb_mg_unique_id(ident)                                     # needs libnccl.so.2, not a GPU
    assert rc in (0, 10008)
    assert rc != 0 or any(ident.raw)
    assert lib.ozb_bounds_report(None) in (10001, 10005) and lib.ozb_selftest_bounds() in (10005, 35, 100, 10003)


def test_how_b_would_travel_is_plain_arithmetic():
    """ozb_mg_schedule: what a sharded product of a given shape would do, without a device. B up to 1 GiB, or a transfer that
    is short against the rank's share of the product, travels whole; the benchmark's large configuration (n = 32768 from four
    ranks up) streams in nine pieces whose GEMMs are launched over five K ranges."""
    from ozaki_blackwell_b200._lib import lib

    def schedule(m, n, k, nm=16):
        lay, pieces, ranges = ctypes.c_int(-1), ctypes.c_int(-1), ctypes.c_int(-1)
        assert lib.ozb_mg_schedule(m, n, k, nm, ctypes.byref(lay), ctypes.byref(pieces), ctypes.byref(ranges)) == 0
        return lay.value, pieces.value, ranges.value

    assert schedule(8192, 8192, 8192) == (0, 1, 1)              # 512 MiB of B: one transfer
    assert schedule(16384, 32768, 32768) == (0, 1, 1)           # two ranks: the transfer is short against 16384 rows
    assert schedule(8192, 32768, 32768) == (1, 9, 5)            # four ranks
    assert schedule(4096, 32768, 32768) == (1, 9, 5)            # eight ranks: 512 MiB first, then 1 GiB pieces
    assert schedule(4096, 32768, 8192) == (1, 4, 1)             # a K of one launch keeps one GEMM launch
    assert schedule(100, 500, 700) == (0, 1, 1)
    assert lib.ozb_mg_schedule(0, 4, 4, 16, None, None, None) == 10001
    assert lib.ozb_mg_schedule(4, 4, 131072, 16, None, None, None) == 10002
    assert lib.ozb_mg_schedule(4, 4, 4, 16, None, None, None) == 0                 # NULL-tolerant


def test_cpp_header_compiles_as_plain_cxx(tmp_path):
    import subprocess
    src = tmp_path / "t.cpp"
    src.write_text('#include "ozaki2.hpp"\nint main() { return oz::MAXM == 49 ? 0 : 1; }\n')
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)], check=True)
    subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", os.path.join(ROOT, "include", "ozb.h")], check=True)


def test_the_pieces_of_b_tile_k_and_so_do_the_ranges():
    """ozb_mg_schedule_pieces for many shapes, both layouts: the pieces cover [0, K) in order without gaps, the K ranges
    cover [0, K) in order without gaps, every range ends where its piece ends, the last piece closes the last range, and
    there are fewer than 64 pieces (the handle's event arrays)."""
    import random
    from ozaki_blackwell_b200._lib import lib
    rng = random.Random(7)
    shapes = [(4096, 32768, 32768), (16384, 32768, 32768), (8192, 8192, 8192), (1, 1, 1), (5, 7, 3), (300, 1000, 777), (64, 16, 131071),
              (8192, 65536, 12289), (8192, 200000, 100000), (128, 131, 12288), (128, 131, 12416)]
    shapes += [(rng.randint(1, 20000), rng.randint(1, 70000), rng.randint(1, 131071)) for _ in range(300)]
    arr = lambda: (ctypes.c_int * 64)()
    for m, n, k in shapes:
        for layout in (-1, 0, 1):
            k0, ln, r0, rl = arr(), arr(), arr(), arr()
            np_ = lib.ozb_mg_schedule_pieces(m, n, k, 16, layout, 64, k0, ln, r0, rl)
            assert 1 <= np_ < 64, (m, n, k, layout, np_)
            at = rat = 0
            for i in range(np_):
                assert k0[i] == at and ln[i] > 0, (m, n, k, layout, i)
                at += ln[i]
                if rl[i] > 0:
                    assert r0[i] == rat and r0[i] + rl[i] == at, (m, n, k, layout, i)
                    rat = at
            assert at == k and rat == k, (m, n, k, layout, at, rat)
            if layout == 0:
                assert np_ == 1
            lay, pcs, rgs = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
            if layout == -1:
                assert lib.ozb_mg_schedule(m, n, k, 16, ctypes.byref(lay), ctypes.byref(pcs), ctypes.byref(rgs)) == 0
                assert pcs.value == np_ and rgs.value == sum(1 for i in range(np_) if rl[i] > 0)
    assert lib.ozb_mg_schedule_pieces(0, 4, 4, 16, -1, 0, None, None, None, None) == -10001
    assert lib.ozb_mg_schedule_pieces(4, 4, 131072, 16, -1, 0, None, None, None, None) == -10002
    assert lib.ozb_mg_schedule_pieces(4, 4, 4, 16, 2, 0, None, None, None, None) == -10001
