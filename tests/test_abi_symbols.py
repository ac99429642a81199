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


def test_cpp_header_compiles_as_plain_cxx(tmp_path):
    import subprocess
    src = tmp_path / "t.cpp"
    src.write_text('#include "ozaki2.hpp"\nint main() { return oz::MAXM == 49 ? 0 : 1; }\n')
    subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)], check=True)
    subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", os.path.join(ROOT, "include", "ozb.h")], check=True)
