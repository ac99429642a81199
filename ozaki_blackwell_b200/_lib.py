"""ctypes binding of libozaki_blackwell.so (the C ABI declared in include/ozb.h).

The library holds sm_100a code only and has no CPU path: importing this module builds nothing and computes nothing;
it fails loudly if the shared library is missing (run `make -C ozaki_blackwell_b200/csrc` or __graft_entry__.build()).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("OZB_LIBRARY") or os.path.join(_HERE, "libozaki_blackwell.so")   # OZB_LIBRARY: another build of the same ABI

if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}`; there is no fallback path")

lib = ctypes.CDLL(LIB_PATH)

_i, _ll, _p, _sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_size_t
_ip = ctypes.POINTER(ctypes.c_int)

# the reference's eight (python/ozaki_blackwell/__init__.py:26-36 of the reference sets the same argtypes)
lib.ozb_version.restype = ctypes.c_char_p
lib.ozb_version.argtypes = []
lib.ozb_error.restype = ctypes.c_char_p
lib.ozb_error.argtypes = [_i]
lib.ozb_device.argtypes = [ctypes.c_char_p, _i, _ip, _ip, _ip]
lib.ozb_dgemm.argtypes = [_i] * 3 + [_p] * 3 + [_i] * 2
lib.ozb_ddgemm.argtypes = [_i] * 3 + [_p] * 6 + [_i]
lib.ozb_tdgemm.argtypes = [_i] * 3 + [_p] * 9 + [_i]
lib.ozb_release.restype = None
lib.ozb_release.argtypes = []
lib.ozb_bench.argtypes = [_i] * 3 + [ctypes.POINTER(ctypes.c_double)]

# additions
lib.ozb_bits_for.argtypes = [_i, _i, _i]
lib.ozb_modulus.argtypes = [_i]
lib.ozb_plan_create.argtypes = [_i, _i, _i, _i, _i, ctypes.POINTER(_p)]
lib.ozb_plan_destroy.restype = None
lib.ozb_plan_destroy.argtypes = [_p]
lib.ozb_plan_dgemm.argtypes = [_p, _p, _ll, _p, _ll, _p, _ll, _p]
lib.ozb_plan_set_a.argtypes = [_p, _p, _ll, _p]
lib.ozb_plan_panel.argtypes = [_p, _p, _ll, _p, _ll, _i, _i, _p]
lib.ozb_plan_b_begin.argtypes = [_p, _p]
lib.ozb_plan_b_rows.argtypes = [_p, _p, _ll, _i, _p]
lib.ozb_plan_b_finish.argtypes = [_p, _p, _ll, _p]
lib.ozb_plan_multiply.argtypes = [_p, _p, _ll, _p]
lib.ozb_cols_absmax.argtypes = [_p, _i, _i, _ll, _p, _p]
lib.ozb_plan_b_rows_residues.argtypes = [_p, _p, _ll, _i, _i, _p, _p]
lib.ozb_plan_view.argtypes = [_p, _ip, _ip, _ip] + [ctypes.POINTER(_p)] * 5
lib.ozb_plan_status.argtypes = [_p]
lib.ozb_plan_profile.argtypes = [_p, _i]
lib.ozb_plan_phase_ms.argtypes = [_p, _i, ctypes.POINTER(ctypes.c_float * 4)]
lib.ozb_plan_kernel_ms.argtypes = [_p, _i, ctypes.POINTER(ctypes.c_float * 5)]
lib.ozb_dgemm_ex.argtypes = [_i, _i, _i, _p, _ll, _p, _ll, _p, _ll, _i, _p]
lib.ozb_dgemm_norm.argtypes = [_i, _i, _i, _p, _ll, _p, _ll, _p, _ll, _i, _p]
lib.ozb_scales_norm.argtypes = [_p, _i, _i, _ll, _i, _i, _p, _p]
lib.ozb_ddgemm_ex.argtypes = [_i, _i, _i, _p, _p, _ll, _p, _p, _ll, _p, _p, _ll, _i, _i, _p]
lib.ozb_bf16_fp8_gemm.argtypes = [_i, _i, _i, _p, _p, _p, _p, _ip, _ip, _p]
lib.ozb_scale_residues_rows.argtypes = [_i, _p, _i, _i, _ll, _i, _p, _p, _i, _sz, _p]
lib.ozb_scale_residues_cols.argtypes = [_i, _p, _i, _i, _ll, _i, _p, _p, _p, _i, _sz, _p]
lib.ozb_scale_residues_cols_static.argtypes = [_i, _p, _i, _i, _ll, _i, _p, _p, _i, _sz, _p]
lib.ozb_gemm_i8.argtypes = [_p, _p, _p, _i, _i, _i, _i, _ll, _ll, _ll, _sz, _sz, _sz, _p]
lib.ozb_gemm_i8_mod.argtypes = [_p, _p, _p, _i, _i, _i, _i, _ll, _ll, _ll, _sz, _sz, _sz, _i, _p]
lib.ozb_gemm_i8_mod_beside.argtypes = [_p, _p, _p, _i, _i, _i, _i, _ll, _ll, _ll, _sz, _sz, _sz, _i, _i, _p, _p]
lib.ozb_crt_i32.argtypes = [_i, _p, _sz, _i, _i, _ll, _p, _p, _p, _ll, _p]
lib.ozb_crt_i8.argtypes = [_i, _p, _sz, _i, _i, _ll, _p, _p, _p, _ll, _p]
lib.ozb_int8_peak.argtypes = [_i, _i, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_double)]
lib.ozb_selftest_wait_expiry.argtypes = [_i]
lib.ozb_dgemm_mg.argtypes = [_i] * 3 + [_p] * 3 + [_i] * 3
lib.ozb_mg_release.restype = None
lib.ozb_mg_release.argtypes = []
lib.ozb_mg_unique_id.argtypes = [_p]
lib.ozb_mg_create.argtypes = [_i, _i, _p, _i, ctypes.POINTER(_p)]
lib.ozb_mg_destroy.restype = None
lib.ozb_mg_destroy.argtypes = [_p]
lib.ozb_mg_dgemm.argtypes = [_p, _i, _i, _i, _p, _ll, _p, _ll, _p, _ll, _i, _i, _i, _p]
lib.ozb_mg_wait.argtypes = [_p]
lib.ozb_mg_info.argtypes = [_p, _ip, _ip, _ip]
lib.ozb_mg_schedule.argtypes = [_i, _i, _i, _i, _ip, _ip, _ip]
lib.ozb_mg_schedule_pieces.argtypes = [_i, _i, _i, _i, _i, _i, _ip, _ip, _ip, _ip]
lib.ozb_status.argtypes = []
lib.ozb_bounds_report.argtypes = [ctypes.POINTER(ctypes.c_ulonglong * 4)]
lib.ozb_selftest_bounds.argtypes = []

# every symbol include/ozb.h declares; tests check that the library exports each one
SYMBOLS = [
    "ozb_version", "ozb_error", "ozb_device", "ozb_dgemm", "ozb_ddgemm", "ozb_tdgemm", "ozb_release", "ozb_bench",
    "ozb_bits_for", "ozb_modulus", "ozb_plan_create", "ozb_plan_destroy", "ozb_plan_dgemm", "ozb_plan_set_a",
    "ozb_plan_panel", "ozb_plan_b_begin", "ozb_plan_b_rows", "ozb_plan_b_finish", "ozb_plan_multiply", "ozb_cols_absmax", "ozb_plan_b_rows_residues", "ozb_plan_view", "ozb_plan_status", "ozb_plan_profile", "ozb_plan_phase_ms", "ozb_plan_kernel_ms", "ozb_dgemm_ex", "ozb_dgemm_norm", "ozb_scales_norm", "ozb_ddgemm_ex", "ozb_bf16_fp8_gemm",
    "ozb_scale_residues_rows", "ozb_scale_residues_cols", "ozb_scale_residues_cols_static", "ozb_gemm_i8", "ozb_gemm_i8_mod", "ozb_gemm_i8_mod_beside", "ozb_crt_i32", "ozb_crt_i8",
    "ozb_status", "ozb_int8_peak", "ozb_selftest_wait_expiry", "ozb_bounds_report", "ozb_selftest_bounds",
    "ozb_dgemm_mg", "ozb_mg_release", "ozb_mg_unique_id", "ozb_mg_create", "ozb_mg_destroy", "ozb_mg_dgemm", "ozb_mg_wait", "ozb_mg_info", "ozb_mg_schedule", "ozb_mg_schedule_pieces",
]
