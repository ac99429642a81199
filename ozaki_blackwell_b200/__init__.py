"""FP64-accurate matrix products on NVIDIA B200 (sm_100a) from exact INT8 tensor-core products: Ozaki scheme II.

Public names and their meaning follow the reference's Python package (python/ozaki_blackwell/__init__.py of
ShabanEjupi/ozaki-blackwell), so that code written against it runs unchanged:

    matmul(a, b, moduli=16, out=None)     C = A B, float64 row-major; 8 <= moduli <= 16
    matmul_dd((ah, al), (bh, bl))         double-double product, returns (Ch, Cl)
    matmul_td(...)                        triple-double: part of the interface, not built here (raises OzakiError)
    device(), release(), bench(n, kind, reps), OzakiError

Operands are either all host arrays (anything numpy can view as float64; the library stages them through the GPU) or all
device arrays exposing __cuda_array_interface__ (torch, cupy, numba, ...; nothing leaves the GPU). Results are bit-identical
to the reference's for the same inputs and modulus count. All arithmetic happens in libozaki_blackwell.so on the GPU: a
missing library is an ImportError, a GPU that is not compute capability 10.x an OzakiError.
"""
import ctypes
import importlib

import numpy as np

from ._lib import lib as _lib

__version__ = "0.1.0"
__all__ = ["matmul", "matmul_dd", "matmul_td", "device", "release", "bench", "OzakiError"]


class OzakiError(RuntimeError):
    """A non-zero status of the C library, with the library's own text for it."""

    def __init__(self, code):
        self.code = int(code)
        super().__init__(_lib.ozb_error(self.code).decode())


class _DeviceSide:
    """How to treat operands that live on the GPU: pointer extraction, stream hand-over, allocation of results."""

    @staticmethod
    def owns(x):
        return hasattr(x, "__cuda_array_interface__")

    @staticmethod
    def describe(x, role):
        iface = x.__cuda_array_interface__
        shape, strides = tuple(iface["shape"]), iface.get("strides")
        if iface["typestr"] != "<f8" or len(shape) != 2:
            raise TypeError(f"{role} must be a two-dimensional float64 device array (typestr {iface['typestr']}, shape {shape})")
        if strides is not None and tuple(strides) != (8 * shape[1], 8):
            raise TypeError(f"{role} must be row-major and dense; make it contiguous first")
        return shape, int(iface["data"][0])

    @staticmethod
    def hand_over(x):
        # the library launches on the legacy default stream: whatever the framework queued on its own stream must be done
        family = type(x).__module__.partition(".")[0]
        if family == "torch":
            importlib.import_module("torch").cuda.current_stream(x.device).synchronize()
        elif family == "cupy":
            importlib.import_module("cupy").cuda.get_current_stream().synchronize()

    @staticmethod
    def result_like(x, shape):
        family = type(x).__module__.partition(".")[0]
        if family == "torch":
            return x.new_empty(shape)
        if family == "cupy":
            return importlib.import_module("cupy").empty(shape, dtype="float64")
        raise TypeError(f"cannot allocate a result for {type(x).__name__}: give out=")

    on_host_flag = 0


class _HostSide:
    """Operands in host memory: made contiguous float64 once, results as numpy arrays."""

    @staticmethod
    def owns(x):
        return not _DeviceSide.owns(x)

    @staticmethod
    def describe(x, role):
        if x.ndim != 2:
            raise ValueError(f"{role} must be two-dimensional, got {x.ndim} dimensions")
        return x.shape, x.ctypes.data

    @staticmethod
    def hand_over(x):
        pass

    @staticmethod
    def result_like(x, shape):
        return np.empty(shape, dtype=np.float64)

    on_host_flag = 1


def _call(entry, left, right, n_results, trailing, out):
    """One product through `entry`: `left` and `right` are the parts of A and B (1 for FP64, 2 for double-double, ...)."""
    left, right = list(left), list(right)
    if len(left) != n_results or len(right) != n_results:
        raise ValueError(f"this product takes {n_results} part(s) per operand, got {len(left)} and {len(right)}")
    parts = left + right
    on_device = [_DeviceSide.owns(x) for x in parts]
    if any(on_device) and not all(on_device):
        raise TypeError("operands must be all on the host or all on the device")
    side = _DeviceSide if on_device[0] else _HostSide
    if side is _HostSide:
        parts = [np.ascontiguousarray(x, dtype=np.float64) for x in parts]
    described = [side.describe(x, "an operand") for x in parts]
    (rows, inner), (inner_b, cols) = described[0][0], described[len(left)][0]
    if inner != inner_b:
        raise ValueError(f"cannot multiply {rows} x {inner} by {inner_b} x {cols}")
    for (shape, _), expected in zip(described, [(rows, inner)] * len(left) + [(inner, cols)] * len(right)):
        if tuple(shape) != expected:
            raise ValueError(f"every part of an operand needs the same shape: {tuple(shape)} against {expected}")
    if out is None:
        results = [side.result_like(parts[0], (rows, cols)) for _ in range(n_results)]
    else:
        results = list(out)
        if len(results) != n_results or not all(side.owns(r) for r in results):
            raise TypeError(f"out= needs {n_results} array(s) on the same side as the operands")
        for r in results:
            if side is _HostSide and not (isinstance(r, np.ndarray) and r.dtype == np.float64 and r.flags.c_contiguous):
                raise TypeError("out= arrays must be C-contiguous float64 numpy arrays")
            if tuple(side.describe(r, "out")[0]) != (rows, cols):
                raise ValueError(f"out= arrays must have shape {(rows, cols)}")
    for x in parts + results:
        side.hand_over(x)
    addresses = [p for _, p in described] + [side.describe(r, "out")[1] for r in results]
    status = entry(rows, cols, inner, *addresses, *trailing, side.on_host_flag)
    if status:
        raise OzakiError(status)
    return results


def matmul(a, b, moduli=16, out=None, devices=1):
    """A @ B with FP64 accuracy. `moduli` (8..16) is the reference's accuracy/speed knob: 16 gives full FP64 accuracy for
    entries spread over 2^+-16, fewer moduli are faster and coarser. `out`: an array to receive the result.
    `devices` > 1 (an addition; the reference is single-GPU) splits the rows of A and C over GPUs 0 .. devices-1 of this
    machine, with B broadcast over NVLink; the result has the same bits."""
    entry = _lib.ozb_dgemm
    if int(devices) > 1:
        def entry(*args):
            return _lib.ozb_dgemm_mg(*args, int(devices))
    return _call(entry, [a], [b], 1, [int(moduli)], None if out is None else [out])[0]


def matmul_dd(a, b, out=None):
    """Double-double product: a = (hi, lo) and b = (hi, lo) pairs of float64 arrays; returns (Ch, Cl). 32 moduli."""
    return tuple(_call(_lib.ozb_ddgemm, a, b, 2, [], out))


def matmul_td(a, b, out=None):
    """Triple-double product of (x0, x1, x2) triples. Kept for interface compatibility: this library does not build it
    and the call raises OzakiError."""
    return tuple(_call(_lib.ozb_tdgemm, a, b, 3, [], out))


def device():
    """The current CUDA device as a dict: name, sm (10 * major + minor), l2_kib, sms."""
    text = ctypes.create_string_buffer(256)
    numbers = [ctypes.c_int() for _ in range(3)]
    status = _lib.ozb_device(text, len(text), *[ctypes.byref(v) for v in numbers])
    if status:
        raise OzakiError(status)
    return dict(zip(("name", "sm", "l2_kib", "sms"), [text.value.decode()] + [v.value for v in numbers]))


def release():
    """Give back the device memory held by the cached plans."""
    _lib.ozb_release()


_BENCH_KINDS = {"fp64": 0, "dd": 1, "td": 2}


def bench(n=4096, kind="fp64", reps=5):
    """The library's built-in timing of an n x n x n product with operands on the device: (median ms, FP64-equivalent
    TFLOP/s). kind: "fp64", "dd" or "td"."""
    if kind not in _BENCH_KINDS:
        raise ValueError(f"kind must be one of {sorted(_BENCH_KINDS)}")
    median = ctypes.c_double()
    status = _lib.ozb_bench(int(n), _BENCH_KINDS[kind], int(reps), ctypes.byref(median))
    if status:
        raise OzakiError(status)
    return median.value, 2.0 * float(n) ** 3 / (median.value * 1e-3) / 1e12
