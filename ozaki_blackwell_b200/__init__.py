"""FP64-accurate matrix products from the INT8 tensor cores of NVIDIA B200 (sm_100a): Ozaki scheme II.

The interface is the reference package's (python/ozaki_blackwell/__init__.py of ShabanEjupi/ozaki-blackwell):

    import numpy as np, ozaki_blackwell_b200 as ob
    C = ob.matmul(A, B)              # float64, NumPy arrays in and out (staged through the GPU)
    C = ob.matmul(At, Bt)            # CUDA arrays (torch tensors, anything with __cuda_array_interface__) stay on the GPU

Arrays are float64 and row-major; `moduli` (8..16) trades accuracy for speed exactly as in the reference, and the result
is bit-identical to the reference's for the same inputs and modulus count. Everything is computed by
libozaki_blackwell.so on the GPU; there is no CPU path.
"""
import ctypes

import numpy as np

from ._lib import lib as _lib

__version__ = "0.1.0"
__all__ = ["matmul", "matmul_dd", "matmul_td", "device", "release", "bench", "OzakiError"]


class OzakiError(RuntimeError):
    pass


def _check(code):
    if code:
        raise OzakiError(_lib.ozb_error(code).decode())


def _is_cuda(x):
    return hasattr(x, "__cuda_array_interface__")


def _cuda_ptr(x, what):
    ai = x.__cuda_array_interface__
    if ai["typestr"] != "<f8" or len(ai["shape"]) != 2:
        raise TypeError(f"{what}: a 2-D float64 CUDA array is needed, got {ai['typestr']} with shape {ai['shape']}")
    if ai.get("strides") not in (None, (ai["shape"][1] * 8, 8)):
        raise TypeError(f"{what}: the CUDA array must be C-contiguous (call .contiguous())")
    return ai["data"][0], tuple(ai["shape"])


def _sync(x):
    """Wait for the stream that produced x: the products run on the legacy default stream, as in the reference."""
    mod = type(x).__module__.split(".")[0]
    if mod == "torch":
        import torch
        torch.cuda.current_stream(x.device).synchronize()
    elif mod == "cupy":
        import cupy
        cupy.cuda.get_current_stream().synchronize()


def _empty_like_cuda(x, shape):
    mod = type(x).__module__.split(".")[0]
    if mod == "torch":
        return x.new_empty(shape)
    if mod == "cupy":
        import cupy
        return cupy.empty(shape, dtype=cupy.float64)
    raise TypeError("for this CUDA array type pass out= (C-contiguous float64 arrays of the result's shape)")


def _shapes(a_parts, b_parts):
    (m, k), (k2, n) = a_parts[0].shape, b_parts[0].shape
    if k != k2:
        raise ValueError(f"inner dimensions differ: {a_parts[0].shape} @ {b_parts[0].shape}")
    if any(x.shape != (m, k) for x in a_parts):
        raise ValueError("all parts of A must have one shape")
    if any(x.shape != (k, n) for x in b_parts):
        raise ValueError("all parts of B must have one shape")
    return m, n, k


def _run(fn, a_parts, b_parts, nout, extra, out):
    if any(_is_cuda(x) for x in a_parts + b_parts):
        if not all(_is_cuda(x) for x in a_parts + b_parts):
            raise TypeError("mix of CUDA and host arrays: move all of them to one side")
        ptrs, shapes = zip(*(_cuda_ptr(x, "input") for x in a_parts + b_parts))
        m, k = shapes[0]
        n = shapes[len(a_parts)][1]
        if any(s != (m, k) for s in shapes[:len(a_parts)]) or any(s != (k, n) for s in shapes[len(a_parts):]):
            raise ValueError(f"shapes do not match: {shapes}")
        outs = list(out) if out is not None else [_empty_like_cuda(a_parts[0], (m, n)) for _ in range(nout)]
        optr = [_cuda_ptr(o, "out")[0] for o in outs]
        for x in a_parts + b_parts + tuple(outs):
            _sync(x)
        _check(fn(m, n, k, *ptrs, *optr, *extra, 0))
        return outs
    a_parts = tuple(np.ascontiguousarray(x, dtype=np.float64) for x in a_parts)
    b_parts = tuple(np.ascontiguousarray(x, dtype=np.float64) for x in b_parts)
    if a_parts[0].ndim != 2 or b_parts[0].ndim != 2:
        raise ValueError("A and B must be 2-D")
    m, n, k = _shapes(a_parts, b_parts)
    outs = list(out) if out is not None else [np.empty((m, n), dtype=np.float64) for _ in range(nout)]
    for o in outs:
        if not (isinstance(o, np.ndarray) and o.dtype == np.float64 and o.shape == (m, n) and o.flags.c_contiguous):
            raise TypeError("out= must hold C-contiguous float64 arrays of the result's shape")
    p = [x.ctypes.data for x in a_parts + b_parts + tuple(outs)]
    _check(fn(m, n, k, *p, *extra, 1))
    return outs


def matmul(a, b, moduli=16, out=None):
    """C = A B in FP64 from INT8 tensor cores; `moduli` in 8..16 (16: FP64 accuracy for exponent spreads up to 2^+-16)."""
    return _run(_lib.ozb_dgemm, (a,), (b,), 1, (int(moduli),), None if out is None else (out,))[0]


def matmul_dd(a, b, out=None):
    """(Ch, Cl) = (Ah + Al)(Bh + Bl) in double-double, 32 moduli. a and b are (hi, lo) pairs."""
    return tuple(_run(_lib.ozb_ddgemm, tuple(a), tuple(b), 2, (), out))


def matmul_td(a, b, out=None):
    """Triple-double product: exported for interface compatibility; this build raises OzakiError."""
    return tuple(_run(_lib.ozb_tdgemm, tuple(a), tuple(b), 3, (), out))


def device():
    """Name, compute capability (e.g. 100), L2 size in KiB and SM count of the current CUDA device."""
    name = ctypes.create_string_buffer(256)
    sm, l2, sms = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    _check(_lib.ozb_device(name, 256, ctypes.byref(sm), ctypes.byref(l2), ctypes.byref(sms)))
    return {"name": name.value.decode(), "sm": sm.value, "l2_kib": l2.value, "sms": sms.value}


def release():
    """Free the device memory of the cached plans."""
    _lib.ozb_release()


def bench(n=4096, kind="fp64", reps=5):
    """Median GPU time (ms) and FP64-equivalent TFLOPS of an n x n x n product on the device, transfers excluded."""
    kinds = {"fp64": 0, "dd": 1, "td": 2}
    ms = ctypes.c_double()
    _check(_lib.ozb_bench(int(n), kinds[kind], int(reps), ctypes.byref(ms)))
    return ms.value, 2.0 * n ** 3 / (ms.value * 1e-3) / 1e12
