"""The allocation-free column pass, ozb_scale_residues_cols_static, against the ordinary entry point.

Some programs cannot allocate GPU memory at the moment they call into this library: their device memory is owned
outright by an allocator of their own (a serving engine, a framework's caching pool), or they sit in a loop that cannot
afford the device-wide synchronisation of cudaMalloc. For them the column pass has a twin whose scratch is a fixed array
inside the library. This test calls the twin through the C ABI twice in a row and requires exactly the output of the
ordinary entry point both times, and exactly the scales and residues of the CPU checker (the reference's scales and
residues<NM>, src/ozaki2.cuh:56-78, restated in oracle/ozaki2_oracle.c); the second call uses smaller magnitudes and fewer
columns than the first, so column maxima left in the shared scratch by the first call would show up as wrong scales. The file name sorts last on purpose:
a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(X, nm, bits):
    import torch
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    rows, cols = X.shape                      # rows = K
    ld = g.round_up(rows, 16)
    Xd = g.dev(X)
    outs = []
    for static in (False, True):
        s = torch.full((cols,), -777, dtype=torch.int32, device="cuda")
        R = torch.full((nm, cols, ld), 55, dtype=torch.int8, device="cuda")
        if static:
            g.check(lib.ozb_scale_residues_cols_static(nm, g.ptr(Xd), rows, cols, cols, bits, g.ptr(s), g.ptr(R), ld, cols * ld, None))
        else:
            cm = torch.zeros((cols,), dtype=torch.int64, device="cuda")
            g.check(lib.ozb_scale_residues_cols(nm, g.ptr(Xd), rows, cols, cols, bits, g.ptr(cm), g.ptr(s), g.ptr(R), ld, cols * ld, None))
        torch.cuda.synchronize()
        outs.append((s.cpu().numpy(), R.cpu().numpy()))
    return outs


def test_static_scratch_variant_matches_twice_in_a_row():
    import gpu_util as g
    import oracle_lib as o
    from ozaki_blackwell_b200._lib import lib
    nm = 16
    first = g.synthetic(700, 1100, 31) * 2.0 ** 40            # large magnitudes, 1100 columns
    second = g.synthetic(520, 900, 32) * 2.0 ** -30           # small magnitudes, fewer columns: stale maxima would be larger
    for X in (first, second):
        bits = lib.ozb_bits_for(nm, X.shape[0], 62)
        (s0, R0), (s1, R1) = _both(X, nm, bits)
        assert np.array_equal(s0, s1), g.describe_mismatch(s1, s0)
        assert np.array_equal(R0[:, :, :X.shape[0]], R1[:, :, :X.shape[0]])
        # and against the checker directly: columns of a row-major K x N matrix (element k of column j at k * N + j)
        K, N = X.shape
        want_s = o.scales(X, N, K, 1, N, bits)
        want_R = o.residues(X, N, K, 1, N, want_s, nm)
        assert np.array_equal(s1, want_s), g.describe_mismatch(s1, want_s)
        assert np.array_equal(R1[:, :, :K], want_R), g.describe_mismatch(R1[:, :, :K], want_R)


def test_static_scratch_variant_rejects_sizes_beyond_its_array():
    import ctypes
    from ozaki_blackwell_b200._lib import lib
    one = ctypes.c_void_p(16)   # never dereferenced: the size check comes first
    assert lib.ozb_scale_residues_cols_static(16, one, 64, 65537, 65537, 50, one, one, 64, 64 * 65537, None) == 10006
    assert b"limit" in lib.ozb_error(10006)
