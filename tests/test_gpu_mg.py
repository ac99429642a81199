"""The library's own multi-GPU layer (ozb_mg_*, ozb_dgemm_mg) through the C ABI. The single-rank cases run on one GPU and
cover both ways B is consumed (in one piece; column maxima first, then pieces of rows feeding GEMMs over K ranges); the
cases with two ranks need two GPUs and are skipped otherwise. Results are compared bit for bit with the CPU checker."""
import ctypes
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _run_child(code, env=None, timeout=300):
    """Runs `code` in a fresh interpreter: the layer reads its environment switches once per process."""
    import subprocess
    e = dict(os.environ)
    e.update(env or {})
    e["PYTHONPATH"] = os.pathsep.join([HERE, ROOT, e.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


_SINGLE = r"""
import ctypes, numpy as np, torch
import gpu_util as g, oracle_lib as o
from ozaki_blackwell_b200._lib import lib
M, N, K, nm = {shape}
A, B = g.synthetic(M, K, 301), g.synthetic(K, N, 302)
want = o.dgemm(A, B, nm)
h = ctypes.c_void_p()
g.check(lib.ozb_mg_create(1, 0, None, 5000, ctypes.byref(h)))
Ad, Bd = g.dev(A), g.dev(B)
Cd = torch.full((M, N + 3), 7.0, dtype=torch.float64, device="cuda")
st = torch.cuda.Stream()
for rep in range(2):
    g.check(lib.ozb_mg_dgemm(h, M, N, K, g.ptr(Ad), K, g.ptr(Bd), N, g.ptr(Cd), N + 3, nm, 0, 0, ctypes.c_void_p(st.cuda_stream)))
g.check(lib.ozb_mg_wait(h))
got = Cd[:, :N].cpu().numpy()
assert g.same_bits(got, want), g.describe_mismatch(got, want)
assert torch.all(Cd[:, N:] == 7.0)
layout, pieces, kernels = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
g.check(lib.ozb_mg_info(h, ctypes.byref(layout), ctypes.byref(pieces), ctypes.byref(kernels)))
assert kernels.value >= 5
print("layout", layout.value, "pieces", pieces.value)
# a strided B is packed first
Bw = torch.zeros((K, N + 5), dtype=torch.float64, device="cuda"); Bw[:, :N] = Bd
Cd.fill_(0)
g.check(lib.ozb_mg_dgemm(h, M, N, K, g.ptr(Ad), K, g.ptr(Bw), N + 5, g.ptr(Cd), N + 3, nm, 0, 0, None))
g.check(lib.ozb_mg_wait(h))
assert g.same_bits(Cd[:, :N].cpu().numpy(), want)
# host operands (pinned), the block pipeline
Ah = torch.from_numpy(A).pin_memory(); Bh = torch.from_numpy(B).pin_memory(); Ch = torch.zeros((M, N), dtype=torch.float64).pin_memory()
g.check(lib.ozb_mg_dgemm(h, M, N, K, g.ptr(Ah), K, g.ptr(Bh), N, g.ptr(Ch), N, nm, 0, 1, None))
assert g.same_bits(Ch.numpy(), want)
assert lib.ozb_mg_dgemm(h, M, N, K, g.ptr(Ad), K - 1, g.ptr(Bd), N, g.ptr(Cd), N + 3, nm, 0, 0, None) == 10001
assert lib.ozb_mg_dgemm(h, M, N, K, g.ptr(Ad), K, None, N, g.ptr(Cd), N + 3, nm, 0, 0, None) == 10001     # the holder must pass B
lib.ozb_mg_destroy(h)
# the reference-shaped call with one device
C1 = np.zeros((M, N))
g.check(lib.ozb_dgemm_mg(M, N, K, A.ctypes.data, B.ctypes.data, C1.ctypes.data, nm, 1, 1))
assert g.same_bits(C1, want)
Cd2 = torch.zeros((M, N), dtype=torch.float64, device="cuda")
g.check(lib.ozb_dgemm_mg(M, N, K, g.ptr(Ad), g.ptr(Bd), g.ptr(Cd2), nm, 0, 1))
assert g.same_bits(Cd2.cpu().numpy(), want)
lib.ozb_mg_release()
print("ok")
"""


@pytest.mark.parametrize("env,shape,expect", [
    ({}, (300, 500, 700, 16), "layout 0 pieces 1"),
    ({"OZ_MG_LAYOUT": "stream", "OZ_MG_PIECE_MB": "1", "OZ_KCHUNK": "1024"}, (300, 500, 2600, 16), "layout 1 pieces"),
    ({"OZ_MG_LAYOUT": "stream", "OZ_MG_PIECE_MB": "1", "OZ_KCHUNK": "1024"}, (130, 270, 1300, 13), "layout 1 pieces"),
])
def test_single_rank_both_layouts(env, shape, expect):
    out = _run_child(_SINGLE.format(shape=shape), env)
    assert expect in out and out.strip().endswith("ok"), out


def _worker(rank, world, ident, M, N, K, nm, src, out_dir):
    import torch
    sys.path.insert(0, HERE)
    sys.path.insert(0, ROOT)
    import gpu_util as g
    from ozaki_blackwell_b200._lib import lib
    from ozaki_blackwell_b200.dist import row_block
    torch.cuda.set_device(rank)
    h = ctypes.c_void_p()
    g.check(lib.ozb_mg_create(world, rank, ident, 4000, ctypes.byref(h)))
    A, B = g.synthetic(M, K, 61), g.synthetic(K, N, 62)
    lo, hi = row_block(M, rank, world)
    m = hi - lo
    a = torch.from_numpy(A[lo:hi].copy()).cuda()
    b = torch.from_numpy(B).cuda() if rank == src else None
    c = torch.zeros((m, N), dtype=torch.float64, device="cuda")
    for _ in range(2):
        g.check(lib.ozb_mg_dgemm(h, m, N, K, g.ptr(a), K, g.ptr(b) if b is not None else None, N, g.ptr(c), N, nm, src, 0, None))
    g.check(lib.ozb_mg_wait(h))
    np.save(os.path.join(out_dir, f"c{rank}.npy"), c.cpu().numpy())
    # host operands
    ah = torch.from_numpy(A[lo:hi].copy()).pin_memory()
    bh = torch.from_numpy(B).pin_memory() if rank == src else None
    ch = torch.zeros((m, N), dtype=torch.float64).pin_memory()
    g.check(lib.ozb_mg_dgemm(h, m, N, K, g.ptr(ah), K, g.ptr(bh) if bh is not None else None, N, g.ptr(ch), N, nm, src, 1, None))
    np.save(os.path.join(out_dir, f"h{rank}.npy"), ch.numpy())
    lib.ozb_mg_destroy(h)


def _spawn(tmp_path, env, shape=(700, 1000, 520, 16), src=0):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from ozaki_blackwell_b200._lib import lib
    ident = ctypes.create_string_buffer(128)
    assert lib.ozb_mg_unique_id(ident) == 0
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        M, N, K, nm = shape
        mp.spawn(_worker, args=(2, ident.raw, M, N, K, nm, src, str(tmp_path)), nprocs=2, join=True)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    return shape


@pytest.mark.parametrize("src", [0, 1])
@pytest.mark.parametrize("env", [{}, {"OZ_MG_LAYOUT": "stream", "OZ_MG_PIECE_MB": "1", "OZ_KCHUNK": "1024"}])
def test_two_ranks_bit_identical_to_the_checker(tmp_path, env, src):
    import gpu_util as g
    import oracle_lib as o
    shape = (700, 1000, 2600, 16) if env else (700, 1000, 520, 16)
    M, N, K, nm = _spawn(tmp_path, env, shape=shape, src=src)
    A, B = g.synthetic(M, K, 61), g.synthetic(K, N, 62)
    want = o.dgemm(A, B, nm)
    for tag in "ch":
        got = np.vstack([np.load(tmp_path / f"{tag}{r}.npy") for r in range(2)])
        assert g.same_bits(got, want), (tag, g.describe_mismatch(got, want))


_LEAVER = r"""
import ctypes, os, sys, time, numpy as np, torch
import gpu_util as g
from ozaki_blackwell_b200._lib import lib
rank, out_dir = int(sys.argv[1]), sys.argv[2]
ident = open(os.path.join(out_dir, "id"), "rb").read()
M, N, K, nm = 256, 512, 384, 16
torch.cuda.set_device(rank)
h = ctypes.c_void_p()
g.check(lib.ozb_mg_create(2, rank, ident, 3000, ctypes.byref(h)))
A, B = g.synthetic(M, K, 61), g.synthetic(K, N, 62)
a = torch.from_numpy(A[rank * 128:(rank + 1) * 128].copy()).cuda()
b = torch.from_numpy(B).cuda() if rank == 1 else None      # the rank that will leave holds B: the survivor is a receiver
c = torch.zeros((128, N), dtype=torch.float64, device="cuda")
bp = g.ptr(b) if b is not None else None
g.check(lib.ozb_mg_dgemm(h, 128, N, K, g.ptr(a), K, bp, N, g.ptr(c), N, nm, 1, 0, None))
g.check(lib.ozb_mg_wait(h))                      # one complete step on both ranks
torch.cuda.synchronize()
if rank == 1:
    # leaves between steps with nothing of its own in flight, without a word to its peer (no collective tear-down)
    open(os.path.join(out_dir, "left"), "w").write("1")
    os._exit(0)
while not os.path.exists(os.path.join(out_dir, "left")):
    time.sleep(0.05)
time.sleep(1.0)
t0 = time.time()
rc = lib.ozb_mg_dgemm(h, 128, N, K, g.ptr(a), K, bp, N, g.ptr(c), N, nm, 1, 0, None)
if rc == 0:
    rc = lib.ozb_mg_wait(h)                      # B never arrives: bounded wait, communicator aborted
took = time.time() - t0
again = lib.ozb_mg_wait(h)
lib.ozb_mg_destroy(h)
alone = g.gpu_dgemm(A[:64], B, nm)               # the device still computes
np.save(os.path.join(out_dir, "alone.npy"), alone)
open(os.path.join(out_dir, "rc"), "w").write(f"{rc} {again} {took:.2f}")
"""


def test_a_rank_that_leaves_between_steps_is_reported(tmp_path):
    """Two ranks finish a step; rank 1, which holds B, then exits. Rank 0's next product never receives B: the bounded host
    wait (3 s here) aborts the communicator and the call reports OZB_ECOMM instead of hanging; the handle stays broken and
    the CUDA context stays usable. Both ranks are child processes that are killed if they outlive the test's patience."""
    import subprocess
    import time
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import gpu_util as g
    import oracle_lib as o
    from ozaki_blackwell_b200._lib import lib
    ident = ctypes.create_string_buffer(128)
    assert lib.ozb_mg_unique_id(ident) == 0
    (tmp_path / "id").write_bytes(ident.raw)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.pathsep.join([HERE, ROOT, os.environ.get("PYTHONPATH", "")]))
    procs = [subprocess.Popen([sys.executable, "-c", _LEAVER, str(r), str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
             for r in range(2)]
    deadline = time.time() + 90
    try:
        while time.time() < deadline and any(p.poll() is None for p in procs):
            time.sleep(0.2)
    finally:
        late = [r for r, p in enumerate(procs) if p.poll() is None]
        for p in procs:
            if p.poll() is None:
                p.kill()
    outs = [p.communicate()[0].decode(errors="replace")[-2000:] for p in procs]
    assert not late, f"ranks {late} did not finish in time\n" + "\n".join(outs)
    assert procs[0].returncode == 0, outs[0]
    rc, again, took = open(tmp_path / "rc").read().split()
    assert int(rc) == 10007 and int(again) == 10007, (rc, again, outs[0])     # OZB_ECOMM, and the handle stays broken
    assert float(took) < 20.0
    A, B = g.synthetic(256, 384, 61), g.synthetic(384, 512, 62)
    assert g.same_bits(np.load(tmp_path / "alone.npy"), o.dgemm(A[:64], B, 16))


def test_one_process_two_devices_reference_shaped_call():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run_child(r"""
import numpy as np, torch
import gpu_util as g, oracle_lib as o
from ozaki_blackwell_b200._lib import lib
M, N, K, nm = 513, 700, 900, 16
A, B = g.synthetic(M, K, 71), g.synthetic(K, N, 72)
want = o.dgemm(A, B, nm)
C = np.zeros((M, N))
for _ in range(2):
    g.check(lib.ozb_dgemm_mg(M, N, K, A.ctypes.data, B.ctypes.data, C.ctypes.data, nm, 1, 2))
assert g.same_bits(C, want), g.describe_mismatch(C, want)
for cur in (0, 1):
    torch.cuda.set_device(cur)
    Ad, Bd = g.dev(A), g.dev(B)
    Cd = torch.zeros((M, N), dtype=torch.float64, device="cuda")
    g.check(lib.ozb_dgemm_mg(M, N, K, g.ptr(Ad), g.ptr(Bd), g.ptr(Cd), nm, 0, 2))
    assert g.same_bits(Cd.cpu().numpy(), want), cur
assert lib.ozb_dgemm_mg(M, N, K, A.ctypes.data, B.ctypes.data, C.ctypes.data, nm, 1, 99) == 10001
import ozaki_blackwell_b200 as ob
assert g.same_bits(ob.matmul(A, B, moduli=nm, devices=2), want)          # the wrapper's keyword, host operands
torch.cuda.set_device(0)
assert g.same_bits(ob.matmul(g.dev(A), g.dev(B), moduli=nm, devices=2).cpu().numpy(), want)   # device operands
lib.ozb_mg_release()
print("ok")
""", {"NCCL_NVLS_ENABLE": "0"})
    assert out.strip().endswith("ok")
