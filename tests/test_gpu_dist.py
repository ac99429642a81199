"""Row-block sharding on real GPUs over NCCL (skipped with fewer than two devices): the rows every rank produces are
bit-identical to the same rows of the single-GPU product, whichever rank holds B."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, M, N, K, nm, src, layout, out_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from ozaki_blackwell_b200.dist import RowShardedGemm, row_block
    import gpu_util as g
    A, B = g.synthetic(M, K, 61), g.synthetic(K, N, 62)
    lo, hi = row_block(M, rank, world)
    a = torch.from_numpy(A[lo:hi].copy()).cuda()
    b = torch.from_numpy(B).cuda() if rank == src else None
    c = torch.zeros((hi - lo, N), dtype=torch.float64, device="cuda")
    op = RowShardedGemm(hi - lo, N, K, nm, src=src, panels=3, layout=layout)
    for _ in range(2):
        op(a, b, c)
    torch.cuda.synchronize()
    op.engine.status()
    np.save(os.path.join(out_dir, f"c{rank}.npy"), c.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["rows", "panels"])
@pytest.mark.parametrize("src", [0, 1])
def test_two_gpus_bit_identical_to_one(tmp_path, src, layout):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import gpu_util as g
    M, N, K, nm = 700, 1000, 520, 16
    port = 29600 + (os.getpid() % 1000) + src + 2 * (layout == "rows")
    mp.spawn(_worker, args=(2, port, M, N, K, nm, src, layout, str(tmp_path)), nprocs=2, join=True)
    A, B = g.synthetic(M, K, 61), g.synthetic(K, N, 62)
    want = g.gpu_dgemm(A, B, nm)
    got = np.vstack([np.load(tmp_path / f"c{r}.npy") for r in range(2)])
    assert g.same_bits(got, want), g.describe_mismatch(got, want)


def test_one_process_two_devices():
    """A process that switches devices: per-device kernel attributes, constant tables and plan caches must follow."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import gpu_util as g
    import oracle_lib as o
    A, B = g.synthetic(300, 260, 71), g.synthetic(260, 280, 72)
    want = o.dgemm(A, B, 16)
    try:
        for dev in (0, 1, 0, 1):
            torch.cuda.set_device(dev)
            got = g.gpu_dgemm(A, B, 16)
            assert g.same_bits(got, want), (dev, g.describe_mismatch(got, want))
        # a plan belongs to the device it was made on: from another current device its calls are refused
        import ctypes
        from ozaki_blackwell_b200._lib import lib
        torch.cuda.set_device(0)
        plan = ctypes.c_void_p()
        g.check(lib.ozb_plan_create(64, 64, 64, 16, 62, ctypes.byref(plan)))
        a = torch.zeros((64, 64), dtype=torch.float64, device="cuda:0")
        torch.cuda.set_device(1)
        assert lib.ozb_plan_set_a(plan, g.ptr(a), 64, None) == 101      # cudaErrorInvalidDevice
        torch.cuda.set_device(0)
        g.check(lib.ozb_plan_set_a(plan, g.ptr(a), 64, None))
        g.check(lib.ozb_plan_status(plan))
        lib.ozb_plan_destroy(plan)
    finally:
        torch.cuda.set_device(0)
