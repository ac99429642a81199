"""The multi-GPU orchestration (row blocks, panel broadcast of B) on two CPU ranks over gloo.

The product path has no CPU implementation, so the ranks here get an engine that answers set_a / panel / full with the
CPU checker; what is under test is the host logic of ozaki_blackwell_b200/dist.py: the partition of rows, the panel
ranges and row chunks, that every rank receives every piece of B from the source rank, and that the assembled result is bit-identical
to the unsharded product.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


class CheckerEngine:
    """set_a / panel / full of the CUDA engine, answered by the CPU checker on torch CPU tensors."""

    def __init__(self, nm, k=None):
        self.nm, self.A, self.calls, self.k = nm, None, [], k

    def set_a(self, a, stream):
        self.A = a.numpy().copy()

    def panel(self, b_panel, c, j0, ncols, stream):
        import oracle_lib as o
        self.calls.append((j0, ncols))
        c[:, j0:j0 + ncols] = torch.from_numpy(o.dgemm(self.A, b_panel.numpy(), self.nm))

    def b_begin(self, stream):
        self.rows, self.B = [], None

    def b_rows(self, rows, stream):
        self.rows.append(rows.numpy().copy())

    def cols_absmax(self, b, colmax, stream):
        m = np.abs(b.numpy()).max(axis=0)
        colmax.copy_(torch.from_numpy(np.maximum(m.view(np.int64), colmax.numpy())))

    def b_rows_residues(self, rows, k0, colmax, stream):
        if k0 == 0:
            self.rows, self.maxima = [], colmax.numpy().copy()
        assert k0 == sum(r.shape[0] for r in self.rows) and k0 % 128 == 0
        self.rows.append(rows.numpy().copy())
        self.B = np.vstack(self.rows)
        if self.B.shape[0] == self.k:               # complete: the maxima sent ahead are those of the whole of B
            assert np.array_equal(self.maxima, np.abs(self.B).max(axis=0).view(np.int64))
            self.calls.append((len(self.rows), self.k))

    def b_finish(self, b, stream):
        self.B = b.numpy().copy()
        assert np.array_equal(np.vstack(self.rows), self.B)     # the chunks that arrived are the whole of B, in order
        self.calls.append((len(self.rows), self.B.shape[0]))

    def multiply(self, c, stream):
        import oracle_lib as o
        c.copy_(torch.from_numpy(o.dgemm(self.A, self.B, self.nm)))

    def full(self, a, b, c, stream):
        import oracle_lib as o
        c.copy_(torch.from_numpy(o.dgemm(a.numpy(), b.numpy(), self.nm)))


def _worker(rank, world, port, M, N, K, nm, panels, src, layout, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ozaki_blackwell_b200.dist import RowShardedGemm, row_block
    rng = np.random.default_rng(123)
    A = rng.uniform(-1, 1, (M, K)) * 2.0 ** rng.integers(-8, 9, (M, K))
    B = rng.uniform(-1, 1, (K, N)) * 2.0 ** rng.integers(-8, 9, (K, N))
    lo, hi = row_block(M, rank, world)
    a_local = torch.from_numpy(A[lo:hi].copy())
    b = torch.from_numpy(B.copy()) if rank == src else None     # only the source rank holds B
    c_local = torch.zeros((hi - lo, N), dtype=torch.float64)
    eng = CheckerEngine(nm, K)
    op = RowShardedGemm(hi - lo, N, K, nm, src=src, panels=panels, engine=eng, device="cpu", layout=layout)
    op(a_local, b, c_local)
    op(a_local, b, c_local)                                     # a second call reuses the staging buffers
    np.save(os.path.join(out_dir, f"c{rank}.npy"), c_local.numpy())
    np.save(os.path.join(out_dir, f"calls{rank}.npy"), np.array(eng.calls))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("layout", ["rows", "panels"])
@pytest.mark.parametrize("src", [0, 1])
def test_two_ranks_match_the_unsharded_product(tmp_path, src, layout):
    import oracle_lib as o
    from ozaki_blackwell_b200.dist import panel_ranges, row_block
    M, N, K, nm, panels, world = 37, 600, 300, 16, 3, 2
    port = 29500 + (os.getpid() % 2000) + src + 2 * (layout == "rows")
    mp.spawn(_worker, args=(world, port, M, N, K, nm, panels, src, layout, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(123)
    A = rng.uniform(-1, 1, (M, K)) * 2.0 ** rng.integers(-8, 9, (M, K))
    B = rng.uniform(-1, 1, (K, N)) * 2.0 ** rng.integers(-8, 9, (K, N))
    want = o.dgemm(A, B, nm)
    got = np.vstack([np.load(tmp_path / f"c{r}.npy") for r in range(world)])
    assert np.array_equal(got.view(np.uint64), want.view(np.uint64))
    for r in range(world):
        calls = [tuple(c) for c in np.load(tmp_path / f"calls{r}.npy")]
        if layout == "panels":
            assert calls == [(lo, hi - lo) for lo, hi in panel_ranges(N, panels)] * 2
        else:
            assert calls == [(1 if r == src else panels, K)] * 2   # the source turns its own B into residues in one go
    assert row_block(M, 0, world) == (0, 19) and row_block(M, 1, world) == (19, 37)


def test_partition_helpers():
    from ozaki_blackwell_b200.dist import panel_ranges, row_block
    for m, w in ((8192, 8), (10, 4), (3, 8), (32768, 8)):
        blocks = [row_block(m, r, w) for r in range(w)]
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert max(h - l for l, h in blocks) - min(h - l for l, h in blocks) <= 1
    from ozaki_blackwell_b200.dist import choose_layout, row_chunks
    from ozaki_blackwell_b200.dist import growing_panels
    assert choose_layout(8192, 8192) == ("rows", 1) and choose_layout(32768, 32768) == ("panels", 0)
    assert growing_panels(32768) == [(0, 2048), (2048, 8192), (8192, 16384), (16384, 32768)]
    for n in (100, 256, 257, 1000, 5000, 12345):
        r = growing_panels(n)
        assert r[0][0] == 0 and r[-1][1] == n and all(a[1] == b[0] for a, b in zip(r, r[1:])) and all(lo % 256 == 0 for lo, _ in r)
    assert choose_layout(8192, 8192, "panels", 3) == ("panels", 3) and choose_layout(32768, 32768, "rows") == ("rows", 1)
    assert row_chunks(1000, 3) == [(0, 384), (384, 768), (768, 1000)] and row_chunks(100, 5) == [(0, 100)]
    for n, p in ((8192, 8), (8192, 1), (300, 4), (1000, 3), (256, 8), (32768, 16), (257, 2)):
        r = panel_ranges(n, p)
        assert r[0][0] == 0 and r[-1][1] == n and len(r) <= max(p, 1)
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(lo % 256 == 0 for lo, _ in r) and all(hi > lo for lo, hi in r)


def _worker_with_a_missing_rank(rank, world, port, out_dir):
    """Rank 1 leaves before the product; rank 0's broadcast must end with an error after the group's short timeout."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from ozaki_blackwell_b200.dist import RowShardedGemm
    if rank == 1:
        os._exit(0)                                             # gone, between steps, with nothing of its own in flight
    op = RowShardedGemm(4, 300, 32, 16, src=0, panels=2, engine=CheckerEngine(16), device="cpu")
    a, b, c = torch.ones((4, 32), dtype=torch.float64), torch.ones((32, 300), dtype=torch.float64), torch.zeros((4, 300), dtype=torch.float64)
    try:
        op(a, b, c)
        outcome = "completed"
    except Exception as e:   # the failure surfaces on the host as an exception, not as a hang
        outcome = "error: " + type(e).__name__
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_a_vanished_rank_becomes_an_error_not_a_hang(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker_with_a_missing_rank, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    [p.start() for p in procs]
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "a rank is still waiting for the one that left"
    outcome = (tmp_path / "outcome.txt").read_text()
    assert outcome.startswith("error"), outcome
