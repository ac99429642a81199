"""What the host link gives each GPU of a job: run as the ranks of the job (one per GPU) and compare with the end-to-end
numbers of `bench.py`. Every rank copies 1 GiB from pinned host memory to its GPU: alone (the ranks take turns), all ranks
at once, and all at once while each also copies 0.5 GiB back. Prints GB/s per rank.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m ozaki_blackwell_b200.host_link_probe
"""
import os
import time

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl")
    barrier = dist.barrier if world > 1 else (lambda: None)
    up_h = torch.ones(1 << 27, dtype=torch.float64).pin_memory()
    up_d = torch.empty(1 << 27, dtype=torch.float64, device="cuda")
    down_h = torch.empty(1 << 26, dtype=torch.float64).pin_memory()
    down_d = torch.ones(1 << 26, dtype=torch.float64, device="cuda")
    side = torch.cuda.Stream()
    gb = up_h.numel() * 8 / 1e9

    def rate(back_too, reps=3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            up_d.copy_(up_h, non_blocking=True)
            if back_too:
                with torch.cuda.stream(side):
                    down_h.copy_(down_d, non_blocking=True)
        torch.cuda.synchronize()
        return gb * reps / (time.perf_counter() - t0)

    rate(False, 1)
    alone = 0.0
    for r in range(world):
        barrier()
        if r == rank:
            alone = rate(False)
        barrier()
    barrier()
    together = rate(False)
    barrier()
    both_ways = rate(True)
    mine = torch.tensor([alone, together, both_ways], dtype=torch.float64, device="cuda")
    every = [torch.empty_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(every, mine)
    else:
        every = [mine]
    if rank == 0:
        for r, v in enumerate(every):
            a, t, b = (float(x) for x in v)
            print(f"rank {r}: host to GPU {a:.1f} GB/s alone, {t:.1f} GB/s with all ranks at once, {b:.1f} GB/s while every rank also copies back")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
