"""Rank program of test_peer_allreduce_gpu.py::test_ranks_on_separate_gpus_agree
(launched with torch.distributed.run, one process per GPU)."""

import os
import sys

import numpy as np


def part_of(rank, n, dtype, call):
    rng = np.random.default_rng(1000 * call + rank)
    return (rng.standard_normal(n) * 100).astype(dtype)


def main():
    import torch
    import torch.distributed as dist

    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime, sharding

    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    rank, world = dist.get_rank(), dist.get_world_size()
    queue = runtime.get_queue()
    call = 0
    for n, dtype in ((4096, np.float32), (1024 + 64, np.float64), (1, np.int64), (16384, np.float32)):
        for op in ("sum", "min", "max"):
            for _ in range(5):
                call += 1
                d = nm.from_host(part_of(rank, n, dtype, call), queue)
                sharding.allreduce(d, op, dist)
                want = part_of(0, n, dtype, call)
                for r in range(1, world):
                    p = part_of(r, n, dtype, call)
                    want = want + p if op == "sum" else (np.where(p < want, p, want) if op == "min"
                                                         else np.where(want < p, p, want))
                got = d.copy_to_host()
                if not np.array_equal(got, want):
                    print(f"rank {rank}: mismatch at call {call} ({op}, {np.dtype(dtype).name}, n={n})")
                    sys.exit(1)
    queue.check_status()
    group = sharding.peer_group(queue, dist)
    if group is None or group.seq != call:
        print(f"rank {rank}: the peer-memory path was not used")
        sys.exit(1)
    # a partial above the mailbox size takes the library collective
    big = nm.from_host(np.full(40000, rank + 1, np.float32), queue)
    sharding.allreduce(big, "sum", dist)
    queue.synchronize()
    torch.cuda.synchronize()
    assert np.all(big.copy_to_host() == world * (world + 1) / 2)
    dist.barrier()
    os.write(1, b"PEER-ALLREDUCE-OK\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
