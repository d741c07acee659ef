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
    # reductions over the sharded axis carry the exchange themselves: one launch
    # each, results equal to the unsharded reduction over all ranks' rows
    from numba_mlir_b200 import reduce_ops, workloads

    def shard(r, call):
        return np.random.default_rng(77 * call + r).standard_normal((1000 + 8 * r, 4096)).astype(np.float32)

    def ints(r, call):
        return np.random.default_rng(55 * call + r).integers(-1000, 1001, (1 << 20) + r).astype(np.int32)

    with sharding.across(dist, queue):
        for call in range(1, 7):
            a = nm.from_host(shard(rank, call), queue)
            out = nm.empty(4096, np.float32, queue)
            before = runtime.launch_count()
            workloads.min_axis0(a, out)
            launched = runtime.launch_count() - before
            whole = np.concatenate([shard(r, call) for r in range(world)])
            if launched != 1 or not np.array_equal(out.copy_to_host(), whole.min(axis=0)):
                print(f"rank {rank}: sharded min(axis=0) wrong at call {call} ({launched} launches)")
                sys.exit(1)
            total = nm.empty((), np.int64, queue)
            workloads.total(nm.from_host(ints(rank, call), queue), total)
            want = sum(int(ints(r, call).sum(dtype=np.int64)) for r in range(world))
            if int(total.copy_to_host()) != want:
                print(f"rank {rank}: sharded integer sum wrong at call {call}")
                sys.exit(1)
            s = reduce_ops.reduce(a, "sum", 0)  # merge-tree path, float sums in rank order
            parts = [shard(r, call).astype(np.float64).sum(axis=0) for r in range(world)]
            if not np.allclose(s.copy_to_host(), sum(parts), rtol=1e-4, atol=1e-2):
                print(f"rank {rank}: sharded sum(axis=0) wrong at call {call}")
                sys.exit(1)
    # the sums and counts of a k-means step behind one flag
    sums = nm.from_host(np.random.default_rng(rank).standard_normal((64, 16)), queue)
    counts = nm.from_host(np.arange(64, dtype=np.int64) * (rank + 1), queue)
    before = runtime.launch_count()
    sharding.allreduce_many([(sums, "sum"), (counts, "sum")], dist)
    if runtime.launch_count() - before != 1:
        print(f"rank {rank}: allreduce_many took more than one launch")
        sys.exit(1)
    want = sum(np.random.default_rng(r).standard_normal((64, 16)) for r in range(world))
    if not np.array_equal(sums.copy_to_host(), want) or \
            not np.array_equal(counts.copy_to_host(), np.arange(64) * (world * (world + 1) // 2)):
        print(f"rank {rank}: allreduce_many wrong")
        sys.exit(1)
    queue.check_status()
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
