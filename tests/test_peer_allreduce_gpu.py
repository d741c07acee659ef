"""The peer-memory all-reduce (csrc/kernels/peer_exchange.cuh, peer_allreduce.cu).

On one GPU the ranks are not run as separate launches (they would wait on one
another); what the peers would have pushed into this rank's mailbox is written
there from the host before the one launch under test, which then finds every
word already tagged.  With two or more GPUs the real exchange runs as one
process per GPU."""

import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = 256
SLOT = 65536            # payload bytes a call can carry
REGION = 2 * SLOT       # the same payload as tagged 8-byte words
MAX_RANKS = 16
MAILBOX = HEADER + 2 * MAX_RANKS * REGION


def _mailboxes(world):
    import numba_mlir_b200 as nm

    return [nm.zeros(MAILBOX, np.uint8) for _ in range(world)]


def _region(seq, src):
    return HEADER + ((seq & 1) * MAX_RANKS + src) * REGION


def _post(box, mirror, seq, src, payload, off=0):
    """What rank `src` pushes into the mailbox `box` for call `seq`: every
    4-byte word of its payload with the call number in the upper half
    (`mirror` is the host copy of the mailbox, kept between calls)."""
    words = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
    words = np.concatenate([words, np.zeros(-words.size % 4, np.uint8)]).view(np.uint32)
    tagged = (np.uint64(seq & 0xFFFFFFFF) << np.uint64(32)) | words.astype(np.uint64)
    start = _region(seq, src) + 2 * off
    mirror[start: start + tagged.nbytes] = tagged.view(np.uint8)
    box.copy_from_host(mirror)


def _launch(queue, op, ty, data, table, rank, world):
    """The rank's own mailbox counts its calls: launch number k is call k."""
    k = queue.builtin(f"nmb_peer_allreduce_{op}_{ty}")
    queue.launch(k, (1,), (1024,),
                 [("ptr", data.ptr), np.int64(data.size), ("ptr", table.ptr), np.int32(rank),
                  np.int32(world), ("ptr", queue.status_ptr)])


def _combine(parts, op):
    want = parts[0].copy()
    for p in parts[1:]:  # rank order, the kernel's own order
        if op == "sum":
            want = want + p
        elif op == "min":
            want = np.where(p < want, p, want)
        else:
            want = np.where(want < p, p, want)
    return want


_TYPES = {"f32": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64}


@pytest.mark.parametrize("op", ["sum", "min", "max"])
@pytest.mark.parametrize("ty", sorted(_TYPES))
def test_combines_all_ranks_in_rank_order(queue, op, ty):
    import numba_mlir_b200 as nm

    world, rank, n = 4, 2, 4099
    dt = _TYPES[ty]
    rng = np.random.default_rng(7)
    boxes = _mailboxes(world)
    mirror = np.zeros(MAILBOX, np.uint8)
    table = nm.from_host(np.asarray([b.ptr for b in boxes], np.uint64))
    for seq in (1, 2, 3):  # slots 1, 0, 1: the second use of a slot overwrites the first
        parts = [(rng.standard_normal(n) * 1000).astype(dt) for _ in range(world)]
        mirror[0:8] = np.asarray([seq - 1], np.uint64).view(np.uint8)  # the rank's own call counter so far
        for r in range(world):
            if r != rank:
                _post(boxes[rank], mirror, seq, r, parts[r])
        data = nm.from_host(parts[rank])
        _launch(queue, op, ty, data, table, rank, world)
        assert np.array_equal(data.copy_to_host(), _combine(parts, op))
        mine = boxes[rank].copy_to_host()
        assert mine[0:8].view(np.uint64)[0] == seq  # the call counter advanced
        # every peer's mailbox holds this rank's partial as words tagged with the call number
        for r in range(world):
            if r != rank:
                got = boxes[r].copy_to_host()[_region(seq, rank): _region(seq, rank) + 2 * parts[rank].nbytes]
                got = got.view(np.uint64)
                assert np.all(got >> np.uint64(32) == seq)
                assert np.array_equal((got & np.uint64(0xFFFFFFFF)).astype(np.uint32),
                                      parts[rank].view(np.uint32))
    queue.check_status()


class _FakeGroup:
    """Stands for sharding.PeerGroup on one GPU: the mailbox table and this
    process's place among the ranks."""

    def __init__(self, table, rank, world):
        self.table, self.rank, self.world = table, rank, world


class _FakeExchange:
    slot_bytes = SLOT

    def __init__(self, group):
        self.group = group

    def allreduce(self, out, op):
        raise AssertionError("the reduction was expected to carry the exchange itself")


@pytest.mark.parametrize("case", ["min_axis0", "max_axis0_one_row_block", "sum_axis0", "int_sum_all",
                                  "min_all_f32"])
def test_reduction_kernels_finish_with_the_exchange(queue, case):
    """A reduction over the sharded axis inside `sharding.across` is ONE launch:
    the block that completes the reduction publishes the result, waits for
    the peers' flags and combines all ranks' results in rank order.  Here the
    peers' results are posted from the host before the launch."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import reduce_ops, runtime

    world, rank = 3, 1
    rng = np.random.default_rng(21)
    boxes = _mailboxes(world)
    mirror = np.zeros(MAILBOX, np.uint8)
    table = nm.from_host(np.asarray([b.ptr for b in boxes], np.uint64))
    queue.shard_exchange = _FakeExchange(_FakeGroup(table, rank, world))
    try:
        for seq in (1, 2, 3):
            if case == "min_axis0":
                a, op, axis = rng.standard_normal((3000, 4096)).astype(np.float32), "min", 0
            elif case == "max_axis0_one_row_block":
                a, op, axis = rng.standard_normal((3, 2048)).astype(np.float32), "max", 0
            elif case == "sum_axis0":
                a, op, axis = rng.integers(-9, 10, (2000, 512)).astype(np.int32), "sum", 0
            elif case == "int_sum_all":
                a, op, axis = rng.integers(-1000, 1001, 1 << 22).astype(np.int32), "sum", None
            else:
                a, op, axis = rng.standard_normal(100003).astype(np.float32), "min", None
            mine = getattr(np, op)(a.astype(np.int64) if a.dtype == np.int32 else a, axis=axis)
            mine = np.asarray(mine)
            parts = [(mine + (r - rank) * 3).astype(mine.dtype) if a.dtype == np.int32
                     else (mine + np.float32(0.25) * (r - rank) * np.sign(rng.standard_normal(mine.shape))).astype(mine.dtype)
                     for r in range(world)]
            parts[rank] = mine
            mirror[0:8] = np.asarray([seq - 1], np.uint64).view(np.uint8)
            for r in range(world):
                if r != rank:
                    _post(boxes[rank], mirror, seq, r, np.ascontiguousarray(parts[r]).reshape(-1))
            before = runtime.launch_count()
            got = reduce_ops.reduce(nm.from_host(a), op, axis)
            assert runtime.launch_count() == before + 1
            assert np.array_equal(got.copy_to_host(), _combine(parts, op))
        queue.check_status()
    finally:
        queue.shard_exchange = None


def test_several_partials_behind_one_flag(queue):
    """nmb_peer_allreduce_multi: float64 sums and int64 counts (a k-means
    step's partials) plus a float32 minimum in one launch."""
    import numba_mlir_b200 as nm

    world, rank = 4, 0
    rng = np.random.default_rng(22)
    boxes = _mailboxes(world)
    mirror = np.zeros(MAILBOX, np.uint8)
    table = nm.from_host(np.asarray([b.ptr for b in boxes], np.uint64))
    k = queue.builtin("nmb_peer_allreduce_multi")
    for seq in (1, 2):
        sums = [rng.standard_normal((64, 16)) * 1e5 for _ in range(world)]
        counts = [rng.integers(0, 1 << 40, 64) for _ in range(world)]
        mins = [rng.standard_normal(7).astype(np.float32) for _ in range(world)]
        mirror[0:8] = np.asarray([seq - 1], np.uint64).view(np.uint8)
        for r in range(1, world):
            payload = np.zeros(64 * 16 * 8 + 64 * 8 + 32, np.uint8)
            payload[:8192] = sums[r].view(np.uint8).reshape(-1)
            payload[8192:8704] = counts[r].view(np.uint8)
            payload[8704:8704 + 28] = mins[r].view(np.uint8)
            _post(boxes[rank], mirror, seq, r, payload)
        d_s, d_c, d_m = nm.from_host(sums[0]), nm.from_host(counts[0]), nm.from_host(mins[0])
        queue.launch(k, (1,), (1024,),
                     [("ptr", d_s.ptr), np.int64(1024), np.int32(1 + 4 * 0),
                      ("ptr", d_c.ptr), np.int64(64), np.int32(3 + 4 * 0),
                      ("ptr", d_m.ptr), np.int64(7), np.int32(0 + 4 * 1),
                      ("ptr", 0), np.int64(0), np.int32(0),
                      ("ptr", table.ptr), np.int32(rank), np.int32(world), ("ptr", queue.status_ptr)])
        assert np.array_equal(d_s.copy_to_host(), _combine(sums, "sum"))
        assert np.array_equal(d_c.copy_to_host(), _combine(counts, "sum"))
        assert np.array_equal(d_m.copy_to_host(), _combine(mins, "min"))
    queue.check_status()


def test_missing_peer_runs_out_and_reports(queue):
    """Words that nothing sends: the wait gives up after its bound (about two
    seconds), the status word is raised and the data are left as they were."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200.runtime import GpuRuntimeError

    world, rank, n = 2, 0, 100
    boxes = _mailboxes(world)
    table = nm.from_host(np.asarray([b.ptr for b in boxes], np.uint64))
    part = np.arange(n, dtype=np.float32)
    data = nm.from_host(part)
    _launch(queue, "sum", "f32", data, table, rank, world)
    with pytest.raises(GpuRuntimeError):
        queue.check_status()
    assert np.array_equal(data.copy_to_host(), part)
    queue.check_status()  # the status word was cleared: the queue stays usable


def test_bad_arguments_are_reported_not_run(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200.runtime import GpuRuntimeError

    boxes = _mailboxes(1)
    table = nm.from_host(np.asarray([boxes[0].ptr], np.uint64))
    data = nm.zeros(8, np.float32)
    k = queue.builtin("nmb_peer_allreduce_sum_f32")
    for n, rank, world in ((20000, 0, 1), (8, 1, 1), (8, 0, 17)):  # > 64 KB, rank >= world, world > 16
        queue.launch(k, (1,), (1024,), [("ptr", data.ptr), np.int64(n), ("ptr", table.ptr), np.int32(rank),
                                        np.int32(world), ("ptr", queue.status_ptr)])
        with pytest.raises(GpuRuntimeError):
            queue.check_status()


def test_ranks_on_separate_gpus_agree():
    """One process per GPU: sum, min and max of float32 / float64 / int64
    partials through sharding.allreduce, many calls in a row (both slots reused),
    results equal to the host's rank-ordered combination on every rank."""
    import torch

    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs two GPUs")
    world = min(n_gpus, 4)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29671",
           os.path.join(ROOT, "tests", "peer_allreduce_ranks.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("PEER-ALLREDUCE-OK") == world, res.stdout[-3000:] + res.stderr[-3000:]
