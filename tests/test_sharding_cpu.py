"""World-size-2 gloo runs (CPU) of the row sharding and the three exchanges
the sharded workloads need: the sharded result must equal the unsharded one."""

import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_range_is_a_balanced_partition():
    from numba_mlir_b200.sharding import row_range

    for n in (0, 1, 7, 16384, 2**22 + 3):
        for world in (1, 2, 3, 8):
            spans = [row_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_peer_exchange_takes_only_what_fits_a_mailbox_slot(monkeypatch):
    """Which partials the peer-memory all-reduce accepts (the rest go through
    torch.distributed), and the switch that turns the path off; host-side
    logic only, no device."""
    from numba_mlir_b200 import lazy, sharding

    queue = object()
    group = sharding.PeerGroup.__new__(sharding.PeerGroup)
    group.ok, group.queue = True, queue

    def part(shape, dtype, q=queue):
        a = lazy.fake_array(shape, dtype)
        a._buf.queue = q
        return a

    assert group.accepts(part((4096,), np.float32))       # 16 KB column minima
    assert group.accepts(part((), np.int64))              # a full sum
    assert group.accepts(part((64, 16), np.float64))      # k-means sums
    assert group.accepts(part((16384,), np.float32))      # exactly one slot
    assert not group.accepts(part((16385,), np.float32))  # above 64 KB
    assert not group.accepts(part((0,), np.float32))
    assert not group.accepts(part((64,), np.int16))       # no kernel for the type
    assert not group.accepts(part((64, 16), np.float64).T)
    assert not group.accepts(part((64,), np.float32, q=object()))  # another queue
    group.ok = False
    assert not group.accepts(part((64,), np.float32))
    monkeypatch.setenv("NUMBA_MLIR_B200_PEER_ALLREDUCE", "0")
    assert sharding.peer_group(queue, None) is None       # returns before touching `dist`


_WORKER = textwrap.dedent(
    """
    import os, sys
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, %(root)r)
    from numba_mlir_b200.sharding import allreduce, shard_rows
    from oracle import configs as O

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    # full int64 sum of an int32 vector (bit-exact)
    (a,) = O.make_inputs("reduce_i32", 1 / 1024)
    part = np.array(shard_rows(a, world, rank).sum(dtype=np.int64))
    allreduce(part, "sum", dist)
    assert int(part) == int(a.sum(dtype=np.int64))

    # min over axis 0 of a row-sharded matrix (bit-exact)
    (m,) = O.make_inputs("reduce_f32", 1 / 256)
    pm = O.min_axis0(np.ascontiguousarray(shard_rows(m, world, rank)))
    allreduce(pm, "min", dist)
    assert np.array_equal(pm, m.min(axis=0))

    # two k-means iterations with sharded points: labels of the shard and the
    # centroids equal the single-process oracle
    pts, c0 = O.make_inputs("kmeans", 1 / 256)
    mine = np.ascontiguousarray(shard_rows(pts, world, rank))
    cent = c0.copy()
    labels = np.zeros(mine.shape[0], np.int32)
    for _ in range(2):
        O.kmeans_assign(mine, cent, labels)
        sums = np.zeros(cent.shape, np.float64)
        counts = np.zeros(cent.shape[0], np.int64)
        O.kmeans_accumulate(mine, labels, sums, counts)
        allreduce(sums, "sum", dist)
        allreduce(counts, "sum", dist)
        cent = O.kmeans_update(cent, sums, counts)
    want_labels, want_cent = O.kmeans(pts, c0, 2)
    from numba_mlir_b200.sharding import row_range
    b, e = row_range(pts.shape[0], world, rank)
    assert np.array_equal(labels, want_labels[b:e])
    # float64 partial sums meet in a different order: equal after rounding
    assert np.array_equal(cent, want_cent)
    dist.barrier()
    dist.destroy_process_group()
    os.write(1, ("rank " + str(rank) + " ok" + chr(10)).encode())  # one write: the ranks share the pipe
    """
)


def test_sharded_reductions_and_kmeans_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER % {"root": ROOT})
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    env = dict(os.environ, OMP_NUM_THREADS="2", NUMBA_NUM_THREADS="2")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "rank 0 ok" in proc.stdout and "rank 1 ok" in proc.stdout
