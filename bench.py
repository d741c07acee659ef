#!/usr/bin/env python
"""Benchmark of the numba-mlir offload path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
                    [--workload NAME] [--no-extra] [--no-cpu] [--profile]

One "step" is one pass of the hot path over one batch of synthetic input.  The
headline workload is the Black-Scholes fused ufunc chain over 2^24 float32
options per GPU (20 algorithmic bytes per option), called through the
`njit(parallel=True)` decorator; the metric is effective HBM GB/s =
algorithmic bytes / device time, whole job over all N GPUs (weak scaling: every
GPU holds a full-size shard, the workloads shard along axis 0).  Inputs and
outputs (320 MB per GPU) exceed the 126 MB L2, so no flush is needed between
iterations; workloads whose operands fit L2 rotate over enough operand sets to
exceed twice its size.  Rank 0 prints ONE JSON line.  With one GPU the line
also carries a device-time table for the other benchmark configurations
("other_configs"), end-to-end legs for a row reduction and the distance matrix,
and the host cost of a launch; with several GPUs "other_configs" holds the
three workloads whose shards exchange partial results (column minimum, integer
sum, k-means), each as weak scaling (a full-size shard per GPU) and strong
scaling (the fixed configuration split N ways).  Every workload's output is
compared with the CPU oracle outside the timed region; a mismatch aborts.

The timed block of K steps is repeated until at least 50 ms of device time
have been measured and the median block is reported.

`--impl reference` times the CPU implementation of the same workload (upstream
Numba njit(parallel=True), which is what the reference's njit is with its MLIR
pipeline off) on the host cores.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "effective_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
L2_BYTES = 126 << 20
MIN_TIMED_MS = 50.0
f32 = np.float32

HOST_BUFFERS_NOTE = ("e2e: inputs start in page-locked host arrays and results end in page-locked host arrays "
                     "(the copy of a pageable user array into them is outside the timed region); the CPU arm "
                     "reads and writes ordinary host arrays")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs"), "measured"
    return 6650.0, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant
# kernel, from the ncu captures summarised under profiles/ (scaled to the full
# workload where the capture ran a smaller case).
NCU_TRAFFIC_BYTES = {
    "black_scholes": 201362432 + 90091008,   # output partly still dirty in L2 at kernel end
    "bcast_add": 16797184 + 0,               # two-launch capture: the result stays in L2
    "sum_axis1": 268446208 + 3861760,        # the few MB of writes are evictions of the previous launch's lines
    "min_axis0": 268525568 + 3505408,
    "argmin_axis1": 268448000 + 4131840,
    "row_norm": 268450048 + 5443072,
    "int_sum": 1073772000 + 4045312,
    "pairwise": 27907072 + 1015498000,       # nmb_contract_tf32x3 (prepass: 8409856 + 0)
    "kmeans": 268472832 + 15567360,
}


def config_of(name, units):
    """The `config` object, identical for the GPU arm and the CPU arm."""
    return {"workload": name, "elements_per_step_per_gpu": int(units), "host_buffers": HOST_BUFFERS_NOTE}


def rotation_sets(bytes_per_set):
    """Operand sets a step rotates over so that consecutive steps never find
    their inputs in L2: the sets together exceed twice the L2 size."""
    return 1 if bytes_per_set > L2_BYTES else int(-(-2 * L2_BYTES // max(bytes_per_set, 1))) + 1


# ------------------------------------------------------------- workloads ----
class Workload:
    """One benchmark configuration.  Sub-classes provide host inputs, the
    device-resident step, optionally an end-to-end step, and `check`, which
    compares one step's output with the CPU oracle (outside any timed region).

    `fraction` is the part of the configuration's leading dimension that one
    GPU holds (1 for a full-size shard)."""

    key = name = dtype = ""
    bytes_per_step = units_per_step = 0
    launches_per_step = 1
    graph_steps = 1
    exchange = None  # what crosses the shards each step, if anything

    def setup_device(self, queue, seed, dist=None):
        raise NotImplementedError

    def step_device(self):
        raise NotImplementedError

    def check(self, dist=None):
        raise NotImplementedError


def _rank_world(dist):
    if dist is None:
        return 0, 1
    return dist.get_rank(), dist.get_world_size()


def _gather_host(dist, array, queue):
    """Every rank's copy of a small host array, in rank order (through the
    process group's device collective)."""
    if dist is None:
        return [array]
    import torch

    t = torch.from_numpy(np.ascontiguousarray(array)).cuda(queue.device)
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t)
    return [p.cpu().numpy() for p in parts]


class BlackScholes(Workload):
    """Config: N = 2^24 float32 options per GPU; spot, strike ~ U[10,50],
    expiry ~ U[1,2], rate 0.1, volatility 0.2; outputs call and put."""

    name = "black_scholes_f32_n2^24"
    key = "black_scholes"
    n = 1 << 24
    bytes_per_step = 20 * n  # 3 float32 reads + 2 float32 writes per option
    units_per_step = n
    dtype = "f32"
    fastmath = False

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        return (rng.uniform(10, 50, self.n).astype(f32), rng.uniform(10, 50, self.n).astype(f32),
                rng.uniform(1, 2, self.n).astype(f32), f32(0.1), f32(0.2))

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm
        from numba_mlir_b200 import workloads

        price, strike, t, self.rate, self.vol = self.host = self.host_inputs(seed)
        self.fn = workloads.black_scholes_fastmath if self.fastmath else workloads.black_scholes
        self.queue = queue
        self.h_in = [nm.pinned_empty(self.n, f32, queue) for _ in range(3)]
        for dst, src in zip(self.h_in, (price, strike, t)):
            dst[:] = src
        self.h_out = [nm.pinned_empty(self.n, f32, queue) for _ in range(2)]
        self.d_in = [nm.from_host(x, queue) for x in (price, strike, t)]
        self.d_out = [nm.empty(self.n, f32, queue) for _ in range(2)]
        self.h2d_bytes = 3 * 4 * self.n
        self.d2h_bytes = 2 * 4 * self.n

    def step_device(self):
        self.fn(*self.d_in, self.rate, self.vol, *self.d_out)

    def step_e2e(self):
        """Host buffers in, host buffers out, through the public API: the
        chunked pipeline overlaps copy-in, kernels and copy-out."""
        import numba_mlir_b200 as nm

        nm.map_host(self.fn, self.h_in, self.h_out, scalars=(self.rate, self.vol), queue=self.queue)

    def check(self, dist=None):
        from oracle import configs as O

        price, strike, t, rate, vol = self.host
        for o in self.d_out:
            self.queue.memset(o.ptr, 0, o.nbytes)
        self.step_device()
        call, put = (o.copy_to_host() for o in self.d_out)
        if self.fastmath:
            wcall, wput = O.black_scholes_f64(price, strike, t, rate, vol)
            tol = dict(rtol=1e-5, atol=4e-5)
        else:
            wcall, wput = np.zeros_like(price), np.zeros_like(price)
            O.black_scholes(price, strike, t, rate, vol, wcall, wput)
            tol = dict(rtol=1e-5, atol=2e-5)
        np.testing.assert_allclose(call, wcall, **tol)
        np.testing.assert_allclose(put, wput, **tol)
        if hasattr(self, "h_out") and getattr(self, "e2e_ran", False):
            np.testing.assert_allclose(np.asarray(self.h_out[0]), wcall, **tol)
            np.testing.assert_allclose(np.asarray(self.h_out[1]), wput, **tol)


class BlackScholesFastmath(BlackScholes):
    """The same chain compiled with fastmath=True, the flags of the
    reference's benchmark driver (numba_mlir/mlir/benchmarking.py:43).  A
    secondary line: the headline keeps the default (IEEE division and sqrt)."""

    name = "black_scholes_f32_n2^24_fastmath"
    key = "black_scholes_fastmath"
    fastmath = True


class BroadcastAdd(Workload):
    """a (2048, 2048) + b (1, 2048), float32; 33.6 MB per call fits L2, so the
    step rotates over 10 operand/result sets (336 MB)."""

    name = "broadcast_add_f32_2048x2048"
    key = "bcast_add"
    bytes_per_step = 33562624
    units_per_step = 2048 * 2048
    dtype = "f32"

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm

        rng = np.random.default_rng(seed)
        self.host_a = rng.uniform(-1, 1, (2048, 2048)).astype(f32)
        self.host_b = rng.uniform(-1, 1, (1, 2048)).astype(f32)
        self.sets = [nm.from_host(self.host_a, queue)]
        self.sets += [nm.from_host(rng.uniform(-1, 1, (2048, 2048)).astype(f32), queue) for _ in range(9)]
        self.b = nm.from_host(self.host_b, queue)
        self.outs = [nm.empty((2048, 2048), f32, queue) for _ in range(10)]
        self.i = 0

    # a recorded graph must cover one full rotation to keep the working set >L2
    # (a step count that is not a multiple of it is launched eagerly instead)
    graph_steps = 10

    def step_device(self):
        from numba_mlir_b200 import workloads

        workloads.broadcast_add(self.sets[self.i % 10], self.b, self.outs[self.i % 10])
        self.i += 1

    def check(self, dist=None):
        from oracle import configs as O

        self.i = 0
        self.step_device()
        want = O.bcast_add(self.host_a, self.host_b)
        assert np.array_equal(self.outs[0].copy_to_host().view(np.uint32), want.view(np.uint32)), \
            "broadcast add differs from the oracle"


class AxisReduction(Workload):
    """float32 (16384, 4096) ~ N(0,1): sum(axis=1), min(axis=0), argmin(axis=1),
    and sqrt(sum(a*a, axis=1)) (a reduction fed by an elementwise chain).
    With `fraction` < 1 the GPU holds that part of the rows and the step
    rotates over several shards' worth of data to stay out of L2."""

    dtype = "f32"

    def __init__(self, which, fraction=1.0):
        self.which = which
        self.key = which
        self.rows = max(8, int(16384 * fraction))
        self.name = f"{which}_f32_{self.rows}x4096"
        self.units_per_step = self.rows * 4096
        out_bytes = {"sum_axis1": 4 * self.rows, "min_axis0": 4 * 4096, "argmin_axis1": 8 * self.rows,
                     "row_norm": 4 * self.rows}[which]
        self.bytes_per_step = self.rows * 4096 * 4 + out_bytes
        self.graph_steps = rotation_sets(self.rows * 4096 * 4)
        if which == "min_axis0":
            self.exchange = "all-reduce(min) of 4096 float32 column minima (16 KB)"

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm
        from numba_mlir_b200 import workloads

        rng = np.random.default_rng(seed)
        self.queue = queue
        self.host = rng.standard_normal((self.rows, 4096)).astype(f32)
        self.sets = [nm.from_host(self.host, queue)]
        for _ in range(self.graph_steps - 1):
            self.sets.append(nm.from_host(rng.standard_normal((self.rows, 4096)).astype(f32), queue))
        self.fn = getattr(workloads, self.which)
        self.dist = dist if self.which == "min_axis0" else None
        shape, dt = {"sum_axis1": (self.rows, f32), "min_axis0": (4096, f32),
                     "argmin_axis1": (self.rows, np.int64), "row_norm": (self.rows, f32)}[self.which]
        self.out = nm.empty(shape, dt, queue)
        self.i = 0
        if self.which == "sum_axis1" and dist is None:
            self.h_in = nm.pinned_empty((self.rows, 4096), f32, queue)
            self.h_in[:] = self.host
            self.h_out = nm.pinned_empty(self.rows, f32, queue)
            self.h2d_bytes, self.d2h_bytes = self.h_in.nbytes, self.h_out.nbytes
            self.step_e2e = self._step_e2e

    def _step_e2e(self):
        import numba_mlir_b200 as nm

        nm.map_host(self.fn, [self.h_in], [self.h_out], queue=self.queue)

    def step_device(self):
        from numba_mlir_b200 import sharding

        # rows are sharded: inside `across` the column minima of all GPUs meet
        # in the reduction kernel's last block (one launch per step)
        with sharding.across(self.dist, self.queue):
            self.fn(self.sets[self.i % len(self.sets)], self.out)
        self.i += 1

    def check(self, dist=None):
        from oracle import configs as O

        self.i = 0
        self.step_device()
        got = self.out.copy_to_host()
        a = self.host
        if self.which == "sum_axis1":
            truth = a.astype(np.float64).sum(axis=1)
            scale = np.abs(a).astype(np.float64).sum(axis=1)
            assert np.all(np.abs(got.astype(np.float64) - truth) <= 1e-5 * scale), "sum(axis=1) out of tolerance"
            if getattr(self, "e2e_ran", False):
                assert np.array_equal(np.asarray(self.h_out).view(np.uint32), got.view(np.uint32))
        elif self.which == "argmin_axis1":
            assert np.array_equal(got, O.argmin_axis1(a)), "argmin(axis=1) differs from the oracle"
        elif self.which == "row_norm":
            truth = np.sqrt((a.astype(np.float64) ** 2).sum(axis=1))
            np.testing.assert_allclose(got, truth, rtol=1e-5)
            np.testing.assert_allclose(O.row_norm(a), truth, rtol=1e-5)
        else:
            # the unsharded result: the shards' oracle minima combined in rank
            # order with the same select(x < m) the oracle applies row by row
            want = None
            for part in _gather_host(self.dist, O.min_axis0(a), self.queue):
                want = part if want is None else np.where(part < want, part, want)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "min(axis=0) differs from the oracle"


class IntSum(Workload):
    """np.sum over 2^28 int32 in [-1000, 1000], int64 accumulation (bit-exact)."""

    key = "int_sum"
    dtype = "int64"
    exchange = "all-reduce(sum) of one int64 (8 B)"

    def __init__(self, fraction=1.0):
        self.n = max(1024, int((1 << 28) * fraction))
        self.name = "int32_sum_n2^28" if fraction == 1.0 else f"int32_sum_n{self.n}"
        self.bytes_per_step = 4 * self.n + 8
        self.units_per_step = self.n
        self.graph_steps = rotation_sets(4 * self.n)

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm
        from numba_mlir_b200 import workloads

        rng = np.random.default_rng(seed)
        self.queue = queue
        self.host = rng.integers(-1000, 1001, self.n, dtype=np.int32)
        self.sets = [nm.from_host(self.host, queue)]
        for _ in range(self.graph_steps - 1):
            self.sets.append(nm.from_host(rng.integers(-1000, 1001, self.n, dtype=np.int32), queue))
        self.fn = workloads.total
        self.dist = dist
        self.out = nm.empty((), np.int64, queue)
        self.i = 0

    def step_device(self):
        from numba_mlir_b200 import sharding

        with sharding.across(self.dist, self.queue):
            self.fn(self.sets[self.i % len(self.sets)], self.out)
        self.i += 1

    def check(self, dist=None):
        from oracle import configs as O

        self.i = 0
        self.step_device()
        got = int(self.out.copy_to_host())
        mine = np.array([int(O.int_sum(self.host))], np.int64)
        want = sum(int(p[0]) for p in _gather_host(self.dist, mine, self.queue))
        assert got == want, f"integer sum {got} differs from the oracle's {want}"


def pairwise_njit():
    """The distance matrix as a user writes it against the decorators."""
    from numba_mlir_b200 import workloads

    return workloads.pairwise_distance


class Pairwise(Workload):
    """X, Y float32 (16384, 64) ~ U[0,1]; D (16384, 16384) float32, 1 GiB out."""

    name = "pairwise_distance_f32_16384x16384x64"
    key = "pairwise"
    dtype = "f32 (3xTF32 tensor cores)"
    bytes_per_step = 1082130432
    units_per_step = 16384 * 16384
    launches_per_step = 2

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm

        rng = np.random.default_rng(seed)
        self.queue = queue
        self.host_x = rng.uniform(0, 1, (16384, 64)).astype(f32)
        self.host_y = rng.uniform(0, 1, (16384, 64)).astype(f32)
        self.x = nm.from_host(self.host_x, queue)
        self.y = nm.from_host(self.host_y, queue)
        self.d = nm.empty((16384, 16384), f32, queue)
        self.fn = pairwise_njit()
        if dist is None:
            self.h_x = nm.pinned_empty((16384, 64), f32, queue)
            self.h_x[:] = self.host_x
            self.h_d = nm.pinned_empty((16384, 16384), f32, queue)
            self.h2d_bytes, self.d2h_bytes = 2 * self.h_x.nbytes, self.h_d.nbytes
            self.step_e2e = self._step_e2e

    def step_device(self):
        self.fn(self.x, self.y, self.d)

    def _step_e2e(self):
        import numba_mlir_b200 as nm

        nm.map_host(self.fn, [self.h_x], [self.h_d], resident=[self.host_y], chunk=2048, queue=self.queue)

    def check(self, dist=None):
        from oracle import configs as O

        self.queue.memset(self.d.ptr, 0, self.d.nbytes)
        self.step_device()
        got = self.d.copy_to_host()
        want = np.zeros_like(got)
        O.pairwise(self.host_x, self.host_y, want)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
        if getattr(self, "e2e_ran", False):
            np.testing.assert_allclose(np.asarray(self.h_d), want, rtol=1e-5, atol=1e-6)


class KMeans(Workload):
    """One Lloyd iteration: N = 2^22 float32 points, D = 16, K = 64, written
    with @kernel; fused assignment + accumulation reads the points once and
    writes the labels (285 MB)."""

    key = "kmeans"
    dtype = "f32"
    launches_per_step = 3
    exchange = "all-reduce(sum) of 64x16 float64 cluster sums and 64 int64 counts (8.7 KB)"

    def __init__(self, fraction=1.0, naive=False, fastmath=False):
        self.n = max(2048, int((1 << 22) * fraction) // 2048 * 2048)
        self.naive = naive
        self.fastmath = fastmath
        self.name = ("kmeans_iteration_n2^22_d16_k64" if fraction == 1.0 else f"kmeans_iteration_n{self.n}_d16_k64") \
            + ("_one_point_per_work_item" if naive else "") + ("_fastmath" if fastmath else "")
        self.bytes_per_step = self.n * 68
        self.units_per_step = self.n
        self.graph_steps = rotation_sets(self.n * 64)

    def setup_device(self, queue, seed, dist=None):
        import numba_mlir_b200 as nm

        rng = np.random.default_rng(seed)

        def points():
            centres = rng.uniform(-10, 10, (64, 16)).astype(f32)
            blob = rng.integers(0, 64, self.n)
            return (centres[blob] + rng.standard_normal((self.n, 16))).astype(f32)

        self.host = points()
        self.sets = [nm.from_host(self.host, queue)]
        for _ in range(self.graph_steps - 1):
            self.sets.append(nm.from_host(points(), queue))
        # every rank starts from the same centroids (rank 0's first points)
        self.c0 = _gather_host(dist, self.host[:64].copy(), queue)[0]
        self.cent = nm.from_host(self.c0, queue)
        self.labels = nm.empty(self.n, np.int32, queue)
        self.sums = nm.zeros((64, 16), np.float64, queue)
        self.counts = nm.zeros(64, np.int64, queue)
        self.dist = dist
        self.queue = queue
        self.i = 0

    def step_device(self):
        from numba_mlir_b200 import workloads

        q = self.queue
        q.memset(self.sums.ptr, 0, self.sums.nbytes)
        q.memset(self.counts.ptr, 0, self.counts.nbytes)
        if self.naive:
            workloads.kmeans_step_naive(self.sets[self.i % len(self.sets)], self.cent, self.labels, self.sums,
                                        self.counts)
        else:
            workloads.kmeans_step(self.sets[self.i % len(self.sets)], self.cent, self.labels, self.sums,
                                  self.counts, fastmath=self.fastmath)
        self.i += 1
        if self.dist is not None:
            from numba_mlir_b200 import sharding

            # sums and counts of all GPUs behind one flag round trip
            sharding.allreduce_many([(self.sums, "sum"), (self.counts, "sum")], self.dist)
        workloads.kmeans_update(self.cent, self.sums, self.counts)

    def check(self, dist=None):
        """One iteration from the initial centroids: the shard's labels are
        bit-exact, the exchanged sums and counts equal the shards' oracle
        partials added up, the new centroids are the oracle's."""
        from oracle import configs as O

        self.i = 0
        self.cent.copy_from_host(self.c0)
        self.step_device()
        want = np.zeros(self.n, np.int32)
        O.kmeans_assign(self.host, self.c0, want)
        got_labels = self.labels.copy_to_host()
        if self.fastmath:
            # fused multiply-adds round the distances differently: a label may
            # differ only where the two centroids are equally near to 1e-5
            bad = np.nonzero(got_labels != want)[0]
            p64 = self.host[bad].astype(np.float64)
            d_got = ((p64 - self.c0[got_labels[bad]].astype(np.float64)) ** 2).sum(axis=1)
            d_want = ((p64 - self.c0[want[bad]].astype(np.float64)) ** 2).sum(axis=1)
            assert np.all(np.abs(d_got - d_want) <= 1e-5 * d_want), "k-means labels (fastmath) are not the nearest"
            want = got_labels
        assert np.array_equal(got_labels, want), "k-means labels differ from the oracle"
        sums, counts = np.zeros((64, 16), np.float64), np.zeros(64, np.int64)
        O.kmeans_accumulate(self.host, want, sums, counts)
        sums = sum(_gather_host(self.dist, sums, self.queue))
        counts = sum(_gather_host(self.dist, counts, self.queue))
        assert np.array_equal(self.counts.copy_to_host(), counts), "k-means counts differ from the oracle"
        np.testing.assert_allclose(self.sums.copy_to_host(), sums, rtol=1e-12, atol=1e-7)
        new = O.kmeans_update(self.c0, sums, counts)
        got = self.cent.copy_to_host()
        ulp = np.abs(got.view(np.int32).astype(np.int64) - new.view(np.int32).astype(np.int64))
        assert ulp.max() <= 1, "k-means centroids differ from the oracle"


WORKLOADS = {
    "black_scholes": BlackScholes,
    "black_scholes_fastmath": BlackScholesFastmath,
    "bcast_add": BroadcastAdd,
    "sum_axis1": lambda: AxisReduction("sum_axis1"),
    "min_axis0": lambda: AxisReduction("min_axis0"),
    "argmin_axis1": lambda: AxisReduction("argmin_axis1"),
    "row_norm": lambda: AxisReduction("row_norm"),
    "int_sum": IntSum,
    "pairwise": Pairwise,
    "kmeans": KMeans,
    "kmeans_naive": lambda: KMeans(naive=True),
    "kmeans_fastmath": lambda: KMeans(fastmath=True),
}

# workloads whose shards exchange partial results: fraction -> workload
SHARDED = {
    "min_axis0": lambda fraction: AxisReduction("min_axis0", fraction),
    "int_sum": lambda fraction: IntSum(fraction),
    "kmeans": lambda fraction: KMeans(fraction),
}


# ---------------------------------------------------------------- clocks ----
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the
    timed regions run."""

    def __init__(self, device_index):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._active = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = device_index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if device_index < len(ids) and ids[device_index].strip().isdigit():
                    idx = int(ids[device_index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                    self.samples.append(mhz)
                    try:
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                    except Exception:
                        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                    for k, bit in names.items():
                        if mask & bit:
                            self.reasons.add(k)
                except Exception:
                    pass
            time.sleep(0.005)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def active(self, on):
        (self._active.set if on else self._active.clear)()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------ CPU timing ----
def time_cpu(key, budget_s, max_steps):
    """Best-of timing of the CPU oracle on the full workload within a budget."""
    import numba

    step, nbytes, units, _name = cpu_case(key, 1.0)
    step()  # compiles; excluded
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max_steps and (len(times) < 3 or time.perf_counter() < t_end):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return times, numba.get_num_threads(), nbytes, units


def cpu_case(key, scale):
    """The CPU oracle of one benchmark configuration on a `scale` fraction of
    its leading dimension: (step function, algorithmic bytes, units, name)."""
    from oracle import configs as O

    if key in ("black_scholes", "black_scholes_fastmath"):  # one CPU form for both
        price, strike, t, rate, vol = O.make_inputs("black_scholes", scale)
        call, put = np.zeros_like(price), np.zeros_like(price)
        return (lambda: O.black_scholes(price, strike, t, rate, vol, call, put),
                20 * price.size, price.size, WORKLOADS[key].name)
    if key == "bcast_add":
        a, b = O.make_inputs("bcast_add", scale)
        return lambda: O.bcast_add(a, b), 2 * a.nbytes + b.nbytes, a.size, BroadcastAdd.name
    if key in ("sum_axis1", "min_axis0", "argmin_axis1", "row_norm"):
        (a,) = O.make_inputs("reduce_f32", scale)
        fn = getattr(O, key)
        out_bytes = {"sum_axis1": 4 * a.shape[0], "min_axis0": 4 * a.shape[1],
                     "argmin_axis1": 8 * a.shape[0], "row_norm": 4 * a.shape[0]}[key]
        return lambda: fn(a), a.nbytes + out_bytes, a.size, f"{key}_f32_16384x4096"
    if key == "int_sum":
        (a,) = O.make_inputs("reduce_i32", scale)
        return lambda: O.int_sum(a), a.nbytes + 8, a.size, IntSum().name
    if key == "pairwise":
        x, y = O.make_inputs("pairwise", scale)
        d = np.zeros((x.shape[0], y.shape[0]), f32)
        return lambda: O.pairwise(x, y, d), d.nbytes + x.nbytes + y.nbytes, d.size, Pairwise.name
    if key in ("kmeans", "kmeans_naive", "kmeans_fastmath"):
        pts, cent = O.make_inputs("kmeans", scale)
        labels = np.zeros(pts.shape[0], np.int32)

        def step():
            O.kmeans_assign(pts, cent, labels)
            sums = np.zeros(cent.shape, np.float64)
            counts = np.zeros(cent.shape[0], np.int64)
            O.kmeans_accumulate(pts, labels, sums, counts)
            O.kmeans_update(cent, sums, counts)

        return step, pts.nbytes + labels.nbytes, pts.shape[0], WORKLOADS[key]().name
    raise ValueError(key)


def run_reference(args):
    """CPU arm: the oracle of --workload on the host cores, rank 0 only.  Each
    step is a bounded sample of the workload (the leading dimension is halved
    until the whole run stays near two minutes whatever --steps is)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import numba

    steps = args.steps if args.steps is not None else 20
    scale = 1.0
    while True:
        step, nbytes, units, name = cpu_case(args.workload, scale)
        step()  # compiles; excluded
        t0 = time.perf_counter()
        step()
        t_one = time.perf_counter() - t0
        if scale <= 1 / 1024 or (steps + max(args.warmup, 1)) * t_one <= 120.0:
            break
        scale /= 2
    full = WORKLOADS[args.workload]()
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    value = nbytes / dt / 1e9
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": full.dtype,
        "data": "synthetic",
        "config": config_of(full.name, full.units_per_step),
        "elements_per_s": units / dt,
        "cpu_baseline": {
            "value": value,
            "unit": UNIT,
            "cores": numba.get_num_threads(),
            "kind": "port",
            "sample": f"{units} of {full.units_per_step} elements per step; upstream "
            f"numba.njit(parallel=True), threading layer {numba.threading_layer()}",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------- GPU timing ---
def time_device(queue, workload, steps, warmup, barrier, use_graph, min_ms=MIN_TIMED_MS, max_blocks=400):
    """Device time of a block of exactly `steps` steps (CUDA events on the
    launching stream).  The block is repeated until `min_ms` of device time
    have been measured; returns (median block ms, kernel launches per block,
    blocks timed).

    With `use_graph` the steps are recorded into a CUDA graph after the warm-up
    and replayed, so that the host cost of submitting short kernels does not
    enter the device timeline."""
    from numba_mlir_b200 import runtime

    for _ in range(max(warmup, 3)):
        workload.step_device()
    barrier()
    graph = None
    captured = 0
    # steps recorded per graph: a workload that rotates over several operand sets
    # to stay larger than L2 records whole rotations
    rotation = getattr(workload, "graph_steps", 1)
    if rotation > 1:
        per_graph = rotation if steps % rotation == 0 else 0
    else:
        # several steps per graph take the gap between graph launches (about a
        # microsecond) out of the short steps; exactly `steps` steps still run
        per_graph = next(d for d in (10, 5, 4, 2, 1) if steps % d == 0)
    if use_graph and per_graph:
        workload.i = 0
        before = runtime.launch_count()
        queue.graph_begin()
        for _ in range(per_graph):
            workload.step_device()
        graph = queue.graph_end()
        captured = runtime.launch_count() - before  # kernel launches recorded in the graph
        queue.graph_launch(graph)
        barrier()
    blocks, total, counted = [], 0.0, 0
    while True:
        count0 = runtime.launch_count()
        e0 = queue.record()
        if graph is not None:
            for _ in range(steps // per_graph):
                queue.graph_launch(graph)
        else:
            for _ in range(steps):
                workload.step_device()
        e1 = queue.record()
        queue.wait(e1)
        ms = queue.elapsed_ms(e0, e1)
        queue.destroy_event(e0)
        queue.destroy_event(e1)
        counted = (steps // per_graph) * captured if graph is not None else runtime.launch_count() - count0
        blocks.append(ms)
        total += ms
        # every rank takes the same number of blocks: the decision is rank 0's
        again = total < min_ms and len(blocks) < max_blocks
        again = barrier(again)
        if not again:
            break
    if graph is not None:
        queue.graph_destroy(graph)
    return statistics.median(blocks), counted, len(blocks)


def time_e2e(w, barrier, steps):
    """Wall-clock seconds per end-to-end step (host buffers in and out)."""
    for _ in range(2):
        w.step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        w.step_e2e()
    barrier()
    w.e2e_ran = True
    return (time.perf_counter() - t0) / steps


def run_gpu(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    import torch

    from numba_mlir_b200 import build as _build

    if rank == 0:
        _build.build()
    from numba_mlir_b200 import runtime

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    numa_node = None
    if world > 1:
        # before any host buffer exists: this rank's cores and page-locked
        # memory sit next to its GPU
        from numba_mlir_b200 import sharding as _sharding

        numa_node = _sharding.bind_host_to_gpu(local_rank)
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
        if rank != 0:
            _build.build()  # no-op: picks up rank 0's library

    queue = runtime.get_queue(f"cuda:{local_rank}")
    flag = torch.zeros(1, device="cuda", dtype=torch.int32) if dist is not None else None

    def barrier(decision=None):
        """Synchronises the device (and the ranks); with a `decision`, returns
        rank 0's to every rank."""
        queue.synchronize()
        torch.cuda.synchronize()
        if dist is None:
            return decision
        if decision is None:
            dist.barrier()
        else:
            flag.fill_(1 if decision else 0)
            dist.broadcast(flag, 0)
            decision = bool(flag.item())
        torch.cuda.synchronize()
        return decision

    def exchange_mode(w):
        """(is there an exchange, does the library's peer-memory kernel carry it)"""
        collective = dist is not None and getattr(w, "dist", None) is not None
        peer = False
        if collective:
            from numba_mlir_b200 import sharding

            peer = sharding.peer_group(queue, dist) is not None  # built here by every rank
        return collective, peer

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    w = WORKLOADS[args.workload]()
    w.setup_device(queue, seed=rank, dist=dist)
    # A step with an exchange between shards is recorded in a graph like the
    # others when the exchange is the library's own peer-memory kernel (its call
    # counter lives on the device); a torch.distributed collective is not captured.
    collective, peer_exchange = exchange_mode(w)
    use_graph = (not collective or peer_exchange) and not args.no_graph

    if args.profile:
        # For a profiler: eager launches of the device-resident step only.
        for _ in range(args.warmup + args.steps):
            w.step_device()
        barrier()
        queue.check_status()
        if rank == 0:
            print(json.dumps({"profile_run": w.name, "steps": args.steps, "warmup": args.warmup,
                              "launches_per_step": w.launches_per_step}), flush=True)
        return

    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.active(True)
    dev_ms, counted, blocks = time_device(queue, w, args.steps, args.warmup, barrier, use_graph)
    sampler.active(False)
    queue.check_status()
    dev_ms = max_over_ranks(dev_ms)

    # -- end-to-end leg (host buffers, copies inside the timed region) ---------
    e2e = None
    if hasattr(w, "step_e2e"):
        e2e_steps = max(1, min(args.steps, 50))
        sampler.active(True)
        e2e = (max_over_ranks(time_e2e(w, barrier, e2e_steps)), e2e_steps)
        sampler.active(False)
    clocks = sampler.stop()
    w.check(dist)  # against the CPU oracle, outside the timed regions; raises on a mismatch
    queue.check_status()

    peak, peak_kind = measured_peaks()
    others = {}
    if not args.no_extra and args.workload == "black_scholes":
        for attr in ("d_in", "d_out", "h_in", "h_out", "host"):
            if hasattr(w, attr):
                delattr(w, attr)

        def entry(ow, graph=True):
            """Times one more workload: device time, its check, optional e2e."""
            ow.setup_device(queue, seed=rank, dist=dist)
            coll, peer = exchange_mode(ow)
            steps = 40 if getattr(ow, "graph_steps", 1) == 1 else 4 * ow.graph_steps
            ms, _launches, nblocks = time_device(queue, ow, steps, 5, barrier,
                                                 graph and (not coll or peer) and not args.no_graph)
            queue.check_status()
            us = max_over_ranks(ms) / steps * 1e3
            gbs = ow.bytes_per_step * world / (us * 1e-6) / 1e9
            rec = {"us_per_step": us, "GB/s": gbs, "frac_of_measured_peak": gbs / world / peak,
                   "frac_of_nominal_8TBs": gbs / world / NOMINAL_HBM_GBS, "timed_blocks": nblocks}
            if coll:
                how = ("in the last block of the reduction kernel" if ow.key in ("min_axis0", "int_sum")
                       else "in one launch of the library's peer-memory kernel")
                rec["exchange"] = ow.exchange + (f" over peer memory, {how}, inside the recorded graph"
                                                 if peer else " by NCCL (torch.distributed), eager launches")
            if hasattr(ow, "step_e2e"):
                s = max_over_ranks(time_e2e(ow, barrier, 5))
                rec["e2e"] = {"value": ow.bytes_per_step * world / s / 1e9, "unit": UNIT, "ms_per_step": s * 1e3,
                              "h2d_bytes_per_step": ow.h2d_bytes, "d2h_bytes_per_step": ow.d2h_bytes}
            ow.check(dist)
            queue.check_status()
            rec["verified"] = "one step's output equals the CPU oracle's"
            return rec

        if world == 1:
            # the other configurations on one GPU
            for key in ("black_scholes_fastmath", "bcast_add", "sum_axis1", "min_axis0", "argmin_axis1",
                        "row_norm", "int_sum", "pairwise", "kmeans", "kmeans_fastmath", "kmeans_naive"):
                ow = WORKLOADS[key]()
                others[ow.name] = entry(ow)
                del ow
        else:
            # the workloads whose shards exchange partials: weak scaling (a
            # full-size shard per GPU) and strong scaling (the configuration's
            # rows split over the GPUs)
            for key, make in SHARDED.items():
                for mode, fraction in (("weak", 1.0), ("strong", 1.0 / world)):
                    ow = make(fraction)
                    rec = entry(ow)
                    rec["scaling"] = mode
                    rec["rows_or_elements_per_gpu"] = ow.units_per_step
                    others[f"{key}:{mode}"] = rec
                    del ow

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        total_bytes = w.bytes_per_step * world
        value = total_bytes / (ms_per_step * 1e-3) / 1e9
        achieved = w.bytes_per_step / (ms_per_step * 1e-3) / 1e9  # per GPU, per launch
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": w.dtype,
            "data": "synthetic",
            "config": config_of(w.name, w.units_per_step),
            "run": {
                "api": "numba_mlir_b200.njit(parallel=True) / @kernel, launched through the gpux* C-ABI",
                "sharding": "axis 0 split across GPUs, full-size shard per GPU"
                + ((", all-reduce of the partials each step by the library's peer-memory kernel"
                    if peer_exchange else ", NCCL all-reduce of the partials each step")
                   if collective else ", no collective"),
                "l2": "working set per step exceeds the 126 MB L2 (or rotates over >2x L2); no flush",
                "launch": ("steps recorded in a CUDA graph (up to 10 per graph) and replayed"
                           if getattr(w, "graph_steps", 1) == 1 else
                           f"{w.graph_steps} steps (one rotation over the operand sets) recorded in a CUDA "
                           "graph and replayed; eager when the step count is not a multiple of that")
                if use_graph else "eager launches",
                "timing": f"median of {blocks} timed blocks of {args.steps} steps (at least {MIN_TIMED_MS:.0f} ms "
                          "of device time in all), CUDA events on the launching stream, max over ranks",
                "verified": "one step's output equals the CPU oracle's (checked outside the timed region)",
                "host_cores_bound_to_rank0": numa_node,
            },
            "elements_per_s": w.units_per_step * world / (ms_per_step * 1e-3),
            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "peak_kind": peak_kind,
                "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(w.key),
            },
            "gpu_launches": counted,
            "clocks": clocks,
        }
        if e2e:
            line["e2e"] = {
                "value": total_bytes / e2e[0] / 1e9,
                "unit": UNIT,
                "h2d_bytes_per_step": w.h2d_bytes,
                "d2h_bytes_per_step": w.d2h_bytes,
                "steps": e2e[1],
            }
        if others:
            line["other_configs"] = others
        if world == 1 and not args.no_extra and not args.no_dispatch and args.workload == "black_scholes":
            line["host_us_per_launch"] = dispatch_times(queue, 5000)
        if world == 1 and not args.no_cpu:
            times, threads, cpu_bytes, cpu_units = time_cpu(args.workload, budget_s=12.0, max_steps=100)
            best = min(times)
            line["cpu_baseline"] = {
                "value": cpu_bytes / best / 1e9,
                "unit": UNIT,
                "cores": threads,
                "kind": "port",
                "sample": f"the full workload ({cpu_units} elements) per step, best of "
                f"{len(times)}; upstream numba.njit(parallel=True)",
                "ms_per_step": best * 1e3,
            }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def dispatch_times(queue, calls):
    """Host cost of one launch, after the reference's kernel-dispatcher
    microbenchmark (benchmarks/benchmarks/microbenchmarks/kernel_dispatcher/
    numba_mlir.py:17-75): a kernel of 1, 2, 6 or 12 array arguments on 8
    int32 elements, called through a configured kernel object
    ("dispatcher") and through `kernel[...]` each time ("full_dispatcher"),
    the same launch repeated from native code (what is left when the
    interpreter is taken out: GPUParamDesc unpacking in the runtime library and
    the driver's launch), plus an `njit` elementwise call replayed from its plan."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, get_global_id, kernel

    def make(count):
        names = ", ".join(f"arg{i + 1}" for i in range(count))
        scope = {"get_global_id": get_global_id}
        exec(f"def func({names}):\n    i = get_global_id(0)\n    arg1[i] = i\n", scope)
        return scope["func"]

    # Host time only: the calls are issued in bursts short enough for the
    # stream's launch queue never to fill (a full queue makes the host wait for
    # the device, about 5.5 us per tiny kernel here), with an untimed
    # synchronize between bursts.
    burst = 200

    def host_time(call):
        spent = 0.0
        for _ in range(max(1, calls // burst)):
            t0 = time.perf_counter()
            for _ in range(burst):
                call()
            spent += time.perf_counter() - t0
            queue.synchronize()
        return spent / (max(1, calls // burst) * burst) * 1e6

    out = {}
    for count in (1, 2, 6, 12):
        array = nm.empty(8, np.int32, queue)
        base = kernel(make(count))
        fn = base[8, DEFAULT_LOCAL_SIZE]
        a = (array,) * count
        fn(*a)
        queue.synchronize()
        out[f"dispatcher_{count}_args_us"] = host_time(lambda: fn(*a))
        out[f"full_dispatcher_{count}_args_us"] = host_time(lambda: base[8, DEFAULT_LOCAL_SIZE](*a))
        # the same launch issued from native code without returning to the
        # interpreter: what the runtime library and the driver cost
        ck, _first = next(iter(fn._launchers.values()))
        handle = ck.handle_on(queue)
        block = ck.block_size_on(queue, handle, (8,))
        spent = 0.0
        for _ in range(max(1, calls // burst)):
            spent += runtime.fastcall().launch_kernel(queue.handle, handle, (1,), block, ck.layout_code(),
                                                      a, (8, 1, 1), burst)
            queue.synchronize()
        out[f"runtime_and_driver_{count}_args_us"] = spent / max(1, calls // burst) * 1e6

    @nm.njit
    def add(x, y, z):
        z[:] = x + y

    x, y, z = (nm.empty(8, np.float32, queue) for _ in range(3))
    add(x, y, z)
    queue.synchronize()
    out["njit_add_3_args_us"] = host_time(lambda: add(x, y, z))
    # with the launch queue kept full, what a long run of back-to-back tiny launches costs per launch
    t0 = time.perf_counter()
    for _ in range(calls):
        add(x, y, z)
    queue.synchronize()
    out["njit_add_3_args_sustained_us"] = (time.perf_counter() - t0) / calls * 1e6
    return out


def run_dispatch(args):
    from numba_mlir_b200 import runtime

    calls = args.steps if args.steps is not None else 20000
    out = dispatch_times(runtime.get_queue("cuda:0"), calls)
    print(json.dumps({"metric": "host_time_per_launch", "unit": "us", "calls": calls, **out}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="black_scholes", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-dispatch", action="store_true",
                    help="skip the dispatcher microbenchmark (tens of thousands of tiny launches)")
    ap.add_argument("--no-graph", action="store_true", help="eager launches instead of a CUDA graph")
    ap.add_argument("--profile", action="store_true",
                    help="run only warmup + steps eager device steps of --workload (for ncu)")
    ap.add_argument("--dispatch", action="store_true",
                    help="host time per launch of tiny kernels (dispatcher microbenchmark)")
    args = ap.parse_args()
    if args.dispatch:
        run_dispatch(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        if args.steps is None:
            args.steps = 3 if args.profile else 2000
        run_gpu(args)


if __name__ == "__main__":
    main()
