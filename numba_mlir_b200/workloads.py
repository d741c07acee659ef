"""User-level programs of the benchmark configurations, written against the
public decorators (what a numba-mlir user would write).  bench.py, the smoke
check and the tests import them from here so that they all run the same code.
"""

import math

import numpy as np

from .decorators import njit, vectorize
from .kernel import (atomic, barrier, get_global_id, get_group_id, get_local_id, get_local_size, kernel, local,
                     private)


@vectorize(nopython=True)
def _nberf(x):
    return math.erf(x)


# Black-Scholes chain of numba_mlir/mlir/tests/test_numpy.py:2827-2852; the
# Python-float constants are written as float32 so that Numba's typing keeps
# the whole chain in float32.
@njit(parallel=True)
def black_scholes(price, strike, t, rate, volatility, call, put):
    mr = -rate
    sig_sig_two = volatility * volatility * np.float32(2)

    P = price
    S = strike
    T = t

    a = np.log(P / S)
    b = T * mr

    z = T * sig_sig_two
    c = np.float32(0.25) * z
    y = np.float32(1.0) / np.sqrt(z)

    w1 = (a - b + c) * y
    w2 = (a - b - c) * y

    d1 = np.float32(0.5) + np.float32(0.5) * _nberf(w1)
    d2 = np.float32(0.5) + np.float32(0.5) * _nberf(w2)

    Se = np.exp(b) * S

    r = P * d1 - Se * d2
    call[:] = r
    put[:] = r - P + Se


# The same chain under fastmath=True, the flags the reference's benchmark driver
# compiles every kernel with (numba_mlir/mlir/benchmarking.py:43): division and
# square root take the approximate instructions and a*b+c contracts.
black_scholes_fastmath = njit(parallel=True, fastmath=True)(black_scholes.py_func)


# The result is written into an argument (as the reference's offload tests do,
# mlir/tests/test_gpu.py:1538-1551), so a call allocates nothing.
@njit(parallel=True)
def broadcast_add(a, b, out):
    out[:] = a + b


@njit(parallel=True)
def sum_axis1(a, out):
    out[:] = np.sum(a, axis=1)


# A reduction fed by an elementwise chain (mlir/tests/test_gpu.py:2198-2224): the
# squares are never written out, the rows are read once.
@njit(parallel=True)
def row_norm(a, out):
    out[:] = np.sqrt(np.square(a).sum(axis=1))


@njit(parallel=True)
def min_axis0(a, out):
    out[:] = np.min(a, axis=0)


@njit(parallel=True)
def argmin_axis1(a, out):
    out[:] = np.argmin(a, axis=1)


@njit(parallel=True)
def total(a, out):
    out[...] = np.sum(a)


# Pairwise Euclidean distances through the norm expansion |x|^2 + |y|^2 - 2 x.y
# with the dot products from np.dot, the route to the device gemm in the
# reference (numba_mlir/mlir/numpy/funcs.py:752-812).  The array front end
# recognises the chain around the product and runs it as the epilogue of the
# tensor-core contraction, with the row norms taken from its packing prepass.
@njit(parallel=True)
def pairwise_distance(x, y, d):
    xx = np.sum(x * x, axis=1)
    yy = np.sum(y * y, axis=1)
    g = np.dot(x, y.T)
    d[:] = np.sqrt(np.maximum(xx.reshape(-1, 1) + yy.reshape(1, -1) - np.float32(2) * g, np.float32(0)))


# New centroids = float32(sum / count); empty clusters keep their centre.
@njit(parallel=True)
def kmeans_update(centroids, sums, counts):
    cnt = counts.reshape(-1, 1)
    centroids[:] = np.where(cnt > 0, (sums / np.maximum(cnt, 1)).astype(np.float32), centroids)


# One Lloyd iteration as a @kernel program: nearest-centroid assignment in
# float32 (index order over the dimensions, separate multiply and add, strict
# `<` so ties keep the lower cluster), then per-cluster sums (float64) and
# counts (int64).  The work-group stages the centroids in local memory and
# every work-item keeps two points in private arrays, so the 64 x 16 inner loop
# runs out of shared memory and registers and one read of a centroid value
# serves both points.  The sums are gathered without per-point atomics: after a
# batch of 256 x 2 points is labelled, 64 work-items (4 point phases x 16
# dimensions) add the batch into float64 accumulator columns in local memory
# that each of them owns, and only the 64 x 16 group totals meet the global
# arrays through atomics, once per group.  (Measured slower: eight phases with
# a 64 KB accumulator, 696 us against 585 us; one, four or eight points per
# work-item through the centroid loop at once instead of two, 639, 664 and
# 836 us against 569 us; persistent groups that take the 512-point batches
# round robin, four groups per multiprocessor, 609 us against 573 us; groups
# of 320 in which 256 work-items only label and 64 only add the batch labelled
# one pass earlier, so that nobody waits while 64 add, 563 us against 571 us:
# the additions are 4 % of the instructions, the kernel is bound by the issue
# rate of the 3 x 64 x 16 subtract, multiply and add instructions per point.)
_KM_K = 64
_KM_D = 16
_KM_PTS = 8
_KM_Q = 2  # points a work-item takes through the centroid loop at once
_KM_PH = 4     # point phases of the accumulation
_KM_COLS = _KM_PH * _KM_D  # accumulator columns per cluster: phases x dimensions
KMEANS_LOCAL_SIZE = 256


@kernel(gpu_use_64bit_index=False)  # 2^22 x 16 elements: every offset fits 32 bits
def _kmeans_kernel(points, centroids, labels, sums, counts):
    lid = get_local_id(0)
    lsz = get_local_size(0)
    base = get_group_id(0) * (lsz * _KM_PTS)

    cent = local.array((_KM_K, _KM_D), np.float32)
    lbl = local.array(KMEANS_LOCAL_SIZE * _KM_Q, np.int32)
    lcnt = local.array(_KM_K, np.int32)
    # Column c = phase * 16 + dimension belongs to work-item c alone: it adds
    # its points into acc[label, c] with plain read-modify-writes, no atomics.
    acc = local.array((_KM_K, _KM_COLS), np.float64)
    j = lid
    while j < _KM_K * _KM_D:
        cent[j // _KM_D, j % _KM_D] = centroids[j // _KM_D, j % _KM_D]
        j += lsz
    j = lid
    while j < _KM_K * _KM_COLS:
        acc[j // _KM_COLS, j % _KM_COLS] = 0.0
        j += lsz
    if lid < _KM_K:
        lcnt[lid] = 0
    barrier()

    jcol = lid & (_KM_D - 1)
    phase = lid >> 4
    # _KM_Q points per work-item go through the centroid loop together, so one
    # read of a centroid value from local memory serves all of them; each point's
    # distance still accumulates over the dimensions in index order.
    p = private.array((_KM_Q, _KM_D), np.float32)
    d = private.array(_KM_Q, np.float32)
    best_d = private.array(_KM_Q, np.float32)
    best = private.array(_KM_Q, np.int32)
    for r in range(_KM_PTS // _KM_Q):
        row0 = base + r * (lsz * _KM_Q)
        for q in range(_KM_Q):
            for jj in range(_KM_D):
                p[q, jj] = points[row0 + q * lsz + lid, jj]
            best[q] = 0
            best_d[q] = np.float32(np.inf)
        for k in range(_KM_K):
            for q in range(_KM_Q):
                d[q] = np.float32(0.0)
            for jj in range(_KM_D):
                c = cent[k, jj]
                for q in range(_KM_Q):
                    t = p[q, jj] - c
                    d[q] += t * t
            for q in range(_KM_Q):
                if d[q] < best_d[q]:
                    best_d[q] = d[q]
                    best[q] = k
        for q in range(_KM_Q):
            labels[row0 + q * lsz + lid] = best[q]
            atomic.add(lcnt, best[q], 1)
            lbl[q * lsz + lid] = best[q]
        barrier()
        if lid < _KM_COLS:
            # the batch's rows were read a moment ago: these loads hit in L1
            # four rows per step: their labels and values are fetched before the
            # first read-modify-write, which would otherwise order every load behind it
            for m in range(phase, KMEANS_LOCAL_SIZE * _KM_Q, 4 * _KM_PH):
                l0 = lbl[m]
                l1 = lbl[m + _KM_PH]
                l2 = lbl[m + 2 * _KM_PH]
                l3 = lbl[m + 3 * _KM_PH]
                x0 = points[row0 + m, jcol]
                x1 = points[row0 + m + _KM_PH, jcol]
                x2 = points[row0 + m + 2 * _KM_PH, jcol]
                x3 = points[row0 + m + 3 * _KM_PH, jcol]
                acc[l0, lid] += x0
                acc[l1, lid] += x1
                acc[l2, lid] += x2
                acc[l3, lid] += x3
        barrier()

    e = lid
    while e < _KM_K * _KM_D:
        k = e // _KM_D
        jj = e % _KM_D
        v = acc[k, jj]
        for ph in range(1, _KM_PH):
            v += acc[k, ph * _KM_D + jj]
        if v != 0.0:
            atomic.add(sums, (k, jj), v)
        e += lsz
    if lid < _KM_K:
        if lcnt[lid] != 0:
            atomic.add(counts, lid, lcnt[lid])


# The same program compiled with fastmath=True: the subtraction, the square and
# the accumulation of two points then run as packed instructions that the
# assembler merges into fused multiply-adds, so a distance is rounded once per
# dimension instead of twice and a label may differ from the default build's
# where two centroids are nearly equally near.
_kmeans_kernel_fastmath = kernel(gpu_use_64bit_index=False, fastmath=True)(_kmeans_kernel.py_func)


# The same iteration in the plain form: one point per work-item, every point
# adds itself to its cluster's sum and count with global atomics.
@kernel(gpu_use_64bit_index=False)
def _kmeans_naive_kernel(points, centroids, labels, sums, counts):
    i = get_global_id(0)
    best = 0
    best_d = np.float32(np.inf)
    for k in range(centroids.shape[0]):
        d = np.float32(0.0)
        for j in range(points.shape[1]):
            t = points[i, j] - centroids[k, j]
            d += t * t
        if d < best_d:
            best_d = d
            best = k
    labels[i] = best
    atomic.add(counts, best, 1)
    for j in range(points.shape[1]):
        atomic.add(sums, (best, j), points[i, j])


def kmeans_step_naive(points, centroids, labels, sums, counts):
    _kmeans_naive_kernel[points.shape[0], KMEANS_LOCAL_SIZE](points, centroids, labels, sums, counts)


def kmeans_step(points, centroids, labels, sums, counts, fastmath=False):
    """Assignment + accumulation for every point.  N must be a multiple of
    256 * 8 because every work-item of a group takes part in the barriers and
    handles 8 points."""
    n = points.shape[0]
    if centroids.shape != (_KM_K, _KM_D):
        raise ValueError("this kernel is written for K = 64 clusters of D = 16 dimensions")
    chunk = KMEANS_LOCAL_SIZE * _KM_PTS
    if n % chunk:
        raise ValueError(f"the number of points must be a multiple of {chunk}")
    (_kmeans_kernel_fastmath if fastmath else _kmeans_kernel)[n // _KM_PTS, KMEANS_LOCAL_SIZE](
        points, centroids, labels, sums, counts)
