"""Oracle restatements of the five benchmark workloads (test infrastructure only).

Each function is compiled by upstream Numba, the reference's own definition of
`njit` with its MLIR pipeline disabled (numba_mlir/numba_mlir/decorators.py:89-98),
in the form upstream Numba accepts, and has a float64 NumPy ground truth beside
it where floating-point tolerance is judged.
"""

import math

import numba
import numpy as np
from numba import njit, prange, vectorize

f32 = np.float32


# --------------------------------------------------------------- inputs -----
def make_inputs(config, scale=1.0, seed=0):
    """Seeded synthetic inputs with the shapes and value distributions of the
    benchmark configurations; `scale` shrinks the leading dimension."""
    rng = np.random.default_rng(seed)
    if config == "bcast_add":
        rows = max(1, int(2048 * scale))
        a = rng.uniform(-1, 1, (rows, 2048)).astype(f32)
        b = rng.uniform(-1, 1, (1, 2048)).astype(f32)
        return a, b
    if config == "black_scholes":
        n = max(1, int(2**24 * scale))
        price = rng.uniform(10, 50, n).astype(f32)
        strike = rng.uniform(10, 50, n).astype(f32)
        t = rng.uniform(1, 2, n).astype(f32)
        return price, strike, t, f32(0.1), f32(0.2)
    if config == "reduce_f32":
        rows = max(1, int(16384 * scale))
        return (rng.standard_normal((rows, 4096)).astype(f32),)
    if config == "reduce_i32":
        n = max(1, int(2**28 * scale))
        return (rng.integers(-1000, 1001, n, dtype=np.int32),)
    if config == "pairwise":
        m = max(1, int(16384 * scale))
        x = rng.uniform(0, 1, (m, 64)).astype(f32)
        y = rng.uniform(0, 1, (m, 64)).astype(f32)
        return x, y
    if config == "kmeans":
        n = max(64, int(2**22 * scale))
        centres = rng.uniform(-10, 10, (64, 16)).astype(f32)
        blob = rng.integers(0, 64, n)
        pts = (centres[blob] + rng.standard_normal((n, 16))).astype(f32)
        return pts, pts[:64].copy()
    raise ValueError(config)


# ------------------------------------------- 1. broadcast elementwise add ---
# eltwise + NumPy broadcasting, numba_mlir/mlir/linalg_builder.py:297-325;
# a (1,N) operand is a stride-0 read (numba_mlir/mlir/array_type.py:54-55).
# Upstream parallel=True rejects the (1,N) array expression, hence the loop.
@njit(parallel=True)
def bcast_add(a, b):
    out = np.empty_like(a)
    for i in prange(a.shape[0]):
        for j in range(a.shape[1]):
            out[i, j] = a[i, j] + b[0, j]
    return out


# ------------------------------------------------------ 2. Black-Scholes ----
# Operation order of numba_mlir/mlir/tests/test_numpy.py:2827-2852 with the
# Python-float constants written as float32 so that Numba's typing keeps the
# whole chain in float32 (a bare 0.25 would promote to float64).
@vectorize(nopython=True)
def _nberf(x):
    return math.erf(x)


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


def black_scholes_f64(price, strike, t, rate, volatility):
    """float64 ground truth of the same chain on the float32 inputs."""
    from scipy.special import erf

    P = price.astype(np.float64)
    S = strike.astype(np.float64)
    T = t.astype(np.float64)
    mr = -float(rate)
    ss2 = float(f32(volatility) * f32(volatility) * f32(2))
    a = np.log(P / S)
    b = T * mr
    z = T * ss2
    c = 0.25 * z
    y = 1.0 / np.sqrt(z)
    w1 = (a - b + c) * y
    w2 = (a - b - c) * y
    d1 = 0.5 + 0.5 * erf(w1)
    d2 = 0.5 + 0.5 * erf(w2)
    Se = np.exp(b) * S
    r = P * d1 - Se * d2
    return r, r - P + Se


# The reference's own body, verbatim typing (bare Python constants): under
# Numba's rules the intermediates that meet a Python float become float64.
@njit(parallel=True)
def black_scholes_ref_typing(price, strike, t, rate, volatility, call, put):
    mr = -rate
    sig_sig_two = volatility * volatility * 2
    P = price
    S = strike
    T = t
    a = np.log(P / S)
    b = T * mr
    z = T * sig_sig_two
    c = 0.25 * z
    y = 1.0 / np.sqrt(z)
    w1 = (a - b + c) * y
    w2 = (a - b - c) * y
    d1 = 0.5 + 0.5 * _nberf(w1)
    d2 = 0.5 + 0.5 * _nberf(w2)
    Se = np.exp(b) * S
    r = P * d1 - Se * d2
    call[:] = r
    put[:] = r - P + Se


# ----------------------------------------------------- 3. reductions --------
# _array_reduce, numba_mlir/mlir/numpy/funcs.py:163-214: accumulator of the
# array dtype for floats, int64 for any integer dtype.
@njit(parallel=True)
def sum_axis1(a):
    # Upstream lowers np.sum(a, axis=1) serially; the explicit row loop is the
    # same per-row left-to-right float32 accumulation, spread over the cores
    # (the reference walks each row in one work-item, LowerToGpu.cpp:162-245).
    out = np.empty(a.shape[0], np.float32)
    for i in prange(a.shape[0]):
        s = np.float32(0.0)
        for j in range(a.shape[1]):
            s += a[i, j]
        out[i] = s
    return out


# sqrt(sum(a*a, axis=1)): the producer-into-reduction fusion the reference tests
# (numba_mlir/mlir/tests/test_gpu.py:2198-2224); float32 accumulation per row.
@njit(parallel=True)
def row_norm(a):
    out = np.empty(a.shape[0], np.float32)
    for i in prange(a.shape[0]):
        s = np.float32(0.0)
        for j in range(a.shape[1]):
            s += a[i, j] * a[i, j]
        out[i] = np.sqrt(s)
    return out


# np.min(axis=0) is supported by the reference (numpy/funcs.py:298-303) but not
# by upstream Numba; min is select(x < m, x, m) (builtin/funcs.py:140-146).
@njit(parallel=True)
def min_axis0(a):
    out = np.empty(a.shape[1], a.dtype)
    for j in prange(a.shape[1]):
        m = a[0, j]
        for i in range(1, a.shape[0]):
            x = a[i, j]
            if x < m:
                m = x
        out[j] = m
    return out


# (value, index) pair-min keeps the lower index on ties
# (numba_mlir/mlir/builtin/funcs.py:126-138) == NumPy's first occurrence.
@njit(parallel=True)
def argmin_axis1(a):
    out = np.empty(a.shape[0], np.int64)
    for i in prange(a.shape[0]):
        best = 0
        m = a[i, 0]
        for j in range(1, a.shape[1]):
            x = a[i, j]
            if x < m:
                m = x
                best = j
        out[i] = best
    return out


# Integer sums accumulate in int64 (numpy/funcs.py:120-123,172-185).
@njit(parallel=True)
def int_sum(a):
    s = np.int64(0)
    for i in prange(a.shape[0]):
        s += np.int64(a[i])
    return s


@njit(parallel=True)
def full_sum_f32(a):
    return a.sum()


# ----------------------------------------------------- 4. pairwise ----------
# Direct loop of numba_mlir/mlir/tests/test_gpu.py:2228-2239 (d is a Python
# float: float64 accumulation of float32 squared differences).
@njit(parallel=True)
def pairwise(X1, X2, D):
    X1_rows = X1.shape[0]
    X2_rows = X2.shape[0]
    X1_cols = X1.shape[1]
    for i in prange(X1_rows):
        for j in range(X2_rows):
            d = 0.0
            for k in range(X1_cols):
                tmp = X1[i, k] - X2[j, k]
                d += tmp * tmp
            D[i, j] = np.sqrt(d)


def pairwise_f64(X1, X2):
    """float64 ground truth (exact differences of the float32 inputs)."""
    a = X1.astype(np.float64)
    b = X2.astype(np.float64)
    d2 = ((a[:, None, :] - b[None, :, :]) ** 2).sum(-1)
    return np.sqrt(d2)


# ----------------------------------------------------- 5. k-means -----------
# One Lloyd iteration with the arithmetic of the @kernel body used by the
# benchmark: float32 squared distance accumulated over the dimensions in index
# order with separate multiply and add (the reference contracts to FMA only
# under fastmath, mlir/tests/test_gpu.py:980-1008); strict `<` so the lowest
# cluster index wins ties; per-cluster sums in float64 and counts in int64
# (atomic.add casts the value to the array dtype, kernel_impl.py:284-291).
@njit(parallel=True)
def kmeans_assign(points, centroids, labels):
    n = points.shape[0]
    k_count = centroids.shape[0]
    dims = points.shape[1]
    for i in prange(n):
        best = 0
        best_d = np.float32(np.inf)
        for k in range(k_count):
            d = np.float32(0.0)
            for j in range(dims):
                t = points[i, j] - centroids[k, j]
                d += t * t
            if d < best_d:
                best_d = d
                best = k
        labels[i] = best


@njit
def kmeans_accumulate(points, labels, sums, counts):
    for i in range(points.shape[0]):
        k = labels[i]
        counts[k] += 1
        for j in range(points.shape[1]):
            sums[k, j] += points[i, j]


def kmeans_update(centroids, sums, counts):
    """New centroids = float32(sum / count); empty clusters keep their centre."""
    new = centroids.copy()
    nz = counts > 0
    new[nz] = (sums[nz] / counts[nz, None].astype(np.float64)).astype(f32)
    return new


def kmeans(points, centroids, iters):
    """Runs `iters` Lloyd iterations; returns (labels int32, centroids f32)."""
    c = centroids.copy()
    labels = np.zeros(points.shape[0], np.int32)
    for _ in range(iters):
        kmeans_assign(points, c, labels)
        sums = np.zeros(c.shape, np.float64)
        counts = np.zeros(c.shape[0], np.int64)
        kmeans_accumulate(points, labels, sums, counts)
        c = kmeans_update(c, sums, counts)
    return labels, c


def threads():
    return numba.get_num_threads()
