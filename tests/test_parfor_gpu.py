"""`prange` loop nests in `njit` functions on the GPU, after the reference's
tests (numba_mlir/mlir/tests/test_gpu.py:1523-1613, test_numpy.py:1039-1057):
the Python function run on NumPy arrays is the expected result."""

import numba
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

_test_values = [True, False, -3, -2, -1, 0, 1, 2, 3, -2.5, -1.0, -0.5, -0.0, 0.0, 0.5, 1.0, 2.5]


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def test_parfor_simple1(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime

    def py_func(a, b, c):
        for i in numba.prange(len(a)):
            c[i] = a[i] + b[i]

    gpu_func = nm.njit(py_func)
    a = np.arange(1024, dtype=np.float32)
    b = np.arange(1024, dtype=np.float32) * 3
    want = np.zeros(a.shape, a.dtype)
    py_func(a, b, want)
    got = _dev(np.zeros(a.shape, a.dtype))
    before = runtime.launch_count()
    gpu_func(_dev(a), _dev(b), got)
    assert runtime.launch_count() - before == 1  # one launch for the loop nest
    np.testing.assert_equal(got.copy_to_host(), want)


@pytest.mark.parametrize("val", _test_values)
def test_parfor_scalar(queue, val):
    import numba_mlir_b200 as nm

    def py_func(a, b, c, d):
        for i in numba.prange(len(a)):
            c[i] = a[i] + b[i] + d

    a = np.arange(1024, dtype=np.float32)
    b = np.arange(1024, dtype=np.float32) * 3
    want = np.zeros(a.shape, a.dtype)
    py_func(a, b, want, val)
    got = _dev(np.zeros(a.shape, a.dtype))
    nm.njit(py_func)(_dev(a), _dev(b), got, val)
    np.testing.assert_equal(got.copy_to_host(), want)


@pytest.mark.parametrize("val", [True, -3, 0, 2.5])
def test_parfor_scalar_capture(queue, val):
    import numba_mlir_b200 as nm

    def py_func(a, b, c):
        for i in numba.prange(len(a)):
            c[i] = a[i] + b[i] + val

    a = np.arange(1024, dtype=np.float32)
    b = np.arange(1024, dtype=np.float32) * 3
    want = np.zeros(a.shape, a.dtype)
    py_func(a, b, want)
    got = _dev(np.zeros(a.shape, a.dtype))
    nm.njit(py_func)(_dev(a), _dev(b), got)
    np.testing.assert_equal(got.copy_to_host(), want)


@pytest.mark.parametrize("shape", [(1, 1), (7, 5), (33, 1000), (1000, 33), (257, 513)])
def test_parfor_2d_nest(queue, shape):
    import numba_mlir_b200 as nm

    def py_func(a, b, c):
        for i in numba.prange(a.shape[0]):
            for j in numba.prange(a.shape[1]):
                c[i, j] = a[i, j] * 2 + b[j, i]

    rng = np.random.default_rng(3)
    a = rng.standard_normal(shape).astype(np.float32)
    b = rng.standard_normal(shape[::-1]).astype(np.float32)
    want = np.zeros(shape, np.float32)
    py_func(a, b, want)
    got = _dev(np.zeros(shape, np.float32))
    nm.njit(py_func, parallel=True)(_dev(a), _dev(b), got)
    np.testing.assert_equal(got.copy_to_host(), want)


def test_parfor_inner_sequential_reduction_and_strided_range(queue):
    import numba_mlir_b200 as nm

    def py_func(a, c):
        for i in numba.prange(1, a.shape[0], 2):
            s = np.float32(0)
            for j in range(a.shape[1]):
                s += a[i, j]
            c[i] = s

    rng = np.random.default_rng(4)
    a = rng.integers(-8, 8, (301, 77)).astype(np.float32)  # exact in float32 in any order
    want = np.full(301, -1, np.float32)
    py_func(a, want)
    got = _dev(np.full(301, -1, np.float32))
    nm.njit(py_func, parallel=True)(_dev(a), got)
    np.testing.assert_equal(got.copy_to_host(), want)


def test_parfor_empty_and_large(queue):
    import numba_mlir_b200 as nm

    def py_func(a, c):
        for i in numba.prange(len(a)):
            c[i] = a[i] + 1

    f = nm.njit(py_func, parallel=True)
    e = _dev(np.zeros(0, np.int32))
    f(e, e)  # empty loop: nothing launched, nothing raised
    n = (1 << 22) + 3  # more iterations than threads in the grid: grid-strided
    a = np.arange(n, dtype=np.int32)
    got = _dev(np.zeros(n, np.int32))
    f(_dev(a), got)
    np.testing.assert_equal(got.copy_to_host(), a + 1)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
def test_prange_atomic(queue, dtype):
    import numba_mlir_b200 as nm

    def py_func(n, s, res):
        for i in numba.prange(n):
            res[i % s] += dtype(i)

    N, S = 10000, 10
    want = np.zeros(S, dtype)
    py_func(N, S, want)
    got = _dev(np.zeros(S, dtype))
    nm.njit(py_func, parallel=True)(N, S, got)
    np.testing.assert_allclose(got.copy_to_host(), want, rtol=1e-5)


def test_pairwise2(queue):
    """The reference's direct-loop pairwise distance
    (numba_mlir/mlir/tests/test_gpu.py:2226-2266): both prange loops map to
    the grid, the k loop runs in the thread."""
    import numba_mlir_b200 as nm

    def py_func(X1, X2, D):
        X1_rows = X1.shape[0]
        X2_rows = X2.shape[0]
        X1_cols = X1.shape[1]

        for i in numba.prange(X1_rows):
            for j in numba.prange(X2_rows):
                d = 0.0
                for k in range(X1_cols):
                    tmp = X1[i, k] - X2[j, k]
                    d += tmp * tmp
                D[i, j] = np.sqrt(d)

    jit_func = nm.njit(py_func)
    dims, npoints = 3, 128
    a = np.arange(npoints * dims, dtype=np.float32).reshape(npoints, dims)
    b = a + 5
    res = np.zeros((npoints, npoints), dtype=np.float32)
    py_func(a, b, res)
    got = _dev(np.zeros_like(res))
    jit_func(_dev(a), _dev(b), got)
    assert jit_func._parfor_kernels and all(k.inner_parallel for k in jit_func._parfor_kernels.values())
    np.testing.assert_allclose(got.copy_to_host(), res, rtol=1e-5)


@pytest.mark.parametrize("n", [0, 1, 255, 256, 1000, (1 << 20) + 7])
def test_prange_scalar_reductions(queue, n):
    """Sums, products, minima and maxima carried across a prange loop (the loop
    form of what the reference lowers through its GPU global reduce,
    mlir/lib/Conversion/GpuToGpuRuntime.cpp:2002-2277), combined per block and
    then in block order by the last block to finish."""
    import numba_mlir_b200 as nm

    def total(a):
        s = 0
        for i in numba.prange(len(a)):
            s += a[i]
        return s

    def fsum_min_max(a):
        s = 0.0
        lo = np.float32(np.inf)
        hi = np.float32(-np.inf)
        for i in numba.prange(len(a)):
            s += a[i]
            lo = min(lo, a[i])
            hi = max(hi, a[i])
        return s * 2 + lo - hi

    rng = np.random.default_rng(n)
    ints = rng.integers(-1000, 1001, n).astype(np.int32)
    got = nm.njit(total, parallel=True)(_dev(ints))
    assert int(got) == int(ints.sum(dtype=np.int64))

    x = (rng.integers(-64, 64, n) / 8).astype(np.float32)  # sums exactly in float64 in any order
    if n:
        got = nm.njit(fsum_min_max, parallel=True)(_dev(x))
        assert got == x.astype(np.float64).sum() * 2 + float(x.min()) - float(x.max())


def test_prange_reduction_with_start_value_product_and_tail_store(queue):
    import numba_mlir_b200 as nm

    def f(a, start, out):
        s = start
        p = 1.0
        for i in numba.prange(len(a)):
            s -= a[i]
            p *= np.float64(1.0) + a[i] * 0
        out[0] = s      # runs once, after every thread is done
        out[1] = p
        return s

    a = np.arange(5000, dtype=np.float64)
    out = _dev(np.zeros(2, np.float64))
    got = nm.njit(f, parallel=True)(_dev(a), 10.0, out)
    assert got == 10.0 - a.sum()
    np.testing.assert_equal(out.copy_to_host(), [10.0 - a.sum(), 1.0])
    # the ticket is back at zero: the same kernel runs again and so do the reductions
    got = nm.njit(f, parallel=True)(_dev(a), 1.0, out)
    assert got == 1.0 - a.sum()
    from numba_mlir_b200 import reduce_ops

    assert reduce_ops.reduce(_dev(a), "sum").copy_to_host() == a.sum()


def test_use_64bit_index_prange_and_kernel(queue):
    """mlir/tests/test_gpu.py:1788-1898: the same program under
    gpu_use_64bit_index True, False and the default gives the same array; with
    False the generated code carries 32-bit index arithmetic."""
    import numba

    import numba_mlir_b200 as nm
    from numba_mlir_b200.kernel import get_global_id, kernel

    def py_func(a):
        ah, aw = a.shape
        for h in numba.prange(ah):
            for w in numba.prange(aw):
                a[h, w] = w + h * aw

    def kern(a):
        aw = a.shape[1]
        h = get_global_id(0)
        w = get_global_id(1)
        a[h, w] = w + h * aw

    for shape in ((6, 8), (257, 1031)):
        want = np.arange(shape[0] * shape[1], dtype=np.float32).reshape(shape)
        for opts in ({}, {"gpu_use_64bit_index": True}, {"gpu_use_64bit_index": False}):
            d = nm.zeros(shape, np.float32)
            nm.njit(py_func, **opts)(d)
            assert np.array_equal(d.copy_to_host(), want), opts
            d = nm.zeros(shape, np.float32)
            kernel(kern, **opts)[shape, ()](d)
            assert np.array_equal(d.copy_to_host(), want), opts
    queue.check_status()


def test_kmeans_kernel_with_32bit_indices_keeps_labels(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from numba_mlir_b200.kernel import kernel
    from oracle import configs as O

    pts, c0 = O.make_inputs("kmeans", 1 / 64)
    n = pts.shape[0]
    labels = nm.zeros(n, np.int32)
    sums, counts = nm.zeros((64, 16), np.float64), nm.zeros(64, np.int64)
    k32 = kernel(workloads._kmeans_kernel.py_func, gpu_use_64bit_index=False)
    k32[n // 8, workloads.KMEANS_LOCAL_SIZE](nm.from_host(pts), nm.from_host(c0), labels, sums, counts)
    want = np.zeros(n, np.int32)
    O.kmeans_assign(pts, c0, want)
    assert np.array_equal(labels.copy_to_host(), want)
    ws, wc = np.zeros((64, 16)), np.zeros(64, np.int64)
    O.kmeans_accumulate(pts, want, ws, wc)
    assert np.array_equal(counts.copy_to_host(), wc)
    np.testing.assert_allclose(sums.copy_to_host(), ws, rtol=1e-12, atol=1e-8)


# --------------------- several loops per function, loops next to expressions ---
def _launched(fn, *args):
    from numba_mlir_b200 import runtime

    before = runtime.launch_count()
    res = fn(*args)
    return res, runtime.launch_count() - before


def test_two_parallel_loops_are_two_kernels(queue):
    """One `gpu.launch` per parallel loop nest of a function
    (mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940); the scalar the second
    loop carries out comes back to the host."""
    import numba

    import numba_mlir_b200 as nm

    def py_func(a, b, out):
        n = len(a)
        for i in numba.prange(n):
            out[i] = a[i] * 2 + b[i]
        total = 0.0
        for i in numba.prange(n):
            total += out[i]
        return total

    rng = np.random.default_rng(3)
    a = rng.integers(-5, 6, 5000).astype(np.float32)
    b = rng.integers(-5, 6, 5000).astype(np.float32)
    want = np.zeros_like(a)
    want_total = py_func(a, b, want)
    f = nm.njit(py_func)
    out = nm.zeros(5000, np.float32)
    f(_dev(a), _dev(b), out)
    (total, n) = _launched(f, _dev(a), _dev(b), out)
    assert n == 2
    assert np.array_equal(out.copy_to_host(), want) and total == want_total


def test_loops_mixed_with_array_expressions_and_host_scalars(queue):
    import numba

    import numba_mlir_b200 as nm

    def py_func(a, w, out):
        scaled = a * w                      # array expression
        m = 0.0
        for i in numba.prange(a.shape[0]):  # loop reading the expression's value
            m = max(m, scaled[i])
        if m > 100.0:                       # host control flow on the loop's result
            m = 100.0
        for i in numba.prange(a.shape[0]):
            out[i] = scaled[i] / m
        out[:] = out + np.float32(1)        # array expression after the loops
        return m

    rng = np.random.default_rng(4)
    a = rng.uniform(1, 9, 3000).astype(np.float32)
    for w in (np.float32(2.0), np.float32(50.0)):
        want = np.zeros_like(a)
        scaled = a * w
        m = min(float(scaled.max()), 100.0)
        want = (scaled / np.float32(m)).astype(np.float32) + np.float32(1)
        out = nm.zeros(3000, np.float32)
        got_m = nm.njit(py_func)(_dev(a), w, out)
        assert float(got_m) == m
        np.testing.assert_allclose(out.copy_to_host(), want, rtol=1e-6)


def test_loops_without_host_scalars_are_replayed_from_the_plan(queue):
    """A function cut at its loops whose loops hand nothing back to the host
    code is recorded once per signature (loops and array expressions alike are
    steps of the plan) and replayed on later calls; new data, a scalar
    argument and a different length all give NumPy's results."""
    import numba

    import numba_mlir_b200 as nm

    def py_func(a, b, alpha, out):
        tmp = a * alpha + b                  # array expression
        for i in numba.prange(a.shape[0]):   # loop over the expression's value
            out[i] = tmp[i] * tmp[i]
        out[:] = out - b                     # array expression between the loops
        for i in numba.prange(a.shape[0] - 1):
            out[i] = out[i] + a[i + 1]

    def want(a, b, alpha):
        tmp = a * alpha + b
        o = tmp * tmp - b
        o[:-1] = o[:-1] + a[1:]
        return o

    f = nm.njit(py_func)
    rng = np.random.default_rng(8)
    for n, alpha in ((4000, 2.0), (4000, 3.0), (4000, -1.5), (1000, 0.5), (1000, 4.0)):
        a = rng.integers(-4, 5, n).astype(np.float32)
        b = rng.integers(-4, 5, n).astype(np.float32)
        out = nm.zeros(n, np.float32)
        f(_dev(a), _dev(b), np.float32(alpha), out)
        assert np.array_equal(out.copy_to_host(), want(a, b, np.float32(alpha)))
    assert len(f._plans) == 2  # one plan per length, reused by the later calls


def test_njit_replace_parfors_offloads_only_the_loops(queue):
    """mlir_njit_replace_parfors (decorators.py:84-104): the loops go to the
    device, the code around them stays on the host, also when there is only
    one loop and host code before it stores to an array."""
    import numba

    import numba_mlir_b200 as nm

    @nm.njit_replace_parfors(parallel=True)
    def f(a, out):
        out[:] = a - np.float32(1)          # a store before the loop: rejected when the whole
        s = 0.0                             # function is one kernel, fine when only the loop is
        for i in numba.prange(a.shape[0]):
            s += out[i] * out[i]
        return s

    a = np.arange(1, 2001, dtype=np.float32)
    out = nm.zeros(2000, np.float32)
    s = f(_dev(a), out)
    assert np.array_equal(out.copy_to_host(), a - 1)
    assert s == float(((a - 1).astype(np.float64) ** 2).sum())


def test_loop_function_carrying_two_scalars_is_refused_clearly(queue):
    import numba

    import numba_mlir_b200 as nm

    def py_func(a, out):
        s = 0.0
        t = 0.0
        for i in numba.prange(a.shape[0]):
            s += a[i]
            t += a[i] * 2
        for i in numba.prange(a.shape[0]):
            out[i] = s + t
        return s

    with pytest.raises(TypeError, match="several scalars"):
        nm.njit(py_func)(_dev(np.ones(8, np.float32)), nm.zeros(8, np.float32))
