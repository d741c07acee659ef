"""Parity of the reduction kernels against the CPU oracle / NumPy, through
the C-ABI.  Integer and index results are bit-exact; float32 sums are within
1e-5 of the float64 truth relative to sum(|a_i|) (a plain relative error is
ill-posed for sums that cancel to ~0) and float min/max are bit-exact."""

import itertools
import math
import warnings

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def _check_float_sum(got, a, axis):
    truth = a.astype(np.float64).sum(axis=axis)
    scale = np.abs(a).astype(np.float64).sum(axis=axis)
    assert np.all(np.abs(got.astype(np.float64) - truth) <= 1e-5 * scale + 1e-30)


def test_config3_axis_reductions(queue):
    from numba_mlir_b200 import reduce_ops
    from oracle import configs as O

    (a,) = O.make_inputs("reduce_f32", 1 / 8)  # (2048, 4096) ~ N(0,1)
    da = _dev(a)
    s1 = reduce_ops.reduce(da, "sum", 1).copy_to_host()
    assert s1.dtype == np.float32 and s1.shape == (a.shape[0],)
    _check_float_sum(s1, a, 1)
    _check_float_sum(O.sum_axis1(a), a, 1)  # the oracle meets the same bound
    m0 = reduce_ops.reduce(da, "min", 0).copy_to_host()
    assert np.array_equal(m0.view(np.uint32), O.min_axis0(a).view(np.uint32))
    am = reduce_ops.reduce(da, "argmin", 1).copy_to_host()
    assert am.dtype == np.int64
    assert np.array_equal(am, O.argmin_axis1(a))
    queue.check_status()


def test_config3_int_sum_bit_exact(queue):
    from numba_mlir_b200 import reduce_ops
    from oracle import configs as O

    (a,) = O.make_inputs("reduce_i32", 1 / 16)  # 2^24 int32 in [-1000, 1000]
    got = reduce_ops.reduce(_dev(a), "sum").copy_to_host()
    assert got.dtype == np.int64
    assert int(got) == int(O.int_sum(a)) == int(a.sum(dtype=np.int64))
    queue.check_status()


def test_int_sum_does_not_wrap_in_int32(queue):
    from numba_mlir_b200 import reduce_ops

    a = np.full(1 << 20, 2**31 - 1, np.int32)
    assert int(reduce_ops.reduce(_dev(a), "sum").copy_to_host()) == (2**31 - 1) * (1 << 20)


@pytest.mark.parametrize("size", [1, 7, 16, 64, 65, 256, 512, 1024 * 1024])
def test_full_sum_float32_arange(queue, size):
    # mlir/tests/test_gpu.py:2045-2062 (test_cfd_reduce1), rtol 1e-5
    from numba_mlir_b200 import reduce_ops

    a = np.arange(size, dtype=np.float32)
    got = reduce_ops.reduce(_dev(a), "sum").copy_to_host()
    np.testing.assert_allclose(got, a.astype(np.float64).sum(), rtol=1e-5)


_shapes = (1, 7, 16, 25, 64, 65)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
@pytest.mark.parametrize("op,axis", [("sum", None), ("sum", 0), ("sum", 1), ("prod", None),
                                     ("prod", 0), ("prod", 1), ("min", None), ("max", None)])
def test_reference_reduce_matrix(queue, op, axis, dtype):
    # mlir/tests/test_gpu.py:2065-2098 (test_cfd_reduce2): a = arange(1, n+1)
    from numba_mlir_b200 import reduce_ops

    fn = {"sum": np.sum, "prod": np.prod, "min": np.amin, "max": np.amax}[op]
    for shape in itertools.product(_shapes, _shapes):
        count = math.prod(shape)
        if op == "prod" and count > 30:
            continue  # the reference skips these (overflow)
        a = np.arange(1, count + 1, dtype=dtype).reshape(shape).copy()
        got = reduce_ops.reduce(_dev(a), op, axis).copy_to_host()
        want = fn(a, axis=axis)
        if np.dtype(dtype).kind == "i":
            assert np.array_equal(got, want), (shape, op, axis)
        else:
            np.testing.assert_allclose(got, want, rtol=1e-5)
    queue.check_status()


@pytest.mark.parametrize("shape", [(3, 12000), (5, 4096 * 3 + 8), (1000, 4), (77, 516), (4100, 260),
                                   (2, 1 << 20), (33, 13), (13, 33), (700, 4096), (37, 4100),
                                   (9, 8192), (1, 4096), (600, 2052)])
@pytest.mark.parametrize("op", ["sum", "min", "max", "argmin", "argmax"])
def test_axis_shapes_float32(queue, shape, op):
    """Multi-tile rows, many-rows-per-tile, column tails and unaligned shapes
    (the last two take the layout-agnostic kernel)."""
    from numba_mlir_b200 import reduce_ops

    rng = np.random.default_rng(3)
    a = rng.standard_normal(shape).astype(np.float32)
    a[:, 0] = a[:, -1]  # ties for argmin/argmax
    fn = {"sum": np.sum, "min": np.min, "max": np.max, "argmin": np.argmin, "argmax": np.argmax}[op]
    for axis in (0, 1):
        got = reduce_ops.reduce(_dev(a), op, axis).copy_to_host()
        if op == "sum":
            _check_float_sum(got, a, axis)
        else:
            assert np.array_equal(got, fn(a, axis=axis)), (shape, op, axis)
    queue.check_status()


def test_argmin_ties_pick_first_occurrence(queue):
    # pair combiner of numba_mlir/mlir/builtin/funcs.py:126-138
    from numba_mlir_b200 import reduce_ops

    a = np.ones((64, 8192), np.float32)
    a[:, 5000] = -1
    a[:, 77] = -1
    a[:, 8191] = -1
    assert np.array_equal(reduce_ops.reduce(_dev(a), "argmin", 1).copy_to_host(), np.full(64, 77))
    assert int(reduce_ops.reduce(_dev(a), "argmin").copy_to_host()) == 77
    b = np.ones((9000, 64), np.float32)
    b[[8000, 123, 4000], :] = -1
    assert np.array_equal(reduce_ops.reduce(_dev(b), "argmin", 0).copy_to_host(), np.full(64, 123))


@pytest.mark.parametrize("cols", [600, 4096, 5000])
def test_argmin_argmax_special_values_and_dense_ties(queue, cols):
    """Rows of equal values, signed zeros, infinities and NaNs (which never win
    a `<` comparison, numba_mlir/mlir/builtin/funcs.py:126-146), and many ties
    inside one 16-byte vector and one tile."""
    from numba_mlir_b200 import reduce_ops

    rng = np.random.default_rng(cols)
    a = rng.integers(0, 3, (40, cols)).astype(np.float32)      # dense ties
    a[1] = 7.0                                                 # one value everywhere
    a[2] = np.inf
    a[3] = -np.inf
    a[4, ::2] = -0.0
    a[4, 1::2] = 0.0
    a[5] = np.nan
    a[5, 123] = 4.0                                            # the only ordered value
    a[6, 17] = np.nan                                          # a NaN among ordinary values
    for op, fn in (("argmin", np.argmin), ("argmax", np.argmax)):
        got = reduce_ops.reduce(_dev(a), op, 1).copy_to_host()
        want = fn(a, axis=1)
        want[5] = 123                                          # NumPy would return the first NaN
        b = a[6].copy()
        b[17] = 1.0                                            # neither the minimum nor the maximum of the row
        want[6] = fn(b)
        np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
@pytest.mark.parametrize("cols", [1024, 4096, 5000])
def test_column_min_max_across_row_blocks(queue, dtype, cols):
    """min/max over axis 0 with enough rows that many row blocks meet in the
    result: columns of one sign and of mixed signs, infinities, signed zeros,
    NaNs (ignored: they never win `x < m`, numba_mlir/mlir/builtin/funcs.py:140-160,
    and the reduction starts from +-inf, numpy/funcs.py:278-295), an all-NaN
    column (the identity comes back), twice in a row (the scratch counters must be
    back at zero)."""
    from numba_mlir_b200 import reduce_ops

    rng = np.random.default_rng(cols)
    rows = 9000
    if np.dtype(dtype).kind == "f":
        a = (rng.standard_normal((rows, cols)) * 100).astype(dtype)
        a[:, 0] = np.abs(a[:, 0]) + 1          # all positive
        a[:, 1] = -np.abs(a[:, 1]) - 1         # all negative
        a[:, 2] = 0.0
        a[4000, 2] = -0.0
        a[5000, 3] = np.inf
        a[6000, 3] = -np.inf
        a[::7, 4] = np.nan
        a[:, 5] = np.nan
        a[:, 6] = np.abs(a[:, 6])
        a[8999, 6] = -1e-30                    # the only negative value, in the last row block
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # All-NaN slice
            want_min, want_max = np.nanmin(a, axis=0), np.nanmax(a, axis=0)
        want_min[5], want_max[5] = np.inf, -np.inf
    else:
        a = rng.integers(-10**6, 10**6, (rows, cols)).astype(dtype)
        a[:, 0] = np.abs(a[:, 0]) + 1
        a[:, 1] = -np.abs(a[:, 1]) - 1
        a[123, 2] = np.iinfo(dtype).min
        a[8123, 3] = np.iinfo(dtype).max
        want_min, want_max = a.min(axis=0), a.max(axis=0)
    d = _dev(a)
    for _ in range(2):
        assert np.array_equal(reduce_ops.reduce(d, "min", 0).copy_to_host(), want_min)
        assert np.array_equal(reduce_ops.reduce(d, "max", 0).copy_to_host(), want_max)
    queue.check_status()


@pytest.mark.parametrize("dtype", [np.float64, np.int64, np.int32])
def test_other_dtypes(queue, dtype):
    from numba_mlir_b200 import reduce_ops

    rng = np.random.default_rng(5)
    a = (rng.standard_normal((300, 2048)) * 1000).astype(dtype)
    for op, fn in (("sum", np.sum), ("min", np.min), ("max", np.max), ("argmax", np.argmax)):
        for axis in (None, 0, 1):
            got = reduce_ops.reduce(_dev(a), op, axis).copy_to_host()
            want = fn(a, axis=axis)
            if dtype == np.float64 and op == "sum":
                np.testing.assert_allclose(got, want, rtol=1e-10, atol=1e-6)
            else:
                assert np.array_equal(got, want), (op, axis)
    queue.check_status()


def test_strided_views_and_3d(queue):
    from numba_mlir_b200 import reduce_ops

    rng = np.random.default_rng(6)
    a = rng.integers(-50, 50, (40, 30, 20)).astype(np.int32)
    d = _dev(a)
    for axis in (0, 1, 2):
        assert np.array_equal(reduce_ops.reduce(d, "sum", axis).copy_to_host(), a.sum(axis=axis))
    m = rng.integers(-50, 50, (64, 48)).astype(np.int64)
    dm = _dev(m)
    assert np.array_equal(reduce_ops.reduce(dm.T, "sum", 0).copy_to_host(), m.T.sum(axis=0))
    assert np.array_equal(reduce_ops.reduce(dm[::2, 1:], "max", 1).copy_to_host(), m[::2, 1:].max(axis=1))
