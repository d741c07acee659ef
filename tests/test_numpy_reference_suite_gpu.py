"""Array-function cases of the reference's NumPy test-suite that reach the
offload path (numba_mlir/mlir/tests/test_numpy.py:483-514,761-792,1296-1307 and
the elementwise tables of mlir/numpy/funcs.py:338-573), restated on device
arrays: NumPy on the host copy is the expected result.  Python scalars are
typed the way Numba types them (float64 / int64), so the cases that mix them
with narrower arrays spell the scalar's type out."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def _host(x):
    return x.copy_to_host() if hasattr(x, "copy_to_host") else x


def _reduce_axis_funcs():
    template = [
        "lambda a: np.%s(a, dtype=np.int16)",
        "lambda a: np.%s(a, dtype=np.int16, axis=0)",
        "lambda a: np.%s(a, axis=0)",
        "lambda a: np.%s(a, axis=1)",
        "lambda a: np.%s(a, axis=-1)",
        "lambda a: np.%s(a, axis=-2)",
        "lambda a: np.%s(a, axis=0, keepdims=False)",
        "lambda a: np.%s(a, axis=0, keepdims=True)",
    ]
    res = []
    for func in ["sum", "amax", "amin", "max", "min", "prod", "mean"]:
        for t in template:
            if ("max" in func or "min" in func) and "dtype=" in t:
                continue
            res.append(t % func)
    return res


@pytest.mark.parametrize("src", _reduce_axis_funcs())
@pytest.mark.parametrize("dtype", [np.int32, np.float32])
def test_reduce_axis(queue, src, dtype):
    import numba_mlir_b200 as nm

    py_func = eval(src)
    arr = np.array([[1, 2, 3], [4, 5, 6]], dtype=dtype)
    want = py_func(arr)
    got = _host(nm.njit(py_func)(_dev(arr)))
    np.testing.assert_equal(np.asarray(got), want)
    assert np.asarray(got).dtype == np.asarray(want).dtype, (np.asarray(got).dtype, np.asarray(want).dtype)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
def test_np_reduce(queue, dtype):
    import numba_mlir_b200 as nm

    arr = np.array([[1, 2, 3], [4, 5, 6]], dtype=dtype)
    got = _host(nm.njit(lambda a: a.sum())(_dev(arr)))
    np.testing.assert_equal(np.asarray(got), arr.sum())


_unary = ["np.sqrt(a)", "np.square(a)", "np.log(a)", "np.exp(a)", "np.sin(a)", "np.cos(a)", "np.tanh(a)",
          "np.abs(a)", "np.negative(a)", "np.floor(a)", "np.ceil(a)", "np.arccos(a * np.float32(0.1))", "-a", "+a",
          "np.logical_not(a)", "np.isnan(a)", "np.isfinite(a)", "a.astype(np.int32)", "a.astype(np.float64)"]
_binary = ["a + b", "a - b", "a * b", "a / b", "a // b", "a % b", "a ** b", "np.add(a, b)",
           "np.subtract(a, b)", "np.multiply(a, b)", "np.true_divide(a, b)", "np.power(a, b)",
           "np.arctan2(a, b)", "np.minimum(a, b)", "np.maximum(a, b)", "np.where(a < b, a, b)",
           "np.logical_and(a, b)", "np.logical_or(a, b)", "np.logical_xor(a, b)", "a < b", "a <= b",
           "a > b", "a >= b", "a == b", "a != b", "np.clip(a, 2, 4)"]


@pytest.mark.parametrize("src", _unary)
def test_unary_array_functions(queue, src):
    import numba_mlir_b200 as nm

    py_func = eval("lambda a: " + src)
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    want = py_func(a)
    got = _host(nm.njit(py_func)(_dev(a)))
    assert got.dtype == want.dtype, (got.dtype, want.dtype)
    np.testing.assert_allclose(got, want, rtol=1e-6)


@pytest.mark.parametrize("src", _binary)
@pytest.mark.parametrize("dtype", [np.int32, np.float32])
def test_binary_array_functions(queue, src, dtype):
    import numba_mlir_b200 as nm

    py_func = eval("lambda a, b: " + src)
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype)
    b = np.array([[3, 1, 2], [6, 4, 5]], dtype)
    want = py_func(a, b)
    got = _host(nm.njit(py_func)(_dev(a), _dev(b)))
    assert got.dtype == want.dtype, (got.dtype, want.dtype)
    np.testing.assert_allclose(got, want, rtol=1e-6)


_bitwise = ["a & b", "a | b", "a ^ b", "a << np.int32(1)", "a >> np.int32(1)", "~a", "np.bitwise_and(a, b)", "np.bitwise_or(a, b)",
            "np.bitwise_xor(a, b)"]


@pytest.mark.parametrize("src", _bitwise)
def test_bitwise_array_functions(queue, src):
    import numba_mlir_b200 as nm

    py_func = eval("lambda a, b: " + src)
    a = np.array([[1, 2, 3], [4, 5, 6]], np.int32)
    b = np.array([[3, 1, 2], [6, 4, 5]], np.int32)
    want = py_func(a, b)
    got = _host(nm.njit(py_func)(_dev(a), _dev(b)))
    assert got.dtype == want.dtype
    np.testing.assert_equal(got, want)
