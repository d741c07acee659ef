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


_A = np.arange(24, dtype=np.float32).reshape(4, 6)
_B = np.arange(6, dtype=np.float32)
_array_cases = {
    "slice_rows": (lambda a: a[1:3] * 2, (_A,)),
    "slice_step": (lambda a: a[::2, 1::2] + 1, (_A,)),
    "negative_index": (lambda a: a[-1] + a[0], (_A,)),
    "row": (lambda a: a[2] * 3, (_A,)),
    "transpose": (lambda a: a.T + 1, (_A,)),
    "np_transpose": (lambda a: np.transpose(a) + 1, (_A,)),
    "zeros": (lambda a: np.zeros((4, 6), np.float32) + a, (_A,)),
    "ones": (lambda a: np.ones((4, 6), np.float32) + a, (_A,)),
    "full": (lambda a: np.full((4, 6), 2.5, np.float32) * a, (_A,)),
    "zeros_like": (lambda a: np.zeros_like(a) + a, (_A,)),
    "ones_like": (lambda a: np.ones_like(a) + a, (_A,)),
    "shape_attributes": (lambda a: a.shape[0] * a + a.ndim + a.size, (_A,)),
    "broadcast_1d": (lambda a, b: a + b, (_A, _B)),
    "outer": (lambda a, b: b.reshape(6, 1) * b.reshape(1, 6), (_A, _B)),
    "flat_sum": (lambda a: a.reshape(-1).sum(), (_A,)),
    "ravel": (lambda a: a.ravel() * 2, (_A,)),
    "flatten": (lambda a: a.flatten() * 2, (_A,)),
    "astype_floordiv": (lambda a: a.astype(np.int32) // 2, (_A,)),
    "where": (lambda a: np.where(a > 5, a, -a), (_A,)),
    "norm": (lambda a: np.sqrt((a * a).sum(axis=1)), (_A,)),
    "mean_axis0": (lambda a: a.mean(axis=0), (_A,)),
    "std": (lambda a: np.std(a), (_A,)),
    "var_axis1": (lambda a: np.var(a, axis=1), (_A,)),
    "copy": (lambda a: a.copy() + 1, (_A,)),
    "np_copy": (lambda a: np.copy(a) + 1, (_A,)),
    "abs": (lambda a: abs(a - 10), (_A,)),
    "exp2": (lambda a: np.exp2(a * np.float32(0.1)), (_A,)),
    "cbrt": (lambda a: np.cbrt(a), (_A,)),
    "degrees": (lambda a: np.degrees(a), (_A,)),
    "arange": (lambda a: np.arange(6) + a, (_A,)),
    "linspace": (lambda a: np.linspace(0, 1, 6) + a, (_A,)),
    "eye": (lambda a: np.eye(4, 6) + a, (_A,)),
    "dot_matrix_vector": (lambda a, b: np.dot(a, b), (_A, _B)),
    "dot_vector_vector": (lambda a, b: np.dot(b, b), (_A, _B)),
    "matmul": (lambda a: a @ a.T, (_A,)),
    "maximum_max": (lambda a: np.maximum(a, 3).max(), (_A,)),
    "any": (lambda a: np.any(a > 20), (_A,)),
    "all_axis0": (lambda a: np.all(a >= 3, axis=0), (_A,)),
    "count_nonzero": (lambda a: np.count_nonzero(a > 5), (_A,)),
    "argmax": (lambda a: np.argmax(a), (_A,)),
    "concatenate": (lambda a: np.concatenate((a, a)), (_A,)),
    "concatenate_axis1": (lambda a: np.concatenate((a, a * 2), axis=1), (_A,)),
    "tuple_result": (lambda a: (a + 1, a * 2), (_A,)),
    "scalar_argument": (lambda a, s: a * s, (_A, np.float32(3))),
}


@pytest.mark.parametrize("name", sorted(_array_cases))
def test_array_functions_and_methods(queue, name):
    import numba_mlir_b200 as nm

    f, args = _array_cases[name]
    want = f(*args)
    got = nm.njit(f)(*[_dev(x) if isinstance(x, np.ndarray) else x for x in args])
    if isinstance(want, tuple):
        for g, w in zip(got, want):
            np.testing.assert_allclose(_host(g), w, rtol=1e-5)
    else:
        np.testing.assert_allclose(np.asarray(_host(got)), np.asarray(want), rtol=1e-5)


def test_in_place_operators_and_slice_assignment_write_through(queue):
    import numba_mlir_b200 as nm

    def f(a, o, p):
        o += a
        o *= np.float32(2)
        p[1:3] = a[1:3] * 2

    o, p = np.ones_like(_A), np.zeros_like(_A)
    f(_A, o, p)
    do, dp = _dev(np.ones_like(_A)), _dev(np.zeros_like(_A))
    nm.njit(f)(_dev(_A), do, dp)
    np.testing.assert_equal(do.copy_to_host(), o)
    np.testing.assert_equal(dp.copy_to_host(), p)


def test_assignment_into_strided_views(queue):
    import numba_mlir_b200 as nm

    def f(a, o, t):
        o[:, 1:4] = a[:, 0:3] * 2
        o[::2, 5] = np.float32(7)
        t.T[:] = a

    o, t = np.zeros_like(_A), np.zeros((6, 4), np.float32)
    f(_A, o, t)
    do, dt = _dev(np.zeros_like(_A)), _dev(np.zeros((6, 4), np.float32))
    nm.njit(f)(_dev(_A), do, dt)
    np.testing.assert_equal(do.copy_to_host(), o)
    np.testing.assert_equal(dt.copy_to_host(), t)
