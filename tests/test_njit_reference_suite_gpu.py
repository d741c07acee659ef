"""The reference's offload tests for `njit` functions on device arrays
(numba_mlir/mlir/tests/test_gpu.py:1616-2220), restated: the Python function
run on NumPy arrays is the expected result."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def test_cfd_simple_and_indirect(queue):
    import numba_mlir_b200 as nm

    def py_func1(a, b):
        b[:] = a * 2

    def py_func2(a, b, c):
        c[:] = a + b

    a = np.arange(1024, dtype=np.float32)
    b = np.arange(1024, dtype=np.float32) * 3
    want = np.zeros_like(a)
    py_func1(a, want)
    got = _dev(np.zeros_like(a))
    nm.njit(py_func1)(_dev(a), got)
    np.testing.assert_equal(got.copy_to_host(), want)

    py_func2(a, b, want)
    nm.njit(py_func2)(_dev(a), _dev(b), got)
    np.testing.assert_equal(got.copy_to_host(), want)

    jit_func1 = nm.njit(py_func1)

    def outer(a, b):
        jit_func1(a, b)

    py_func1(a, want)
    got = _dev(np.zeros_like(a))
    nm.njit(outer)(_dev(a), got)
    np.testing.assert_equal(got.copy_to_host(), want)


def test_cfd_f64_truncate_option_is_accepted(queue):
    import numba_mlir_b200 as nm

    def py_func(a, b, c):
        c[:] = a + b

    a = np.arange(1024, dtype=np.float32)
    want = np.zeros_like(a)
    py_func(a, 2.5, want)
    got = _dev(np.zeros_like(a))
    nm.njit(py_func, gpu_fp64_truncate=True)(_dev(a), 2.5, got)
    np.testing.assert_equal(got.copy_to_host(), want)


def test_cfd_reshape(queue):
    import numba_mlir_b200 as nm

    def py_func1(a):
        b = a.reshape(17, 23, 56)
        b[:] = 42

    jit_func1 = nm.njit(py_func1)

    def py_func2(a):
        jit_func1(a)

    want = np.zeros((23, 56, 17), np.float32)
    py_func1(want)
    got = _dev(np.zeros((23, 56, 17), np.float32))
    nm.njit(py_func2)(got)
    np.testing.assert_equal(got.copy_to_host(), want)


def test_l2_norm(queue):
    import numba_mlir_b200 as nm

    def py_func(a, d):
        sq = np.square(a)
        sum = sq.sum(axis=1)
        d[:] = np.sqrt(sum)

    src = np.arange(10 * 10, dtype=np.float32).reshape(10, 10)
    want = np.zeros(10, np.float32)
    py_func(src, want)
    got = _dev(np.zeros(10, np.float32))
    nm.njit(py_func)(_dev(src), got)
    np.testing.assert_allclose(got.copy_to_host(), want, rtol=1e-5)


@pytest.mark.parametrize("a_shape,b_shape", [((4, 8), (8, 16)), ((128, 64), (64, 256)), ((1, 3), (3, 1))])
def test_cfd_dot(queue, a_shape, b_shape):
    import numba_mlir_b200 as nm

    def py_func(a, b, c):
        c[:] = np.dot(a, b)

    a = np.arange(np.prod(a_shape), dtype=np.float32).reshape(a_shape) % 7
    b = np.arange(np.prod(b_shape), dtype=np.float32).reshape(b_shape) % 5
    want = np.zeros((a_shape[0], b_shape[1]), np.float32)
    py_func(a, b, want)
    got = _dev(np.zeros_like(want))
    nm.njit(py_func)(_dev(a), _dev(b), got)
    np.testing.assert_equal(got.copy_to_host(), want)  # small integer-valued floats: exact
