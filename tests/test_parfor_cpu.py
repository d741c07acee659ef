"""Host-side checks of the `prange` path: loop analysis, generated source
(NVRTC-compiled for sm_100a without a device) and launch shapes."""

import numba
import numpy as np
import pytest


def _compile(fn, args):
    from numba_mlir_b200 import codegen_ir, runtime

    ck = codegen_ir.compile_parfor(fn, args)
    assert len(runtime.compile_to_cubin(ck.source)) > 0
    return ck


def test_outer_loop_is_grid_strided_and_extent_is_known(runtime_lib):
    def f(a, b, c):
        for i in numba.prange(len(a)):
            c[i] = a[i] + b[i]

    x = np.zeros(1000, np.float32)
    ck = _compile(f, (x, x, x))
    assert not ck.inner_parallel
    assert ck.extents((x, x, x)) == [1000]
    assert "nmb_oid" in ck.source and "nmb_iid" not in ck.source


def test_directly_nested_prange_takes_the_x_dimension(runtime_lib):
    def f(a, c, d):
        n = a.shape[0]
        for i in numba.prange(n):
            for j in numba.prange(a.shape[1]):
                c[i, j] = a[i, j] * d

    x = np.zeros((8, 48), np.float32)
    ck = _compile(f, (x, x, np.float32(2)))
    assert ck.inner_parallel
    assert ck.extents((x, x, 2.0)) == [8, 48]


def test_inner_reduction_keeps_the_inner_loop_sequential(runtime_lib):
    def f(a, c):
        for i in numba.prange(a.shape[0]):
            s = 0.0
            for j in numba.prange(a.shape[1]):
                s += a[i, j]
            c[i] = s

    x = np.zeros((8, 48), np.float32)
    ck = _compile(f, (x, np.zeros(8, np.float32)))
    assert not ck.inner_parallel


def test_update_of_an_element_becomes_an_atomic(runtime_lib):
    def f(n, s, res):
        for i in numba.prange(n):
            res[i % s] += np.float32(i)

    ck = _compile(f, (10000, 10, np.zeros(10, np.float32)))
    assert "nmb::atomic_add" in ck.source
    assert ck.extents((10000, 10, None)) == [10000]


def test_store_before_the_loop_is_rejected_and_after_it_runs_once(runtime_lib):
    from numba_mlir_b200 import codegen_ir

    def before(a):
        a[0] = 1.0
        for i in numba.prange(len(a)):
            a[i] = 2.0

    with pytest.raises(codegen_ir.UnsupportedError, match="before"):
        codegen_ir.compile_parfor(before, (np.zeros(4, np.float32),))

    def after(a, out):
        for i in numba.prange(len(a)):
            a[i] = 2.0
        out[0] = 5.0

    ck = _compile(after, (np.zeros(4, np.float32), np.zeros(1, np.float32)))
    assert ck.epilogue == 8  # no reductions, but the tail needs the ticket


def test_launch_shapes():
    from numba_mlir_b200.decorators import parfor_launch_shape as shape

    assert shape([1024], False) == ((4,), (256,))
    assert shape([0], False) == (None, None)
    assert shape([None], False) == ((148 * 8,), (256,))
    grid, block = shape([16384, 4096], True)
    assert block == (256, 1) and grid[0] == 16 and grid[0] * grid[1] <= 148 * 32
    assert shape([8, 16], True) == ((1, 1), (16, 16))
    grid, block = shape([1 << 22, 3], True)
    assert block == (4, 64) and grid[0] == 1


def test_reductions_are_recognised_and_get_the_grid_epilogue(runtime_lib):
    def f(a):
        s = 0.0
        m = a[0]
        for i in numba.prange(len(a)):
            s += a[i]
            m = min(m, a[i])
        return s + m

    ck = _compile(f, (np.zeros(100, np.float32),))
    assert ck.epilogue == 16 and ck.return_dtype == np.float64 and not ck.inner_parallel
    assert "nmb_ticket" in ck.source and "nmb::block_reduce" in ck.source


def test_running_value_read_inside_the_loop_is_not_a_reduction():
    from numba_mlir_b200 import codegen_ir

    def f(a, out):
        s = 0.0
        for i in numba.prange(len(a)):
            s += a[i]
            out[i] = s  # a prefix sum: order dependent

    with pytest.raises(codegen_ir.UnsupportedError, match="not a reduction"):
        codegen_ir.compile_parfor(f, (np.zeros(4, np.float32), np.zeros(4, np.float32)))
