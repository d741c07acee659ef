"""The reference's `@kernel` test-suite (numba_mlir/mlir/tests/test_gpu.py:180-1393),
restated: same kernel bodies, inputs and launch shapes; the expected values come
from the CPU simulator restatement (oracle/kernel_sim.py) or, for barriers and
group operations, from NumPy on the work-group structure."""

import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def _run(func, gsize, lsize, host_args, sim=True, **kernel_options):
    """Device run (and simulator run) of `func`; returns (sim outputs or None, gpu outputs)."""
    from numba_mlir_b200.kernel import kernel
    from oracle.kernel_sim import kernel_sim

    sim_args = None
    if sim:
        sim_args = [a.copy() if isinstance(a, np.ndarray) else a for a in host_args]
        kernel_sim(func)[gsize, lsize](*sim_args)
    dev_args = [_dev(a) if isinstance(a, np.ndarray) else a for a in host_args]
    kernel(func, **kernel_options)[gsize, lsize](*dev_args)
    gpu = [a.copy_to_host() if hasattr(a, "copy_to_host") else a for a in dev_args]
    return sim_args, gpu


def _local():
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE

    return DEFAULT_LOCAL_SIZE


def test_simple3(queue):
    from numba_mlir_b200.kernel import get_global_id

    def func(a, b):
        i = get_global_id(0)
        b[i, 0] = a[i, 0]
        b[i, 1] = a[i, 1]

    a = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    sim, gpu = _run(func, a.shape[0], _local(), [a, np.zeros_like(a)])
    np.testing.assert_equal(gpu[1], sim[1])


_vals = [True, False, -3, 0, 2, -2.5, -0.0, 0.5]


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
def test_scalar_and_scalar_capture(queue, dtype):
    from numba_mlir_b200.kernel import get_global_id

    get_id = get_global_id
    a = np.arange(-6, 6, dtype=dtype)
    for val in _vals:
        def func(a, b, c):
            i = get_id(0)
            c[i] = a[i] + b

        sim, gpu = _run(func, a.shape, _local(), [a, val, np.zeros_like(a)])
        np.testing.assert_equal(gpu[2], sim[2], err_msg=f"argument {val!r}")

        def func_capture(a, c):
            i = get_id(0)
            c[i] = a[i] + val

        sim, gpu = _run(func_capture, a.shape, _local(), [a, np.zeros_like(a)])
        np.testing.assert_equal(gpu[1], sim[1], err_msg=f"captured {val!r}")


def test_empty_kernel_and_list_args(queue):
    from numba_mlir_b200.kernel import get_global_id

    def empty(a):
        pass

    a = np.array([[[1, 2, 3], [4, 5, 6]]], np.float32)
    _sim, gpu = _run(empty, a.shape, _local(), [a])
    np.testing.assert_equal(gpu[0], a)

    def add(a, b, c):
        i = get_global_id(0)
        c[i] = a[i] + b[i]

    x = np.array([1, 2, 3, 4, 5, 6], np.float32)
    y = np.array([7, 8, 9, 10, 11, 12], np.float32)
    sim, gpu = _run(add, [x.shape[0]], [], [x, y, np.zeros_like(x)])
    np.testing.assert_equal(gpu[2], sim[2])


def test_slice(queue):
    """Partial indexing yields array views inside the kernel."""
    from numba_mlir_b200.kernel import get_global_id

    def func(a, b):
        i = get_global_id(0)
        b1 = b[i]
        j = get_global_id(1)
        b2 = b1[j]
        k = get_global_id(2)
        b2[k] = a[i, j, k]

    a = np.arange(3 * 4 * 5).reshape((3, 4, 5))
    sim, gpu = _run(func, a.shape, _local(), [a, np.zeros_like(a)])
    np.testing.assert_equal(gpu[1], sim[1])


def test_inner_loop(queue):
    from numba_mlir_b200.kernel import get_global_id

    def func(a, b, c):
        i = get_global_id(0)
        res = 0.0
        for j in range(a[i]):
            res = res + b[j]
        c[i] = res

    a = np.array([1, 2, 3, 4], np.int32)
    b = np.array([5, 6, 7, 8, 9], np.float32)
    sim, gpu = _run(func, a.shape, _local(), [a, b, np.zeros(a.shape, b.dtype)])
    np.testing.assert_equal(gpu[2], sim[2])


@pytest.mark.parametrize("op", ["sqrt", "log", "exp", "sin", "cos", "erf", "tanh", "floor", "ceil", "acos"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_math_funcs_unary(queue, op, dtype):
    from numba_mlir_b200.kernel import get_global_id

    f = getattr(math, op)

    def func(a, b):
        i = get_global_id(0)
        b[i] = f(a[i])

    a = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9], dtype)
    sim, gpu = _run(func, a.shape, _local(), [a, np.zeros_like(a)])
    np.testing.assert_allclose(gpu[1], sim[1], rtol=1e-5)


@pytest.mark.parametrize("op", ["+", "-", "*", "/", "//", "%", "**"])
@pytest.mark.parametrize("dtype", [np.int32, np.float32, np.float64])
def test_gpu_ops_binary(queue, op, dtype):
    from numba_mlir_b200.kernel import get_global_id, kernel_func

    f = eval(f"lambda a, b: a {op} b")
    inner = kernel_func(f)

    def func(a, b, c):
        i = get_global_id(0)
        c[i] = inner(a[i], b[i])

    def func_sim(a, b, c):
        i = get_global_id(0)
        c[i] = f(a[i], b[i])

    a = np.array([11, 12, 13, 14, 15], dtype)
    b = np.array([1, 2, 3, 4, 5], dtype)
    sim, _ = _run_sim_only(func_sim, a.shape, [a, b, np.zeros_like(a)])
    _none, gpu = _run(func, a.shape, _local(), [a, b, np.zeros_like(a)], sim=False)
    np.testing.assert_allclose(gpu[2], sim[2], rtol=1e-5)


def _run_sim_only(func, gsize, host_args):
    from oracle.kernel_sim import kernel_sim

    sim_args = [a.copy() if isinstance(a, np.ndarray) else a for a in host_args]
    kernel_sim(func)[gsize, _local()](*sim_args)
    return sim_args, None


_shapes = [(1,), (7,), (1, 1), (7, 13), (1, 1, 1), (7, 13, 23)]


@pytest.mark.parametrize("shape", _shapes)
@pytest.mark.parametrize("lsize", [None, (1, 1, 1), (2, 4, 8)])
def test_ids_and_sizes_in_1_to_3_dims(queue, shape, lsize):
    from numba_mlir_b200.kernel import (get_global_id, get_global_size, get_group_id, get_local_id,
                                        get_local_size)

    def f1(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        gid[i] = i
        lid[i] = get_local_id(0)
        grp[i] = get_group_id(0)
        gsz[i] = get_global_size(0)
        lsz[i] = get_local_size(0)

    def f2(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        j = get_global_id(1)
        gid[i, j] = i + j * 100
        lid[i, j] = get_local_id(0) + get_local_id(1) * 100
        grp[i, j] = get_group_id(0) + get_group_id(1) * 100
        gsz[i, j] = get_global_size(0) + get_global_size(1) * 100
        lsz[i, j] = get_local_size(0) + get_local_size(1) * 100

    def f3(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        j = get_global_id(1)
        k = get_global_id(2)
        gid[i, j, k] = i + j * 100 + k * 10000
        lid[i, j, k] = get_local_id(0) + get_local_id(1) * 100 + get_local_id(2) * 10000
        grp[i, j, k] = get_group_id(0) + get_group_id(1) * 100 + get_group_id(2) * 10000
        gsz[i, j, k] = get_global_size(0) + get_global_size(1) * 100 + get_global_size(2) * 10000
        lsz[i, j, k] = get_local_size(0) + get_local_size(1) * 100 + get_local_size(2) * 10000

    func = [f1, f2, f3][len(shape) - 1]
    ls = _local() if lsize is None else lsize[: len(shape)]
    outs = [np.zeros(shape, np.int32) for _ in range(5)]
    sim, gpu = _run(func, shape, ls, outs)
    names = ["global_id", "local_id", "group_id", "global_size", "local_size"]
    for name, s, g in zip(names, sim, gpu):
        if lsize is None and name in ("local_id", "group_id", "local_size"):
            continue  # the default local size is the implementation's choice
        np.testing.assert_equal(g, s, err_msg=name)


@pytest.mark.parametrize("sub", [False, True])
def test_atomics_different_types_and_dims(queue, sub):
    from numba_mlir_b200.kernel import atomic, get_global_id

    atomic_op = atomic.sub if sub else atomic.add

    def plus_one(a, b):
        i = get_global_id(0)
        atomic_op(b, 0, a[i] + 1)

    def literal(a, b):
        i = get_global_id(0)
        atomic_op(b, 0, 1)

    a = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9], np.int32)
    for func in (plus_one, literal):
        sim, gpu = _run(func, a.shape, _local(), [a, np.zeros(1, np.int32)])
        np.testing.assert_equal(gpu[1], sim[1])

    def f1(a, b):
        i = get_global_id(0)
        j = get_global_id(1)
        atomic_op(b, (i % 2, 0), a[i, j])

    def f2(a, b):
        i = get_global_id(0)
        j = get_global_id(1)
        atomic_op(b, (i % 2, j % 2), a[i, j])

    m = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], np.int32)
    for func in (f1, f2):
        sim, gpu = _run(func, m.shape, _local(), [m, np.zeros((2, 2), np.int32)])
        np.testing.assert_equal(gpu[1], sim[1])

    def dims(a, b, c):
        i = get_global_id(0)
        j = get_global_id(1)
        atomic_op(a, (i, j), c[i, j])
        atomic_op(b, (i), c[i, j])

    c = np.array([[1, 2, 3], [4, 5, 6]], np.int32)
    sim, gpu = _run(dims, c.shape, _local(), [np.zeros(c.shape, np.int32), np.zeros(2, np.int32), c])
    np.testing.assert_equal(gpu[0], sim[0])
    np.testing.assert_equal(gpu[1], sim[1])


@pytest.mark.parametrize("fastmath", [False, True])
def test_fastmath(queue, fastmath):
    from numba_mlir_b200.kernel import get_global_id

    def func(a, b, c, res):
        i = get_global_id(0)
        res[i] = a[i] * b[i] + c[i]

    def nested(a, b, res):
        i = get_global_id(0)
        d = np.float32(0)
        for j in range(10):
            d += a[i] * b[i]
        res[i] = d

    a = np.array([1, 2, 3, 4], np.float32)
    b = np.array([5, 6, 7, 8], np.float32)
    c = np.array([9, 10, 11, 12], np.float32)
    sim, gpu = _run(func, a.shape, _local(), [a, b, c, np.zeros_like(a)], fastmath=fastmath)
    np.testing.assert_equal(gpu[3], sim[3])
    sim, gpu = _run(nested, a.shape, _local(), [a, b, np.zeros_like(a)], fastmath=fastmath)
    np.testing.assert_equal(gpu[2], sim[2])


@pytest.mark.parametrize("global_size,local_size", [(1, 1), (2, 2), (27, 7), (67, 17), (101, 33), (4, 1)])
def test_barrier_ops_and_barrier1(queue, global_size, local_size):
    from numba_mlir_b200.kernel import (GLOBAL_MEM_FENCE, LOCAL_MEM_FENCE, atomic, barrier,
                                        get_global_id, mem_fence)

    atomic_add = atomic.add
    a = np.arange(global_size, dtype=np.int64)
    for op in (barrier, mem_fence):
        for flags in (LOCAL_MEM_FENCE, GLOBAL_MEM_FENCE):
            def func(a, b):
                i = get_global_id(0)
                v = a[i]  # noqa: F841
                op(flags)
                b[i] = a[i]

            _none, gpu = _run(func, global_size, local_size, [a, np.zeros_like(a)], sim=False)
            np.testing.assert_equal(gpu[1], a)

    def barrier1(a, b):
        i = get_global_id(0)
        off = i // local_size
        atomic_add(a, off, i)
        barrier(GLOBAL_MEM_FENCE)
        b[i] = a[off]

    count = (global_size + local_size - 1) // local_size
    _none, gpu = _run(barrier1, global_size, local_size,
                      [np.zeros(count, np.int64), np.zeros(global_size, np.int64)], sim=False)
    ids = np.arange(global_size)
    group_sums = np.bincount(ids // local_size, weights=ids, minlength=count).astype(np.int64)
    np.testing.assert_equal(gpu[0], group_sums)
    np.testing.assert_equal(gpu[1], group_sums[ids // local_size])


@pytest.mark.parametrize("blocksize", [1, 10, 17, 64, 67, 101])
def test_local_and_private_memory(queue, blocksize):
    from numba_mlir_b200.kernel import LOCAL_MEM_FENCE, barrier, get_global_id, local, private

    local_array = local.array
    private_array = private.array
    arr = np.arange(blocksize).astype(np.float32)

    def local1(A):
        lm = local_array(shape=blocksize, dtype=np.float32)
        i = get_global_id(0)
        lm[i] = A[i]
        barrier(LOCAL_MEM_FENCE)
        A[i] += lm[blocksize - 1 - i]

    def local2(A):
        lm = local_array(shape=(1, blocksize), dtype=np.float32)
        i = get_global_id(0)
        lm[0, i] = A[i]
        barrier(LOCAL_MEM_FENCE)
        A[i] += lm[0, blocksize - 1 - i]

    for func in (local1, local2):
        _none, gpu = _run(func, blocksize, blocksize, [arr], sim=False)
        np.testing.assert_allclose(gpu[0], arr + arr[::-1])

    def private1(A):
        i = get_global_id(0)
        prvt_mem = private_array(shape=1, dtype=np.float32)
        prvt_mem[0] = i
        barrier(LOCAL_MEM_FENCE)
        A[i] = prvt_mem[0] * 2

    def private2(A):
        i = get_global_id(0)
        prvt_mem = private_array(shape=(1, 1), dtype=np.float32)
        prvt_mem[0, 0] = i
        barrier(LOCAL_MEM_FENCE)
        A[i] = prvt_mem[0, 0] * 2

    def private4(A):
        i = get_global_id(0)
        S = 10
        prvt_mem = private_array(shape=(S, S), dtype=np.float32)
        for j in range(S):
            for k in range(S):
                prvt_mem[j, k] = i
        barrier(LOCAL_MEM_FENCE)
        A[i] = prvt_mem[i % S, i % S] * 2

    for func in (private1, private2, private4):
        _none, gpu = _run(func, blocksize, blocksize, [np.zeros(blocksize, np.float32)], sim=False)
        np.testing.assert_allclose(gpu[0], 2 * np.arange(blocksize, dtype=np.float32))

    for priv_size in (1, 11, 27):
        def private3(A):
            i = get_global_id(0)
            prvt_mem = private_array(shape=priv_size, dtype=np.float32)
            for j in range(priv_size):
                prvt_mem[j] = j + i
            res = 0
            for j in range(priv_size):
                res += prvt_mem[(j + i) % priv_size]
            A[i] = res

        sim, gpu = _run(private3, blocksize, blocksize, [np.zeros(blocksize, np.float32)])
        np.testing.assert_allclose(gpu[0], sim[0])


@pytest.mark.parametrize("name", ["reduce_add", "reduce_mul", "reduce_min", "reduce_max"])
@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
def test_group_func(queue, name, dtype):
    """Work-group reductions, including groups cut short by the global size."""
    from numba_mlir_b200.kernel import get_global_id, group

    group_op = getattr(group, name)
    np_op = {"reduce_add": np.add, "reduce_mul": np.multiply, "reduce_min": np.minimum,
             "reduce_max": np.maximum}[name]

    def func(a, b):
        i = get_global_id(0)
        v = group_op(a[i])
        b[i] = v

    for global_size in (1, 2, 4, 27, 67, 101):
        for local_size in (1, 2, 7, 17, 33):
            if global_size > 25 and name == "reduce_mul" and dtype is np.int64:
                continue  # the reference skips these (overflow)
            a = np.arange(global_size, dtype=dtype)
            want = np.zeros_like(a)
            for lo in range(0, global_size, local_size):
                with np.errstate(over="ignore"):
                    want[lo:lo + local_size] = np_op.reduce(a[lo:lo + local_size], dtype=dtype)
            _none, gpu = _run(func, (global_size,), (local_size,), [a, np.zeros_like(a)], sim=False)
            np.testing.assert_allclose(gpu[1], want, rtol=1e-5,
                                       err_msg=f"global {global_size} local {local_size}")


def test_kernel_suite_against_the_reference_simulators_golden_vectors(queue):
    """The cases of tests/kernel_cases.py on the device against what the
    reference's own kernel_sim_impl.py produced (tests/golden/kernel_sim.npz):
    exact for integer results and index bookkeeping, rtol 1e-5 (the reference's
    tolerance) for floating-point math."""
    import os

    from kernel_cases import cases
    from numba_mlir_b200.kernel import kernel

    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "kernel_sim.npz"))
    seen = 0
    for key, func, gsize, lsize, args, out_index, exact in cases(for_device=True):
        dev_args = [_dev(a) if isinstance(a, np.ndarray) else a for a in args]
        kernel(func)[gsize, lsize](*dev_args)
        got, want = dev_args[out_index].copy_to_host(), golden[key]
        assert got.dtype == want.dtype, key
        if exact:
            np.testing.assert_equal(got, want, err_msg=key)
        else:
            np.testing.assert_allclose(got, want, rtol=1e-5, err_msg=key)
        seen += 1
    assert seen == 98
