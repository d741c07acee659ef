"""`@kernel` programs on the GPU against the reference simulator's golden
vectors (tests/golden/kernel_sim.npz) and the CPU simulator restatement."""

import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "kernel_sim.npz"))


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def _both(func, gsize, lsize, host_args):
    """Runs `func` under the CPU simulator and on the device; returns the two
    lists of output arrays (all array arguments are copied back)."""
    from numba_mlir_b200.kernel import kernel
    from oracle.kernel_sim import kernel_sim

    sim_args = [a.copy() if isinstance(a, np.ndarray) else a for a in host_args]
    kernel_sim(func)[gsize, lsize](*sim_args)
    dev_args = [_dev(a) if isinstance(a, np.ndarray) else a for a in host_args]
    kernel(func)[gsize, lsize](*dev_args)
    gpu = [a.copy_to_host() if hasattr(a, "copy_to_host") else a for a in dev_args]
    return sim_args, gpu


def test_simple_add_kernel(queue):
    # README.md:66-92 of the reference
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, get_global_id

    def foo(a, b, c):
        i = get_global_id(0)
        j = get_global_id(1)
        c[i, j] = a[i, j] + b[i, j]

    a = np.arange(35, dtype=np.float32).reshape(5, 7)
    b = a * 3
    sim, gpu = _both(foo, a.shape, DEFAULT_LOCAL_SIZE, [a, b, np.zeros_like(a)])
    assert np.array_equal(gpu[2], a + b) and np.array_equal(sim[2], gpu[2])


@pytest.mark.parametrize("gsize,lsize", [(27, 7), (67, 17), (101, 33), (4, 2)])
def test_ids_and_sizes(queue, gsize, lsize):
    # mlir/tests/test_gpu.py:580-803; global size not a multiple of local size
    from numba_mlir_b200.kernel import (get_global_id, get_global_size, get_group_id,
                                        get_local_id, get_local_size, kernel)

    def k_ids(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        gid[i] = i
        lid[i] = get_local_id(0)
        grp[i] = get_group_id(0)
        gsz[i] = get_global_size(0)
        lsz[i] = get_local_size(0)

    arrs = [_dev(np.full(gsize, -1, np.int64)) for _ in range(5)]
    kernel(k_ids)[gsize, lsize](*arrs)
    for name, arr in zip(("gid", "lid", "grp", "gsz", "lsz"), arrs):
        assert np.array_equal(arr.copy_to_host(), GOLDEN[f"ids_{gsize}_{lsize}_{name}"]), name


def test_ids_2d(queue):
    from numba_mlir_b200.kernel import get_global_id, get_group_id, get_local_id, kernel

    def k_ids2(out2):
        i = get_global_id(0)
        j = get_global_id(1)
        out2[i, j] = 1000 * get_group_id(0) + 100 * get_group_id(1) + 10 * get_local_id(0) + get_local_id(1)

    res = _dev(np.zeros((5, 7), np.int64))
    kernel(k_ids2)[(5, 7), (2, 3)](res)
    assert np.array_equal(res.copy_to_host(), GOLDEN["ids2d_5x7_2x3"])


@pytest.mark.parametrize("dtype", ["int32", "int64", "float32"])
@pytest.mark.parametrize("opname", ["add", "sub"])
def test_atomics(queue, dtype, opname):
    # mlir/tests/test_gpu.py:820-870; integer and small-integer float sums are
    # order independent, so the result is bit-exact
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, atomic, get_global_id, kernel

    atomic_op = getattr(atomic, opname)

    def func(a, b):
        i = get_global_id(0)
        atomic_op(b, 0, a[i])

    def func_off(a, b):
        i = get_global_id(0)
        atomic_op(b, i % 2, a[i])

    a = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9], dtype)
    res = _dev(np.zeros([1], dtype))
    kernel(func)[a.shape, DEFAULT_LOCAL_SIZE](_dev(a), res)
    assert np.array_equal(res.copy_to_host(), GOLDEN[f"atomic_{opname}_{dtype}"])
    res = _dev(np.zeros([2], dtype))
    kernel(func_off)[a.shape, DEFAULT_LOCAL_SIZE](_dev(a), res)
    assert np.array_equal(res.copy_to_host(), GOLDEN[f"atomic_{opname}_offset_{dtype}"])


def test_atomics_inline_attribute_and_2d_index(queue):
    # the `atomic.add(...)` spelling the reference marks xfail (test_gpu.py:848-855)
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, atomic, get_global_id, kernel

    def k_2d(a, b):
        i = get_global_id(0)
        j = get_global_id(1)
        atomic.add(b, (i % 2, j % 2), a[i, j])

    for dtype in ("int32", "int64", "float32"):
        a2 = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], dtype)
        res = _dev(np.zeros((2, 2), dtype))
        kernel(k_2d)[a2.shape, DEFAULT_LOCAL_SIZE](_dev(a2), res)
        assert np.array_equal(res.copy_to_host(), GOLDEN[f"atomic_add_2d_{dtype}"])


def test_pairwise_kernel_reference_case(queue):
    # mlir/tests/test_gpu.py:1396-1430, rtol 1e-5 (bit-exact here: same typing)
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, get_global_id, kernel

    def func(X1, X2, D):
        i = get_global_id(0)
        j = get_global_id(1)
        X1_cols = X1.shape[1]
        d = 0.0
        for k in range(X1_cols):
            tmp = X1[i, k] - X2[j, k]
            d += tmp * tmp
        D[i, j] = np.sqrt(d)

    a = np.arange(128 * 3, dtype=np.float32).reshape(128, 3)
    b = a + 5
    res = _dev(np.zeros((128, 128), np.float32))
    kernel(func)[(a.shape[0], b.shape[0]), DEFAULT_LOCAL_SIZE](_dev(a), _dev(b), res)
    np.testing.assert_allclose(res.copy_to_host(), GOLDEN["pairwise1"], rtol=1e-5)


def test_scalars_closures_math_and_casts(queue):
    # mlir/tests/test_gpu.py:287-344,524-567
    import math

    from numba_mlir_b200.kernel import get_global_id, kernel

    scale = 2.5  # captured Python float -> float64

    def func(a, out, n, bias):
        i = get_global_id(0)
        if i < n:
            x = a[i]
            out[i] = math.sqrt(abs(x)) * scale + math.erf(x) + bias - float(i // 3) + (i % 4)

    a = np.linspace(-3, 3, 100).astype(np.float32)
    out = _dev(np.zeros(100, np.float64))
    kernel(func)[128](_dev(a), out, 100, np.float32(0.5))
    i = np.arange(100)
    from scipy.special import erf

    want = np.sqrt(np.abs(a)).astype(np.float32).astype(np.float64) * 2.5 + erf(a.astype(np.float64)) \
        + 0.5 - (i // 3) + (i % 4)
    np.testing.assert_allclose(out.copy_to_host(), want, rtol=1e-6, atol=1e-6)


def test_local_memory_barrier_and_group_reduce(queue):
    # mlir/tests/test_gpu.py:1074-1135,1138-1327,1361-1393
    from numba_mlir_b200.kernel import (LOCAL_MEM_FENCE, barrier, get_global_id, get_local_id,
                                        get_local_size, group, kernel, local)

    def func(a, b, c):
        i = get_global_id(0)
        l = get_local_id(0)
        tmp = local.array(64, np.float32)
        tmp[l] = a[i]
        barrier(LOCAL_MEM_FENCE)
        b[i] = tmp[get_local_size(0) - 1 - l]
        c[i] = group.reduce_add(a[i]) + group.reduce_max(a[i])

    a = np.arange(256, dtype=np.float32)
    b, c = _dev(np.zeros_like(a)), _dev(np.zeros_like(a))
    kernel(func)[256, 64](_dev(a), b, c)
    blocks = a.reshape(4, 64)
    assert np.array_equal(b.copy_to_host(), blocks[:, ::-1].reshape(-1))
    want_c = np.repeat(blocks.sum(axis=1) + blocks.max(axis=1), 64)
    assert np.array_equal(c.copy_to_host(), want_c)


_BIG_LOCAL = 20000  # float32 elements: 80 KB, above the 48 KB of static shared memory


def _big_local_kernel():
    from numba_mlir_b200.kernel import barrier, get_group_id, get_local_id, get_local_size, local

    def func(a, out):
        lid = get_local_id(0)
        lsz = get_local_size(0)
        g = get_group_id(0)
        buf = local.array(_BIG_LOCAL, np.float32)
        idx = local.array(64, np.int32)
        j = lid
        while j < _BIG_LOCAL:
            buf[j] = a[g * _BIG_LOCAL + j]
            j += lsz
        if lid < 64:
            idx[lid] = lid
        barrier()
        j = lid
        while j < _BIG_LOCAL:
            out[g * _BIG_LOCAL + j] = buf[_BIG_LOCAL - 1 - j] + idx[j % 64]
            j += lsz

    return func


def test_local_arrays_beyond_static_shared_memory(queue):
    """Local arrays larger than 48 KB per group (the reference's local memory
    is bounded only by the device, mlir/kernel_impl.py:366-437) come out of the
    dynamic shared memory requested with a {NULL, size, ptr} launch parameter
    (GpuRuntimeToLlvm.cpp:514-528)."""
    from numba_mlir_b200.kernel import kernel

    groups = 6
    rng = np.random.default_rng(3)
    a = rng.standard_normal(groups * _BIG_LOCAL).astype(np.float32)
    out = _dev(np.zeros_like(a))
    k = kernel(_big_local_kernel())
    k[groups * 256, 256](_dev(a), out)
    blocks = a.reshape(groups, _BIG_LOCAL)
    want = blocks[:, ::-1] + (np.arange(_BIG_LOCAL) % 64).astype(np.float32)
    assert np.array_equal(out.copy_to_host(), want.reshape(-1))
    queue.check_status()


def test_private_array_and_kernel_func(queue):
    from numba_mlir_b200.kernel import get_global_id, kernel, kernel_func, private

    @kernel_func
    def sq(x):
        return x * x

    def func(a, out):
        i = get_global_id(0)
        tmp = private.array(4, np.float32)
        for k in range(4):
            tmp[k] = sq(a[i] + k)
        s = np.float32(0)
        for k in range(4):
            s += tmp[k]
        out[i] = s

    a = np.arange(50, dtype=np.float32)
    out = _dev(np.zeros_like(a))
    kernel(func)[50](_dev(a), out)
    want = sum((a + k) ** 2 for k in range(4))
    assert np.array_equal(out.copy_to_host(), want.astype(np.float32))


def test_packed_inner_loops_round_like_the_scalar_loop(queue):
    """Independent constant-trip loops over private arrays run two iterations
    at a time with packed float32 add/sub (numba_mlir_b200/codegen_ir.py).
    Every operation must still round on its own: x*y - float32(x*y) is
    exactly zero unless a product were fused into the subtraction, and the
    squared-distance accumulation equals NumPy's operation by operation."""
    from numba_mlir_b200.kernel import get_global_id, kernel, private

    def residual(x, y, z, out):
        i = get_global_id(0)
        v = private.array(4, np.float32)
        for q in range(4):
            t = x[4 * i + q] * y[4 * i + q]
            v[q] = t - z[4 * i + q]
        for q in range(4):
            out[4 * i + q] = v[q]

    def sqdist(x, c, out):
        i = get_global_id(0)
        p = private.array((2, 8), np.float32)
        d = private.array(2, np.float32)
        for q in range(2):
            for j in range(8):
                p[q, j] = x[2 * i + q, j]
            d[q] = np.float32(0.0)
        for j in range(8):
            cj = c[j]
            for q in range(2):
                t = p[q, j] - cj
                d[q] += t * t
        for q in range(2):
            out[2 * i + q] = d[q]

    rng = np.random.default_rng(11)
    n = 1 << 16
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    z = x * y
    out = _dev(np.ones(n, np.float32))
    kernel(residual)[n // 4](_dev(x), _dev(y), _dev(z), out)
    assert not out.copy_to_host().any()

    pts = rng.standard_normal((n, 8)).astype(np.float32)
    c = rng.standard_normal(8).astype(np.float32)
    out = _dev(np.zeros(n, np.float32))
    kernel(sqdist)[n // 2](_dev(pts), _dev(c), out)
    want = np.zeros(n, np.float32)
    for j in range(8):
        t = pts[:, j] - c[j]
        want = want + t * t
    assert np.array_equal(out.copy_to_host(), want)
    # fastmath=True allows a*b+c to contract: the products are packed too (and
    # merged with the sums), the result agrees to rounding
    out = _dev(np.zeros(n, np.float32))
    kernel(sqdist, fastmath=True)[n // 2](_dev(pts), _dev(c), out)
    np.testing.assert_allclose(out.copy_to_host(), want, rtol=2e-6)


def test_kwargs_and_mixed_devices_are_rejected(queue):
    from numba_mlir_b200.kernel import get_global_id, kernel

    def func(a):
        i = get_global_id(0)
        a[i] = 1

    a = _dev(np.zeros(4, np.float32))
    with pytest.raises(ValueError, match="kwargs"):
        kernel(func)[4](a=a)
    with pytest.raises(ValueError):
        kernel(func)[(1, 2, 3, 4)]


def test_kmeans_kernel_bit_exact_labels(queue):
    """Config 5 at reduced size: 3 Lloyd iterations of the @kernel body against
    the CPU oracle; labels bit-exact, centroids identical after the float64
    sums are rounded to float32."""
    from numba_mlir_b200 import zeros
    from numba_mlir_b200.workloads import kmeans_step
    from oracle import configs as O

    pts, c0 = O.make_inputs("kmeans", 1 / 64)  # 65536 points
    n, k, d = pts.shape[0], c0.shape[0], c0.shape[1]
    d_pts, cent = _dev(pts), c0.copy()
    labels = zeros(n, np.int32)
    for _ in range(3):
        sums, counts = zeros((k, d), np.float64), zeros(k, np.int64)
        kmeans_step(d_pts, _dev(cent), labels, sums, counts)
        cent = O.kmeans_update(cent, sums.copy_to_host(), counts.copy_to_host())
    want_labels, want_cent = O.kmeans(pts, c0, 3)
    assert np.array_equal(labels.copy_to_host(), want_labels)
    assert np.array_equal(cent.view(np.uint32), want_cent.view(np.uint32))
