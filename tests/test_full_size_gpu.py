"""Parity at the sizes and through the code paths that the benchmark times.

Every case calls the product through the decorators (and those through the
gpux* C-ABI) and compares with the CPU oracle on identical seeded inputs:
bit-exact for min, argmin, integer sums and cluster labels; the Black-Scholes
chain within atol 2e-5 + rtol 1e-5; float32 sums within 1e-5 of the float64
truth relative to sum(|a_i|); distances and products within 1e-5 relative.
The reference tests the same programs at small sizes only
(mlir/tests/test_gpu.py:2226-2266 pairwise, :2065-2098 reductions,
mlir/tests/test_numpy.py:2796-2866 Black-Scholes)."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


# ------------------------------------------------------------ contraction ---
# The contraction kernel is persistent: min(tiles, SMs) CTAs each walk a
# contiguous run of 128 x 128 output tiles.  These sizes give every CTA several
# tiles, so the operand ring, the accumulator ring, the norm ring and the
# staging buffers all wrap, and a CTA's run crosses tile rows.
@pytest.mark.parametrize("m,n,k", [(4096, 4096, 64), (4000, 5000, 64), (2048, 2304, 160),
                                   (2176, 2048, 40), (16384, 16384, 64)])
def test_pairwise_distance_many_tiles_per_cta(queue, m, n, k):
    from numba_mlir_b200 import contraction
    from oracle import configs as O

    rng = np.random.default_rng(m + n + k)
    x = rng.uniform(0, 1, (m, k)).astype(np.float32)
    y = rng.uniform(0, 1, (n, k)).astype(np.float32)
    got = contraction.pairwise_distance(_dev(x), _dev(y)).copy_to_host()
    queue.check_status()
    want = np.zeros((m, n), np.float32)
    O.pairwise(x, y, want)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 64), (3000, 2500, 72), (2048, 2048, 200)])
def test_gemm_many_tiles_per_cta(queue, m, n, k):
    from numba_mlir_b200 import contraction, zeros

    rng = np.random.default_rng(m * 3 + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c = zeros((m, n), np.float32)
    contraction.gemm(_dev(a), _dev(b), c)
    queue.check_status()
    truth = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.all(np.abs(c.copy_to_host() - truth) <= 1e-5 * scale)


def test_pairwise_distance_repeated_calls_reuse_the_pack_buffers(queue):
    """Two different problems back to back on one queue (the second call's
    prepass overwrites the operand images while nothing of the first is left
    in flight) give the same answers as each alone."""
    from numba_mlir_b200 import contraction
    from oracle import configs as O

    rng = np.random.default_rng(11)
    for m, n in ((4096, 2048), (2048, 4096), (4096, 2048)):
        x = rng.uniform(0, 1, (m, 64)).astype(np.float32)
        y = rng.uniform(0, 1, (n, 64)).astype(np.float32)
        got = contraction.pairwise_distance(_dev(x), _dev(y)).copy_to_host()
        want = np.zeros((m, n), np.float32)
        O.pairwise(x, y, want)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    queue.check_status()


# ------------------------------------------------- the benchmark's configs ---
def test_config2_black_scholes_full_size(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    price, strike, t, rate, vol = O.make_inputs("black_scholes")
    n = price.size
    assert n == 1 << 24
    call, put = nm.empty(n, np.float32), nm.empty(n, np.float32)
    workloads.black_scholes(_dev(price), _dev(strike), _dev(t), rate, vol, call, put)
    queue.check_status()
    ocall, oput = np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.black_scholes(price, strike, t, rate, vol, ocall, oput)
    np.testing.assert_allclose(call.copy_to_host(), ocall, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(put.copy_to_host(), oput, rtol=1e-5, atol=2e-5)
    # no further from the float64 truth than twice the CPU oracle's own error
    tcall, tput = O.black_scholes_f64(price, strike, t, rate, vol)
    for got, ora, truth in ((call.copy_to_host(), ocall, tcall), (put.copy_to_host(), oput, tput)):
        assert np.abs(got - truth).max() <= 2 * np.abs(ora - truth).max() + 1e-6


def test_config2_black_scholes_fastmath_full_size(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    price, strike, t, rate, vol = O.make_inputs("black_scholes")
    n = price.size
    call, put = nm.empty(n, np.float32), nm.empty(n, np.float32)
    workloads.black_scholes_fastmath(_dev(price), _dev(strike), _dev(t), rate, vol, call, put)
    queue.check_status()
    tcall, tput = O.black_scholes_f64(price, strike, t, rate, vol)
    np.testing.assert_allclose(call.copy_to_host(), tcall, rtol=1e-5, atol=4e-5)
    np.testing.assert_allclose(put.copy_to_host(), tput, rtol=1e-5, atol=4e-5)


def test_config3_axis_reductions_full_size(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    (a,) = O.make_inputs("reduce_f32")
    assert a.shape == (16384, 4096)
    da = _dev(a)
    s1 = nm.empty(a.shape[0], np.float32)
    workloads.sum_axis1(da, s1)
    truth = a.astype(np.float64).sum(axis=1)
    scale = np.abs(a).astype(np.float64).sum(axis=1)
    assert np.all(np.abs(s1.copy_to_host().astype(np.float64) - truth) <= 1e-5 * scale)
    m0 = nm.empty(a.shape[1], np.float32)
    workloads.min_axis0(da, m0)
    assert np.array_equal(m0.copy_to_host().view(np.uint32), O.min_axis0(a).view(np.uint32))
    am = nm.empty(a.shape[0], np.int64)
    workloads.argmin_axis1(da, am)
    assert np.array_equal(am.copy_to_host(), O.argmin_axis1(a))
    queue.check_status()


def test_config3_int_sum_full_size(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    (a,) = O.make_inputs("reduce_i32")
    assert a.size == 1 << 28
    out = nm.empty((), np.int64)
    workloads.total(_dev(a), out)
    queue.check_status()
    assert int(out.copy_to_host()) == int(O.int_sum(a)) == int(a.sum(dtype=np.int64))


def test_config5_kmeans_device_resident_lloyd_loop(queue):
    """Ten Lloyd iterations exactly as the benchmark runs them: the @kernel
    assignment + accumulation and the njit centroid update both on the device,
    centroids never leaving it.  Labels bit-exact, centroids bit-equal."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    pts, c0 = O.make_inputs("kmeans")
    assert pts.shape == (1 << 22, 16)
    d_pts, cent = _dev(pts), _dev(c0)
    labels = nm.empty(pts.shape[0], np.int32)
    sums, counts = nm.zeros(c0.shape, np.float64), nm.zeros(c0.shape[0], np.int64)
    for _ in range(10):
        queue.memset(sums.ptr, 0, sums.nbytes)
        queue.memset(counts.ptr, 0, counts.nbytes)
        workloads.kmeans_step(d_pts, cent, labels, sums, counts)
        workloads.kmeans_update(cent, sums, counts)
    queue.check_status()
    want_labels, want_cent = O.kmeans(pts, c0, 10)
    assert np.array_equal(labels.copy_to_host(), want_labels)
    assert np.array_equal(cent.copy_to_host().view(np.uint32), want_cent.view(np.uint32))


def test_kmeans_update_keeps_empty_clusters(queue):
    """The njit centroid update against the oracle's, with empty clusters."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    rng = np.random.default_rng(5)
    cent = rng.uniform(-10, 10, (64, 16)).astype(np.float32)
    counts = rng.integers(0, 3, 64).astype(np.int64) * rng.integers(1, 100000, 64)
    assert (counts == 0).any() and (counts > 0).any()
    sums = rng.standard_normal((64, 16)) * counts[:, None]
    d_cent = _dev(cent)
    workloads.kmeans_update(d_cent, _dev(sums), _dev(counts))
    want = O.kmeans_update(cent, sums, counts)
    assert np.array_equal(d_cent.copy_to_host().view(np.uint32), want.view(np.uint32))
    del nm
