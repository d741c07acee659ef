"""Parity of the tcgen05 contraction (gemm entry + fused pairwise distance),
through the C-ABI symbols _mlir_ciface_mkl_gemm_float32_device and
_mlir_ciface_nmb_pairwise_distance_float32_device."""

import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 64), (300, 200, 64), (128, 128, 8), (77, 513, 13),
                                   (129, 127, 3), (256, 130, 100), (64, 64, 160), (1, 1, 64)])
def test_pairwise_distance_matches_oracle(queue, m, n, k):
    """Config 4 data (uniform[0,1]) at reduced and ragged sizes; 1e-5 relative
    against the reference's direct loop (mlir/tests/test_gpu.py:2228-2239) run
    by the CPU oracle, which accumulates float32 differences in float64."""
    from numba_mlir_b200 import contraction
    from oracle import configs as O

    rng = np.random.default_rng(0)
    x = rng.uniform(0, 1, (m, k)).astype(np.float32)
    y = rng.uniform(0, 1, (n, k)).astype(np.float32)
    got = contraction.pairwise_distance(_dev(x), _dev(y)).copy_to_host()
    want = np.zeros((m, n), np.float32)
    O.pairwise(x, y, want)
    queue.check_status()
    if k >= 8:
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    # The norm expansion cancels for near-coincident points (they exist in low
    # dimension): the squared distance is good to a few float32 ulps of the
    # norms it is a difference of.
    xx = (x.astype(np.float64) ** 2).sum(1)[:, None]
    yy = (y.astype(np.float64) ** 2).sum(1)[None, :]
    assert np.all(np.abs(got.astype(np.float64) ** 2 - want.astype(np.float64) ** 2)
                  <= 4e-6 * (xx + yy) + 1e-9)


def test_pairwise_distance_views_and_output_stride(queue):
    from numba_mlir_b200 import contraction, empty
    from oracle import configs as O

    rng = np.random.default_rng(1)
    x = rng.uniform(0, 1, (200, 64)).astype(np.float32)
    y = rng.uniform(0, 1, (64, 150)).astype(np.float32)  # used transposed: (150, 64)
    out = empty((200, 256), np.float32)
    view = out[:, 3:153]  # row stride 256, unaligned start: scalar store path
    contraction.pairwise_distance(_dev(x), _dev(y).T, view)
    want = np.zeros((200, 150), np.float32)
    O.pairwise(x, np.ascontiguousarray(y.T), want)
    queue.check_status()
    np.testing.assert_allclose(out.copy_to_host()[:, 3:153], want, rtol=1e-5, atol=1e-6)


def test_gemm_reference_dot_case(queue):
    # mlir/tests/test_gpu.py:2101-2138 (test_cfd_dot): exact on small integers
    from numba_mlir_b200 import contraction, zeros

    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    c = zeros((2, 2), np.float32)
    contraction.gemm(_dev(a), _dev(b), c)
    assert np.array_equal(c.copy_to_host(), np.dot(a, b))


_sq = [np.zeros((4, 4), np.float32), np.ones((4, 4), np.float32),
       np.arange(16).reshape(4, 4).astype(np.float32)]
_rect = [np.zeros((4, 6), np.float32), np.ones((4, 6), np.float32),
         np.arange(24).reshape(4, 6).astype(np.float32)]


@pytest.mark.parametrize("alpha,beta", list(itertools.product([0, 1, 0.5], [0, 1, 0.5])))
def test_gemm_alpha_beta_matrix(queue, alpha, beta):
    # mlir/tests/test_gpu.py:2141-2193 (test_internal_gemm), exact equality
    from numba_mlir_b200 import contraction

    cases = list(itertools.product(_sq, _sq, _sq)) + [(a, b.T, c) for a, b, c in
                                                      itertools.product(_rect, _rect, _sq)]
    for a, b, c in cases:
        dc = _dev(c.copy())
        db = _dev(np.ascontiguousarray(b.T)).T if not b.flags.c_contiguous else _dev(b)
        contraction.gemm(_dev(a), db, dc, alpha, beta)
        want = alpha * np.dot(a, b) + beta * c
        assert np.array_equal(dc.copy_to_host(), want.astype(np.float32)), (alpha, beta)
    queue.check_status()


@pytest.mark.parametrize("m,n,k", [(256, 384, 64), (100, 50, 200), (513, 129, 31)])
def test_gemm_random_fp32_accuracy(queue, m, n, k):
    """3xTF32 keeps fp32-level accuracy: 1e-5 relative to sum(|a_ik b_kj|)."""
    from numba_mlir_b200 import contraction, zeros

    rng = np.random.default_rng(2)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c = zeros((m, n), np.float32)
    contraction.gemm(_dev(a), _dev(b), c)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    queue.check_status()
    assert np.all(np.abs(c.copy_to_host() - truth) <= 1e-5 * scale)


def test_gemm_column_major_output_and_errors(queue):
    from numba_mlir_b200 import contraction, runtime, zeros

    rng = np.random.default_rng(3)
    a = rng.integers(-8, 8, (40, 24)).astype(np.float32)
    b = rng.integers(-8, 8, (24, 56)).astype(np.float32)
    ct = zeros((56, 40), np.float32)  # C^T storage: C is column-major
    contraction.gemm(_dev(a), _dev(b), ct.T)
    assert np.array_equal(ct.copy_to_host().T, a @ b)
    with pytest.raises(runtime.GpuRuntimeError, match="shape mismatch"):
        contraction.gemm(_dev(a), _dev(a), zeros((40, 40), np.float32))


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (65, 33, 17), (200, 300, 129), (64, 64, 16), (7, 513, 1000),
                                   (2500, 2300, 70)])  # the last one takes the 128 x 128 tiles
def test_gemm_float64_matches_numpy(queue, m, n, k):
    """The float64 entry the reference registers beside the float32 one
    (mlir/math_runtime.py:36-40): sums in index order with fused multiply-adds,
    compared with NumPy's float64 product; operands with any strides; alpha,
    beta; np.dot and @ on float64 device arrays reach it."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import contraction

    rng = np.random.default_rng(m * 1000 + n + k)
    a = rng.standard_normal((m, k))
    b = rng.standard_normal((k, n))
    c0 = rng.standard_normal((m, n))
    scale = np.abs(a) @ np.abs(b) + 1.0

    c = _dev(c0.copy())
    contraction.gemm(_dev(a), _dev(b), c)
    assert np.all(np.abs(c.copy_to_host() - a @ b) <= 1e-14 * k * scale)

    # transposed views (no copies) and alpha / beta
    at, bt = _dev(np.ascontiguousarray(a.T)).T, _dev(np.ascontiguousarray(b.T)).T
    c = _dev(c0.copy())
    contraction.gemm(at, bt, c, alpha=-0.5, beta=2.0)
    assert np.all(np.abs(c.copy_to_host() - (-0.5 * (a @ b) + 2.0 * c0)) <= 1e-14 * k * (scale + np.abs(c0)))

    got = nm.njit(lambda x, y: np.dot(x, y) + 1.0)(_dev(a), _dev(b))
    assert got.dtype == np.float64
    assert np.all(np.abs(got.copy_to_host() - (a @ b + 1.0)) <= 1e-14 * k * scale)
    got = nm.njit(lambda x, y: x @ y)(_dev(a), _dev(b))
    assert np.all(np.abs(got.copy_to_host() - a @ b) <= 1e-14 * k * scale)


def test_gemm_float64_rejects_mixed_types_and_bad_shapes(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import contraction, runtime

    a = _dev(np.ones((4, 3)))
    b32 = _dev(np.ones((3, 5), np.float32))
    with pytest.raises(TypeError):
        contraction.gemm(a, b32, _dev(np.zeros((4, 5))))
    with pytest.raises(TypeError):
        nm.njit(lambda x, y: np.dot(x, y))(a, b32)
    with pytest.raises(runtime.GpuRuntimeError, match="shape mismatch"):
        contraction.gemm(a, _dev(np.ones((4, 5))), _dev(np.zeros((4, 5))))
