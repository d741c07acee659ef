"""Pins the CPU oracle before anything is judged against it (no GPU needed).

1. oracle/kernel_sim.py against golden vectors produced by the reference's own
   simulator (tests/golden/make_golden.py ran kernel_sim_impl.py of the
   reference; the .npz is committed).
2. oracle/configs.py against the known-answer form of the reference's tests:
   the same inputs, the plain NumPy/Python evaluation the reference compares
   its JIT output with.
"""

import math
import os

import numpy as np
import pytest

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "kernel_sim.npz"))


# ------------------------------------------------------------ kernel API ----
@pytest.mark.parametrize("dtype", ["int32", "int64", "float32"])
@pytest.mark.parametrize("opname", ["add", "sub"])
def test_sim_atomics_match_reference_simulator(dtype, opname):
    # mlir/tests/test_gpu.py:820-870
    from numba_mlir_b200.kernel import DEFAULT_LOCAL_SIZE, atomic, get_global_id
    from oracle.kernel_sim import kernel_sim

    atomic_op = getattr(atomic, opname)

    def func(a, b):
        i = get_global_id(0)
        atomic_op(b, 0, a[i])

    def func_off(a, b):
        i = get_global_id(0)
        atomic_op(b, i % 2, a[i])

    a = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9], dtype)
    res = np.zeros([1], dtype)
    kernel_sim(func)[a.shape, DEFAULT_LOCAL_SIZE](a, res)
    assert np.array_equal(res, GOLDEN[f"atomic_{opname}_{dtype}"])
    res = np.zeros([2], dtype)
    kernel_sim(func_off)[a.shape, DEFAULT_LOCAL_SIZE](a, res)
    assert np.array_equal(res, GOLDEN[f"atomic_{opname}_offset_{dtype}"])


@pytest.mark.parametrize("gsize,lsize", [(27, 7), (67, 17), (101, 33), (4, 2)])
def test_sim_ids_match_reference_simulator(gsize, lsize):
    from numba_mlir_b200.kernel import (get_global_id, get_global_size, get_group_id,
                                        get_local_id, get_local_size)
    from oracle.kernel_sim import kernel_sim

    def k_ids(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        gid[i] = i
        lid[i] = get_local_id(0)
        grp[i] = get_group_id(0)
        gsz[i] = get_global_size(0)
        lsz[i] = get_local_size(0)

    arrs = [np.full(gsize, -1, np.int64) for _ in range(5)]
    kernel_sim(k_ids)[gsize, lsize](*arrs)
    for name, arr in zip(("gid", "lid", "grp", "gsz", "lsz"), arrs):
        assert np.array_equal(arr, GOLDEN[f"ids_{gsize}_{lsize}_{name}"]), name


def test_sim_pairwise_matches_reference_simulator():
    # mlir/tests/test_gpu.py:1396-1430
    from numba_mlir_b200.kernel import get_global_id
    from oracle.kernel_sim import kernel_sim

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
    res = np.zeros((128, 128), np.float32)
    kernel_sim(func)[(128, 128), ()](a, b, res)
    assert np.array_equal(res, GOLDEN["pairwise1"])


# ------------------------------------------------------------- workloads ----
def test_black_scholes_oracle_vs_reference_known_answer():
    """mlir/tests/test_numpy.py:2796-2866: nopt = 524288, seed 777777, the JIT
    result must be within atol 1e-3 of the NumPy evaluation of the same body."""
    from scipy.special import erf

    from oracle import configs as O

    nopt, seed = 524288, 777777
    f32 = np.float32
    np.random.seed(seed)
    price = np.random.uniform(f32(10), f32(50), nopt).astype(f32)
    strike = np.random.uniform(f32(10), f32(50), nopt).astype(f32)
    t = np.random.uniform(f32(1), f32(2), nopt).astype(f32)
    rate, vol = f32(0.1), f32(0.2)

    # the reference test's py_func, evaluated by NumPy
    mr = -rate
    sig_sig_two = vol * vol * 2
    a = np.log(price / strike)
    b = t * mr
    z = t * sig_sig_two
    c = 0.25 * z
    y = 1.0 / np.sqrt(z)
    w1 = (a - b + c) * y
    w2 = (a - b - c) * y
    d1 = 0.5 + 0.5 * erf(w1)
    d2 = 0.5 + 0.5 * erf(w2)
    Se = np.exp(b) * strike
    r = price * d1 - Se * d2
    want_call, want_put = r, r - price + Se

    for fn in (O.black_scholes, O.black_scholes_ref_typing):
        call, put = np.zeros(nopt, f32), -np.ones(nopt, f32)
        fn(price, strike, t, rate, vol, call, put)
        np.testing.assert_allclose(call, want_call, atol=1e-3)
        np.testing.assert_allclose(put, want_put, atol=1e-3)
    c64, p64 = O.black_scholes_f64(price, strike, t, rate, vol)
    np.testing.assert_allclose(c64, want_call, atol=1e-3)


def test_pairwise_oracle_vs_reference_known_answer():
    # mlir/tests/test_gpu.py:2226-2266: 128 points x 3 dims, rtol 1e-5
    from oracle import configs as O

    a = np.arange(128 * 3, dtype=np.float32).reshape(128, 3)
    b = a + 5
    res = np.zeros((128, 128), np.float32)
    O.pairwise(a, b, res)
    np.testing.assert_allclose(res, GOLDEN["pairwise1"], rtol=1e-5)
    np.testing.assert_allclose(res, O.pairwise_f64(a, b), rtol=1e-5)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32])
def test_reduction_oracles_vs_reference_known_answers(dtype):
    # mlir/tests/test_gpu.py:2065-2098: a = arange(1, n+1).reshape(shape)
    from oracle import configs as O

    for shape in ((7, 16), (25, 64), (65, 65), (64, 25)):
        count = math.prod(shape)
        a = np.arange(1, count + 1, dtype=dtype).reshape(shape).copy()
        assert np.array_equal(O.min_axis0(a), a.min(axis=0))
        assert np.array_equal(O.argmin_axis1(a), a.argmin(axis=1))
        if dtype == np.float32:
            np.testing.assert_allclose(O.sum_axis1(a), a.sum(axis=1), rtol=1e-5)
            np.testing.assert_allclose(O.full_sum_f32(a), a.sum(), rtol=1e-5)
        else:
            assert O.int_sum(a.reshape(-1)) == a.sum(dtype=np.int64)


def test_argmin_oracle_first_occurrence():
    """No reference test pins argmin (xfail there); NumPy's first-minimum rule
    and the pair combiner of builtin/funcs.py:126-138 agree."""
    from oracle import configs as O

    a = np.ones((5, 9), np.float32)
    a[:, [2, 6]] = -1
    assert np.array_equal(O.argmin_axis1(a), np.full(5, 2))


def test_bcast_add_oracle_vs_numpy():
    # mlir/tests/test_numpy.py:483-514 semantics (NumPy broadcasting)
    from oracle import configs as O

    a, b = O.make_inputs("bcast_add", 1 / 16)
    assert np.array_equal(O.bcast_add(a, b), a + b)


def test_kmeans_oracle_assignment_vs_float64_argmin():
    """Labels agree with a float64 evaluation wherever the two nearest centres
    are not within float32 rounding of each other."""
    from oracle import configs as O

    pts, c0 = O.make_inputs("kmeans", 1 / 256)
    labels = np.zeros(pts.shape[0], np.int32)
    O.kmeans_assign(pts, c0, labels)
    d = ((pts[:, None, :].astype(np.float64) - c0[None].astype(np.float64)) ** 2).sum(-1)
    srt = np.sort(d, axis=1)
    clear = (srt[:, 1] - srt[:, 0]) > 1e-4 * srt[:, 0]
    assert clear.mean() > 0.99
    assert np.array_equal(labels[clear], d.argmin(axis=1)[clear])


def test_simulator_restatement_matches_the_reference_simulator_on_the_kernel_suite():
    """Every non-barrier case of tests/kernel_cases.py: oracle/kernel_sim.py gives
    what the reference's kernel_sim_impl.py gave (tests/golden/kernel_sim.npz)."""
    from kernel_cases import cases
    from oracle.kernel_sim import kernel_sim

    seen = 0
    for key, func, gsize, lsize, args, out_index, _exact in cases():
        run_args = [a.copy() if isinstance(a, np.ndarray) else a for a in args]
        kernel_sim(func)[gsize, lsize](*run_args)
        got, want = run_args[out_index], GOLDEN[key]
        assert got.dtype == want.dtype and np.array_equal(got, want, equal_nan=True), key
        seen += 1
    assert seen == 98
