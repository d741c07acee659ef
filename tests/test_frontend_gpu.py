"""The decorator surface on the GPU: `njit` array expressions (fused ufunc
chains, broadcasting, reductions, dot), `vectorize`, and plan replay, checked
against the CPU oracle / NumPy."""

import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a):
    from numba_mlir_b200 import from_host

    return from_host(a)


def _host(x):
    """Host value of a result that may be a device array or already a scalar."""
    return x.copy_to_host() if hasattr(x, "copy_to_host") else x


def test_config1_broadcast_add_through_njit(queue):
    import numba_mlir_b200 as nm
    from oracle import configs as O

    @nm.njit(parallel=True)
    def add(a, b):
        return a + b

    a, b = O.make_inputs("bcast_add")
    got = add(_dev(a), _dev(b))
    assert isinstance(got, nm.DeviceArray) and got.dtype == np.float32
    want = O.bcast_add(a, b)
    assert np.array_equal(got.copy_to_host().view(np.uint32), want.view(np.uint32))
    # second call replays the recorded plan on new data
    a2 = a[::-1].copy()
    assert np.array_equal(add(_dev(a2), _dev(b)).copy_to_host(), a2 + b)
    assert len(add._plans) == 1


def _black_scholes_body():
    import numba_mlir_b200 as nm

    @nm.vectorize(nopython=True)
    def _nberf(x):
        return math.erf(x)

    # numba_mlir/mlir/tests/test_numpy.py:2827-2852 with float32 constants
    def black_scholes(price, strike, t, rate, volatility, call, put):
        mr = -rate
        sig_sig_two = volatility * volatility * np.float32(2)
        P = price
        S = strike
        T = t
        a = np.log(P / S)
        b = T * mr
        z = T * sig_sig_two
        c = np.float32(0.25) * z
        y = np.float32(1.0) / np.sqrt(z)
        w1 = (a - b + c) * y
        w2 = (a - b - c) * y
        d1 = np.float32(0.5) + np.float32(0.5) * _nberf(w1)
        d2 = np.float32(0.5) + np.float32(0.5) * _nberf(w2)
        Se = np.exp(b) * S
        r = P * d1 - Se * d2
        call[:] = r
        put[:] = r - P + Se

    return nm.njit(parallel=True)(black_scholes)


@pytest.mark.parametrize("n", [524288, 1000003])
def test_config2_black_scholes_fuses_into_one_kernel(queue, n):
    """One launch for the whole chain (the reference asserts one scf.parallel,
    mlir/tests/test_numpy.py:2865-2866); same tolerance as the builtin kernel."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime
    from oracle import configs as O

    bs = _black_scholes_body()
    price, strike, t, rate, vol = O.make_inputs("black_scholes", n / 2**24, seed=777777)
    price, strike, t = price[:n], strike[:n], t[:n]
    call, put = nm.empty(n), nm.empty(n)
    args = (_dev(price), _dev(strike), _dev(t), rate, vol, call, put)
    bs(*args)
    before = runtime.launch_count()
    bs(*args)  # replay
    assert runtime.launch_count() - before == 1
    ocall, oput = np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.black_scholes(price, strike, t, rate, vol, ocall, oput)
    np.testing.assert_allclose(call.copy_to_host(), ocall, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(put.copy_to_host(), oput, rtol=1e-5, atol=2e-5)
    # scalar arguments are kernel parameters: a new rate needs no new plan
    bs(_dev(price), _dev(strike), _dev(t), np.float32(0.05), vol, call, put)
    O.black_scholes(price, strike, t, np.float32(0.05), vol, ocall, oput)
    np.testing.assert_allclose(call.copy_to_host(), ocall, rtol=1e-5, atol=2e-5)
    assert len(bs._plans) == 1


def _ulps(got, want64):
    want = want64.astype(np.float32)
    return np.abs(got.astype(np.float64) - want64) / np.spacing(np.abs(want)).astype(np.float64)


def test_fastmath_division_and_sqrt_stay_within_two_ulp(queue):
    """fastmath=True (numba_mlir/mlir/tests/test_gpu.py:981-1010,1900-1934):
    division, sqrt and 1/sqrt take the approximate instructions, whose error
    stays within 2 ulp of the exact float32 result; the default is bit-exact."""
    import numba_mlir_b200 as nm

    def f(a, b):
        return a / b, np.sqrt(a), np.float32(1.0) / np.sqrt(a)

    rng = np.random.default_rng(11)
    a = np.exp(rng.uniform(-60, 60, 1 << 18)).astype(np.float32)
    b = (np.exp(rng.uniform(-40, 40, 1 << 18)) * rng.choice([-1.0, 1.0], 1 << 18)).astype(np.float32)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    truth = (a64 / b64, np.sqrt(a64), 1.0 / np.sqrt(a64))
    exact = nm.njit(f)(_dev(a), _dev(b))
    with np.errstate(over="ignore"):
        want = (a / b, np.sqrt(a), np.float32(1.0) / np.sqrt(a))
    for got, w in zip(exact, want):
        assert np.array_equal(got.copy_to_host(), w)
    fast = nm.njit(f, fastmath=True)(_dev(a), _dev(b))
    for got, t in zip(fast, truth):
        g = got.copy_to_host()
        with np.errstate(over="ignore"):
            ok = np.isfinite(t.astype(np.float32)) & (np.abs(t) > 1e-37)
        assert _ulps(g[ok], t[ok]).max() <= 2.0


@pytest.mark.parametrize("n", [524288, 1000003])
def test_black_scholes_fastmath_matches_oracle(queue, n):
    """The benchmark-driver flags (numba_mlir/mlir/benchmarking.py:43) on the
    chain of mlir/tests/test_numpy.py:2827-2852: one kernel, same tolerance
    against the oracle as the default build and well inside the reference's
    own atol of 1e-3 (test_numpy.py:2861-2862)."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime, workloads
    from oracle import configs as O

    price, strike, t, rate, vol = O.make_inputs("black_scholes", n / 2**24, seed=777777)
    price, strike, t = price[:n], strike[:n], t[:n]
    call, put = nm.empty(n), nm.empty(n)
    args = (_dev(price), _dev(strike), _dev(t), rate, vol, call, put)
    workloads.black_scholes_fastmath(*args)
    before = runtime.launch_count()
    workloads.black_scholes_fastmath(*args)
    assert runtime.launch_count() - before == 1
    ocall, oput = np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.black_scholes(price, strike, t, rate, vol, ocall, oput)
    np.testing.assert_allclose(call.copy_to_host(), ocall, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(put.copy_to_host(), oput, rtol=1e-5, atol=2e-5)
    c64, p64 = O.black_scholes_f64(price, strike, t, rate, vol)
    for got, orc, truth in ((call.copy_to_host(), ocall, c64), (put.copy_to_host(), oput, p64)):
        assert np.abs(got - truth).max() <= 2 * np.abs(orc - truth).max() + 1e-6


def test_config3_reductions_through_njit(queue):
    import numba_mlir_b200 as nm
    from oracle import configs as O

    @nm.njit(parallel=True)
    def red(a):
        return np.sum(a, axis=1), np.min(a, axis=0), np.argmin(a, axis=1)

    @nm.njit(parallel=True)
    def isum(a):
        return a.sum()

    (a,) = O.make_inputs("reduce_f32", 1 / 16)
    s, m, am = red(_dev(a))
    truth = a.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(s.copy_to_host() - truth) <= 1e-5 * np.abs(a).astype(np.float64).sum(axis=1))
    assert np.array_equal(m.copy_to_host(), O.min_axis0(a))
    assert np.array_equal(am.copy_to_host(), O.argmin_axis1(a))
    (ai,) = O.make_inputs("reduce_i32", 1 / 64)
    r = isum(_dev(ai))
    assert r.dtype == np.int64 and int(r.copy_to_host()) == int(O.int_sum(ai))


_bcast_arrays = [np.array([1]), np.array([[1]]), np.array([[1, 2], [3, 4]]), np.array([5, 6]),
                 np.array([[5], [6]]), np.array([[5, 6]])]


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
def test_reference_broadcast_matrix(queue, dtype):
    # mlir/tests/test_numpy.py:483-514 (test_broadcast)
    import numba_mlir_b200 as nm

    @nm.njit
    def add(a, b):
        return np.add(a, b)

    for a in _bcast_arrays:
        for b in _bcast_arrays:
            a_, b_ = a.astype(dtype), b.astype(dtype)
            got = add(_dev(a_), _dev(b_)).copy_to_host()
            want = np.add(a_, b_)
            assert got.shape == want.shape and got.dtype == want.dtype
            assert np.array_equal(got, want)
        assert np.array_equal(add(_dev(a.astype(dtype)), 1).copy_to_host(), a.astype(dtype) + 1)


@pytest.mark.parametrize("shapes", [((1, 1), (1, 7), (7, 1)), ((7, 7), (1, 7), (7, 7)),
                                    ((7, 1), (7, 7), (1, 1)), ((2, 3, 4), (2, 1, 4), (3, 4))])
def test_reference_broadcast_fusion(queue, shapes):
    # mlir/tests/test_numpy.py:1270-1293 (a + b * c is one loop)
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime

    @nm.njit
    def f(a, b, c):
        return a + b * c

    arrs = [np.arange(math.prod(s)).reshape(s) for s in shapes]
    before = runtime.launch_count()
    got = f(*[_dev(x) for x in arrs]).copy_to_host()
    assert runtime.launch_count() - before == 1
    assert np.array_equal(got, arrs[0] + arrs[1] * arrs[2])


def test_numba_typing_of_python_scalars(queue):
    """A Python float is float64 under Numba's rules, so float32 * 0.5 is
    computed and returned in float64, exactly as the CPU oracle does."""
    import numba
    import numba_mlir_b200 as nm

    def f(a):
        return a * 0.5 + 1

    a = np.linspace(-3, 3, 1000).astype(np.float32)
    got = nm.njit(f)(_dev(a)).copy_to_host()
    want = numba.njit(f)(a)
    assert got.dtype == want.dtype == np.float64
    assert np.array_equal(got, want)


def test_unary_math_against_oracle_within_2ulp(queue):
    """log, exp, sqrt, erf on float32: <= 2 ulp from the CPU oracle (libm via
    Numba); the reference tolerates rtol 1e-5 (mlir/tests/test_gpu.py:501-548)."""
    import numba
    import numba_mlir_b200 as nm

    @nm.vectorize
    def gerf(x):
        return math.erf(x)

    @numba.vectorize(nopython=True)
    def cerf(x):
        return math.erf(x)

    rng = np.random.default_rng(0)
    cases = {
        "log": (lambda a: np.log(a), rng.uniform(0.01, 100, 200000)),
        "exp": (lambda a: np.exp(a), rng.uniform(-20, 20, 200000)),
        "sqrt": (lambda a: np.sqrt(a), rng.uniform(0, 1000, 200000)),
    }

    def ulps(x, y):
        xi = x.view(np.int32).astype(np.int64)
        yi = y.view(np.int32).astype(np.int64)
        xi = np.where(xi < 0, -(xi & 0x7FFFFFFF), xi)
        yi = np.where(yi < 0, -(yi & 0x7FFFFFFF), yi)
        return np.abs(xi - yi).max()

    for name, (fn, x) in cases.items():
        x = x.astype(np.float32)
        got = nm.njit(fn)(_dev(x)).copy_to_host()
        want = numba.njit(parallel=True)(fn)(x)
        assert got.dtype == np.float32
        assert ulps(got, want) <= 2, name
    x = rng.uniform(-4, 4, 200000).astype(np.float32)
    got = nm.njit(lambda a: gerf(a))(_dev(x)).copy_to_host()
    assert ulps(got, cerf(x)) <= 2


def test_erf_float32_within_2ulp_of_the_true_value(queue):
    """The library's own erf: every float32 in [2^-7, 4.5) at stride 3 (both
    ranges, the switch at 1 and the saturation at 3.92), a logarithmic sweep
    below, and the special values, against float64 erf rounded to float32."""
    import numba_mlir_b200 as nm

    @nm.vectorize
    def gerf(x):
        return math.erf(x)

    lo, hi = np.float32(2.0**-7).view(np.int32), np.float32(4.5).view(np.int32)
    pos = np.arange(lo, hi, 3, dtype=np.int32).view(np.float32)
    tiny = np.logspace(-44, -2, 100000).astype(np.float32)
    x = np.concatenate([pos, -pos[::7], tiny, -tiny[::3],
                        np.array([0.0, -0.0, 1.0, -1.0, 0.99999994, 1.0000001, 3.9, 3.92, 4.0, 4.0000005,
                                  10.0, -10.0, 1e30, np.inf, -np.inf], np.float32)])
    got = nm.njit(lambda a: gerf(a))(_dev(x)).copy_to_host()
    from scipy import special

    truth = special.erf(x.astype(np.float64))
    want = truth.astype(np.float32)
    ulp = np.spacing(np.abs(want)).astype(np.float64)
    ok = np.isfinite(truth) & (want != 0)
    err = np.abs(got.astype(np.float64) - truth)[ok] / ulp[ok]
    assert err.max() <= 2.0, (err.max(), x[ok][err.argmax()])
    assert np.array_equal(np.signbit(got), np.signbit(x))
    assert got[x == 0].tolist() == [0.0, -0.0] and np.signbit(got[x == 0]).tolist() == [False, True]
    assert got[np.isinf(x)].tolist() == [1.0, -1.0]
    nan = nm.njit(lambda a: gerf(a))(_dev(np.array([np.nan], np.float32))).copy_to_host()
    assert np.isnan(nan[0])


@pytest.mark.parametrize("n", [1, 7, 1024, 4096 + 3, 1 << 20])
def test_paired_float32_arithmetic_is_bit_identical_to_numpy(queue, n):
    """The chain's float32 +, -, * run as f32x2 instructions over pairs of
    elements (and element by element at a ragged end): every result is the
    IEEE-rounded one NumPy computes, cancellation included."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    c = (a * np.float32(1.0001)).astype(np.float32)
    d = (b * np.float32(0.9999)).astype(np.float32)
    a[:1] = np.float32(1e-42)  # a subnormal operand and result
    s = np.float32(3.0)

    @nm.njit
    def f(a, b, c, d, s):
        return a * b - c * d, (a + b) * (c - d) + s * a, np.sqrt((a - c) * (a - c)) * (b + d)

    r0, r1, r2 = f(_dev(a), _dev(b), _dev(c), _dev(d), s)
    # products that feed a subtraction: every element differs if one is fused into it
    np.testing.assert_array_equal(r0.copy_to_host(), a * b - c * d)
    np.testing.assert_array_equal(r1.copy_to_host(), (a + b) * (c - d) + s * a)
    np.testing.assert_array_equal(r2.copy_to_host(), np.sqrt((a - c) * (a - c)) * (b + d))
    # a*b - float32(a*b) is exactly zero when the product rounds on its own
    ab = a * b

    @nm.njit
    def residual(a, b, ab):
        return a * b - ab

    assert not residual(_dev(a), _dev(b), _dev(ab)).copy_to_host().any()


def test_chains_with_division_and_square_root_match_numpy_bit_for_bit(queue):
    """Quotients, square roots and 1/sqrt of ordinary, tiny, huge, zero,
    subnormal, infinite, negative and NaN operands are the IEEE-rounded values
    NumPy computes, in the aligned (paired) and the unaligned (one element at a
    time) forms of the chain."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import from_host

    rng = np.random.default_rng(5)
    n = 1 << 16
    a = (rng.standard_normal(n) * 10.0 ** rng.integers(-30, 30, n)).astype(np.float32)
    b = (rng.standard_normal(n) * 10.0 ** rng.integers(-30, 30, n)).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-42, -1e-42, 3.4028235e38, 1.1754944e-38,
                        1.0, -1.0, 3.0, 2.0 ** -60, 2.0 ** 60, 2.0 ** -61, 2.0 ** 61, 2.0 ** 100, 2.0 ** -100,
                        2.0 ** 101, 2.0 ** -101], np.float32)
    k = special.size
    a[: k * k] = np.repeat(special, k)
    b[: k * k] = np.tile(special, k)
    # an in-range value next to each special one, and the other way round
    a[k * k: 2 * k * k: 2] = np.float32(1.5)
    f = nm.njit(lambda x, y: (x / y, np.sqrt(np.abs(x)), np.float32(1) / np.sqrt(np.abs(y)), np.float32(1) / x))
    with np.errstate(all="ignore"):
        want = (a / b, np.sqrt(np.abs(a)), np.float32(1) / np.sqrt(np.abs(b)), np.float32(1) / a)
        got = f(from_host(a), from_host(b))
        for g, w in zip(got, want):
            np.testing.assert_array_equal(g.copy_to_host(), w)
        pa = from_host(np.concatenate([np.zeros(1, np.float32), a]))[1:]
        pb = from_host(np.concatenate([np.zeros(1, np.float32), b]))[1:]
        for g, w in zip(f(pa, pb), want):
            np.testing.assert_array_equal(g.copy_to_host(), w)


def test_log_float32_within_1ulp_and_pair_forms_equal_scalar_forms(queue):
    """The library's own float32 log: every float32 of three binades around 1
    at stride 5, a logarithmic sweep over the whole range, subnormals and the
    special values, against float64 log rounded to float32 (1 ulp).  The
    two-values-at-once forms of log and erf (used where a chain runs over
    16-byte aligned data) give the very bits of the scalar forms (used for
    unaligned data and ragged ends)."""
    import numba_mlir_b200 as nm

    @nm.vectorize
    def gerf(x):
        return math.erf(x)

    lo, hi = np.float32(0.25).view(np.int32), np.float32(4.0).view(np.int32)
    near = np.arange(lo, hi, 5, dtype=np.int32).view(np.float32)
    sweep = np.logspace(-37.5, 38.4, 200001).astype(np.float32)
    sub = np.logspace(-45, -38, 5000).astype(np.float32)
    x = np.concatenate([near, sweep, sub, np.array([1.0, 0.99999994, 1.0000001, 0.70710677, 0.7071068, 1.4142135,
                                                    1.4142137, 3.4028235e38, 1.1754944e-38], np.float32)])
    if x.size % 2:
        x = x[:-1]
    flog = nm.njit(lambda a: np.log(a))
    got = flog(_dev(x)).copy_to_host()
    truth = np.log(x.astype(np.float64))
    want = truth.astype(np.float32)
    ulp = np.spacing(np.abs(want)).astype(np.float64)
    ok = want != 0
    err = np.abs(got.astype(np.float64) - truth)[ok] / ulp[ok]
    assert err.max() <= 1.0, (err.max(), x[ok][err.argmax()])
    special = np.array([0.0, -0.0, -1.0, np.inf, -np.inf, np.nan, 1.0], np.float32)
    with np.errstate(all="ignore"):
        np.testing.assert_array_equal(flog(_dev(special)).copy_to_host(), np.log(special))
    # unaligned views take the one-element forms: same bits
    pad = np.concatenate([np.zeros(1, np.float32), x])
    np.testing.assert_array_equal(flog(_dev(pad)[1:]).copy_to_host(), got)
    y = np.concatenate([np.linspace(-5, 5, 100001).astype(np.float32), np.float32([np.nan])])
    ferf = nm.njit(lambda a: gerf(a))
    pad = np.concatenate([np.zeros(1, np.float32), y])
    np.testing.assert_array_equal(ferf(_dev(pad)[1:]).copy_to_host(), ferf(_dev(y)).copy_to_host())


def test_where_compare_cast_and_strided_operands(queue):
    import numba_mlir_b200 as nm

    @nm.njit
    def f(a, b):
        return np.where(a > b, a - b, np.float32(0)) + np.abs(b)

    rng = np.random.default_rng(4)
    a = rng.standard_normal((64, 48)).astype(np.float32)
    b = rng.standard_normal((48, 64)).astype(np.float32)
    got = f(_dev(a), _dev(b).T).copy_to_host()
    want = np.where(a > b.T, a - b.T, np.float32(0)) + np.abs(b.T)
    assert np.array_equal(got, want)
    i = rng.integers(-5, 5, 1000).astype(np.int32)
    got = nm.njit(lambda x: (x * x).astype(np.float32) / np.float32(2))(_dev(i)).copy_to_host()
    assert np.array_equal(got, (i * i).astype(np.float32) / np.float32(2))


def test_stacking_flipping_outer_and_triangles(queue):
    """The array-building functions of the reference's NumPy table
    (numba_mlir/mlir/numpy/funcs.py: hstack, vstack, dstack, flip, outer,
    tril, triu, eye) against NumPy, on arrays and on expressions."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(9)
    a = rng.standard_normal((6, 8)).astype(np.float32)
    b = rng.standard_normal((6, 8)).astype(np.float32)
    v = rng.standard_normal(8).astype(np.float32)
    w = rng.standard_normal(5).astype(np.float32)
    cases = [
        (lambda a, b, v, w: np.vstack((a, b + 1)), None),
        (lambda a, b, v, w: np.hstack((a, b * 2)), None),
        (lambda a, b, v, w: np.dstack((a, b)), None),
        (lambda a, b, v, w: np.hstack((v, w)), None),
        (lambda a, b, v, w: np.vstack((v, v * 3)), None),
        (lambda a, b, v, w: np.dstack((v, v)), None),
        (lambda a, b, v, w: np.flip(a) + b, None),
        (lambda a, b, v, w: np.flip(a, axis=1) * 2, None),
        (lambda a, b, v, w: np.flip(a + b, axis=0), None),
        (lambda a, b, v, w: np.outer(v, w), None),
        (lambda a, b, v, w: np.outer(a, w + 1), None),
        (lambda a, b, v, w: np.tril(a), None),
        (lambda a, b, v, w: np.triu(a, 1) + np.tril(b, -2), None),
        (lambda a, b, v, w: np.tril(a + b, k=2), None),
        (lambda a, b, v, w: a * np.eye(6, 8, dtype=np.float32), None),
        (lambda a, b, v, w: np.eye(6, 8, 1) + a, None),
        (lambda a, b, v, w: v + np.arange(8, dtype=np.float32), None),
        (lambda a, b, v, w: np.arange(3, 19, 2) * v.astype(np.int64), None),
        (lambda a, b, v, w: np.arange(0.0, 0.8, 0.1) + v, None),
        (lambda a, b, v, w: a + np.arange(8).astype(np.float32), None),  # (float32 + int64 is float32 under Numba's typing)
        (lambda a, b, v, w: (np.arange(6).reshape(6, 1) * 10 + np.arange(8)) * (a > 0), None),
    ]
    for fn, _ in cases:
        got = nm.njit(fn)(_dev(a), _dev(b), _dev(v), _dev(w)).copy_to_host()
        want = fn(a, b, v, w)
        assert got.shape == want.shape and got.dtype == want.dtype
        np.testing.assert_array_equal(got, want)


def test_cov_uses_the_float64_product(queue):
    """np.cov (numba_mlir/mlir/numpy/funcs.py: numpy.cov): float64 whatever the
    input type, variables in rows or columns, bias and ddof, a single variable."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(21)
    m32 = rng.standard_normal((5, 200)).astype(np.float32)
    m64 = rng.standard_normal((3, 50))
    v = rng.standard_normal(300).astype(np.float32)
    cases = [
        (lambda m: np.cov(m), m32),
        (lambda m: np.cov(m), m64),
        (lambda m: np.cov(m, rowvar=False), m64.T.copy()),
        (lambda m: np.cov(m, bias=True), m32),
        (lambda m: np.cov(m, ddof=2) * 2.0, m64),
        (lambda m: np.cov(m), v),
    ]
    for fn, data in cases:
        got = nm.njit(fn)(_dev(data)).copy_to_host()
        want = fn(data)
        assert got.dtype == np.float64 and got.shape == np.shape(want)
        np.testing.assert_allclose(got, want, rtol=1e-10, atol=1e-12)


def test_arrays_created_inside_a_function(queue):
    """np.empty / zeros / ones / full with a shape inside an njit function are
    device arrays (numba_mlir/mlir/numpy/funcs.py: numpy.empty, zeros, ones);
    the function can fill them, return them, and is replayed from its plan."""
    import numba_mlir_b200 as nm

    def f(a, s):
        out = np.empty(a.shape, a.dtype)
        out[:] = a * s
        acc = np.zeros((a.shape[0], 1), np.float32)
        acc += out.sum(axis=1).reshape(-1, 1)
        return out + np.ones(a.shape, dtype=np.float32), acc, np.full(a.shape[1], 3, np.int32)

    g = nm.njit(f)
    rng = np.random.default_rng(17)
    for _ in range(3):
        a = rng.integers(-3, 4, (33, 20)).astype(np.float32)
        s = np.float32(rng.integers(1, 5))
        got = g(_dev(a), s)
        want = f(a, s)
        for x, y in zip(got, want):
            assert x.dtype == y.dtype and np.array_equal(x.copy_to_host(), y)
    assert len(g._plans) == 1


def test_layout_conversions_inside_a_function(queue):
    """np.asfortranarray (numba_mlir/mlir/numpy/funcs.py: numpy.asfortranarray),
    np.ascontiguousarray and np.asarray of traced arrays: same values, the
    requested order."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(23)
    a = rng.standard_normal((6, 8)).astype(np.float32)
    f = nm.njit(lambda x: np.asfortranarray(x))(_dev(a))
    assert f.shape == (6, 8) and f.strides == (4, 24)
    np.testing.assert_array_equal(f.copy_to_host(), a)
    g = nm.njit(lambda x: np.ascontiguousarray(x.T) + np.float32(1))(_dev(a))
    assert g.shape == (8, 6) and g.is_c_contiguous
    np.testing.assert_array_equal(g.copy_to_host(), a.T + np.float32(1))
    h = nm.njit(lambda x: np.asarray(x) * np.asfortranarray(x + np.float32(2)))(_dev(a))
    np.testing.assert_array_equal(h.copy_to_host(), a * (a + np.float32(2)))


def test_array_attributes_inside_a_function(queue):
    """array.size / itemsize / strides / shape / T / dtype and len() of traced
    arrays (the attributes numba_mlir/mlir/numpy/funcs.py registers) are the
    ones NumPy reports, for arguments, views and unevaluated expressions."""
    import numba_mlir_b200 as nm

    def f(a):
        v = a[1:, ::2]
        e = a + a
        return (a * np.float32(a.size + a.itemsize + a.strides[0] + len(a))
                + np.float32(v.strides[0] + v.strides[1] + v.size + e.strides[0] + e.T.shape[0] + e.nbytes))

    a = np.arange(48, dtype=np.float32).reshape(6, 8)
    got = nm.njit(f)(_dev(a))
    np.testing.assert_array_equal(got.copy_to_host(), f(a))


def test_out_arguments_and_atleast_2d(queue):
    """np.add(a, b, c), np.true_divide(a, b, out=c), np.clip(a, lo, hi, out)
    store into the given array, converted to its type, and return it
    (numba_mlir/mlir/tests/test_numpy.py: test_binary_inplace,
    test_ternary_inplace); np.atleast_2d gives the (1, n) view."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(31)
    a = rng.standard_normal((5, 8)).astype(np.float32)
    b = rng.standard_normal(8).astype(np.float32) + np.float32(3)

    def f(a, b, c, d, e):
        r = np.add(a, b, c)
        np.true_divide(a, b, out=d)
        np.clip(a, np.float32(-0.5), np.float32(0.5), e)
        np.maximum(r, d, out=r)
        return np.atleast_2d(b) * np.float32(2), np.atleast_2d(a)

    outs = [np.zeros((5, 8), np.float64), np.zeros((5, 8), np.float32), np.zeros((5, 8), np.float32)]
    want_outs = [o.copy() for o in outs]
    want = f(a, b, *want_outs)
    dev = [_dev(o) for o in outs]
    got = nm.njit(f)(_dev(a), _dev(b), *dev)
    for g, w in zip(dev, want_outs):
        np.testing.assert_array_equal(g.copy_to_host(), w)
    for g, w in zip(got, want):
        assert g.shape == w.shape
        np.testing.assert_array_equal(g.copy_to_host(), w)


@pytest.mark.parametrize("offset", [[], [0], [1, 2, 3], [3, 2, 1], [-1, 0, -4, 2]])
def test_indexing_with_an_index_array(queue, offset):
    """a[m] with an integer array m (numba_mlir/mlir/tests/test_numpy.py:
    test_getitem_offset), on arrays, views and expressions, for one- and
    two-dimensional sources; negative indices count from the end."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(len(offset))
    a = rng.standard_normal(9).astype(np.float32)
    b = rng.integers(-9, 9, (4, 6)).astype(np.int64)
    for dt in (np.int32, np.int64):
        m = np.array(offset, dt)
        for fn, args in ((lambda a, m: a[m], (a, m)),
                         (lambda a, m: a[::2][m] + (a * 2)[m], (a, m)),
                         (lambda a, m: a[::-1][m], (a, m)),
                         (lambda b, m: b[m], (b, m)),
                         (lambda b, m: b.T[m] + 1, (b, m))):
            got = nm.njit(fn)(*[_dev(x) for x in args])
            want = fn(*args)
            assert got.shape == want.shape and got.dtype == want.dtype
            np.testing.assert_array_equal(got.copy_to_host(), want)
    if offset:
        m2 = np.array([offset, offset[::-1]], np.int32)
        take = nm.njit(lambda a, m: a[m])
        got = take(_dev(a), _dev(m2))
        np.testing.assert_array_equal(got.copy_to_host(), a[m2])
        # the second call replays the recorded plan on new data
        a2, m3 = a[::-1].copy(), (m2 * 0 + 1).astype(np.int32)
        np.testing.assert_array_equal(take(_dev(a2), _dev(m3)).copy_to_host(), a2[m3])
        assert len(take._plans) == 1


def test_axis_views(queue):
    """np.expand_dims, squeeze, swapaxes, transpose with axes and broadcast_to
    are views (new axes, dropped axes, permuted or zero strides) that the
    chains read in place; the second call replays the recorded plan."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(12)
    v = rng.standard_normal(16).astype(np.float32)
    m = rng.standard_normal((4, 1)).astype(np.float32)
    t = rng.standard_normal((3, 4, 5)).astype(np.float32)
    one = rng.standard_normal((1, 16, 1)).astype(np.float32)
    cases = [
        (lambda a: np.expand_dims(a, 0) + np.expand_dims(a, -1), v),
        (lambda a: np.expand_dims(a + 1, (0, 2)) * 2, t[0]),
        (lambda a: np.squeeze(a) + 1, one),
        (lambda a: np.squeeze(a * 2, axis=0) + np.squeeze(a, axis=(0, 2))[:, None], one),
        (lambda a: np.broadcast_to(a, (4, 16)) + 1, v),
        (lambda a: np.broadcast_to(a, (3, 4, 5)) * 2, m),
        (lambda a: np.swapaxes(a, 0, 2) + 1, t),
        (lambda a: np.transpose(a, (1, 2, 0)) - np.transpose(a + 1, (1, 2, 0)), t),
        (lambda a: np.swapaxes(a, -1, 1).sum(axis=0), t),
    ]
    for fn, x in cases:
        f = nm.njit(fn)
        for data in (x, (x * 3).astype(x.dtype)):
            got, want = f(_dev(data)), fn(data)
            assert got.shape == want.shape and got.dtype == want.dtype
            np.testing.assert_allclose(got.copy_to_host(), want, rtol=1e-6)


@pytest.mark.parametrize("i", list(range(-2, 3)))
def test_scalar_arguments_and_computed_positions_as_indices(queue, i):
    """a[b] = 42; return a[b] with a scalar argument b (numba_mlir/mlir/tests/
    test_numpy.py: test_setitem1, test_setitem2), and a position computed on
    the device (a[np.argmax(a)]) as an index."""
    import numba_mlir_b200 as nm

    def f(a, b):
        a[b] = 42
        return a[b]

    def g(a, b, c):
        a[b, c] = 42
        return a[b, c]

    arr = np.asarray([1, 2, 3])
    d = _dev(arr.copy())
    host = arr.copy()
    assert int(np.asarray(_host(nm.njit(f)(d, i)))) == f(host, i)
    np.testing.assert_array_equal(d.copy_to_host(), host)
    arr2 = np.asarray([[1, 2, 3], [4, 5, 6]])
    d2 = _dev(arr2.copy())
    host2 = arr2.copy()
    assert int(np.asarray(_host(nm.njit(g)(d2, 1, i)))) == g(host2, 1, i)
    np.testing.assert_array_equal(d2.copy_to_host(), host2)
    rng = np.random.default_rng(i + 2)
    x = rng.standard_normal(1000).astype(np.float32)
    got = nm.njit(lambda a: a[np.argmax(a)] - a[np.argmin(a)])(_dev(x))
    assert np.float32(np.asarray(_host(got))) == x[np.argmax(x)] - x[np.argmin(x)]


@pytest.mark.parametrize("pattern", [[True], [False], [True, False], [False, True]])
def test_indexing_with_a_mask(queue, pattern):
    """a[m] with a boolean array of a's shape (numba_mlir/mlir/tests/
    test_numpy.py: test_getitem_mask): the selected elements in order, for
    sizes of one block, many blocks and more blocks than one scan step holds;
    masks computed inside the function; two-dimensional arrays."""
    import numba_mlir_b200 as nm

    f = nm.njit(lambda a, m: a[m])
    rng = np.random.default_rng(3)
    for n in (1, 7, 2048, 100003, 1300003):
        a = rng.standard_normal(n).astype(np.float32)
        m = np.resize(pattern, n)
        got = f(_dev(a), _dev(m))
        assert got.shape == a[m].shape
        np.testing.assert_array_equal(got.copy_to_host(), a[m])
    a = rng.standard_normal(300001)
    got = nm.njit(lambda a: a[a > 0.5] * 2)(_dev(a))
    np.testing.assert_array_equal(got.copy_to_host(), a[a > 0.5] * 2)
    b = rng.integers(-5, 5, (37, 53)).astype(np.int32)
    got = nm.njit(lambda b: b.T[b.T > 0])(_dev(b))
    np.testing.assert_array_equal(got.copy_to_host(), b.T[b.T > 0])
    empty = f(_dev(np.zeros(0, np.float32)), _dev(np.zeros(0, np.bool_)))
    assert empty.shape == (0,)


def test_dot_and_norm_expansion_distance(queue):
    """np.dot on device arrays reaches the tensor-core gemm (numpy/funcs.py:752-812);
    the distance matrix written with it matches the direct loop to 1e-5."""
    import numba_mlir_b200 as nm
    from oracle import configs as O

    @nm.njit(parallel=True)
    def dist(x, y):
        xx = np.sum(x * x, axis=1)
        yy = np.sum(y * y, axis=1)
        g = np.dot(x, y.T)
        return np.sqrt(np.maximum(xx.reshape(-1, 1) + yy.reshape(1, -1) - np.float32(2) * g, np.float32(0)))

    rng = np.random.default_rng(5)
    x = rng.uniform(0, 1, (256, 64)).astype(np.float32)
    y = rng.uniform(0, 1, (192, 64)).astype(np.float32)
    got = dist(_dev(x), _dev(y)).copy_to_host()
    want = np.zeros((256, 192), np.float32)
    O.pairwise(x, y, want)
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-6)


def test_no_device_argument_is_an_error_not_a_cpu_run(queue):
    import numba_mlir_b200 as nm

    with pytest.raises(TypeError, match="no CPU fallback"):
        nm.njit(lambda a: a + 1)(np.ones(4, np.float32))


def test_value_dependent_control_flow_still_works(queue):
    import numba_mlir_b200 as nm

    @nm.njit
    def f(a, flag):
        if flag > 0:
            return a + 1
        return a - 1

    a = np.arange(10, dtype=np.float32)
    assert np.array_equal(f(_dev(a), 1).copy_to_host(), a + 1)
    assert np.array_equal(f(_dev(a), -1).copy_to_host(), a - 1)


# --------------------------------------------- order of reads and writes ------
def test_store_after_an_unevaluated_read_keeps_the_old_values(queue):
    """NumPy semantics when an array is overwritten while an expression that
    reads it has not been evaluated yet (first call and plan replay)."""
    import numba_mlir_b200 as nm

    @nm.njit
    def g(a, o):
        b = a + np.float32(1)
        a[:] = np.float32(0)
        s = a.sum()
        o[:] = b
        return s

    for _ in range(2):
        a = np.arange(1000, dtype=np.float32)
        da, do = _dev(a), _dev(np.zeros_like(a))
        s = g(da, do)
        assert float(s.copy_to_host()) == 0.0
        assert np.array_equal(do.copy_to_host(), a + 1)
        assert not da.copy_to_host().any()


def test_overlapping_self_assignment_copies_like_numpy(queue):
    import numba_mlir_b200 as nm

    @nm.njit
    def shift(a):
        a[1:] = a[:-1]

    @nm.njit
    def rev(a):
        b = a[::-1] + np.float32(1)
        a[:] = np.float32(0)
        return b

    @nm.njit
    def flip_in_place(a):
        a[:] = a[::-1]

    @nm.njit
    def rows_down(m):
        m[1:, :] = m[:-1, :] * np.float32(2)

    for n in (5, 1000, 100003):
        a = np.arange(n, dtype=np.float32)
        da = _dev(a)
        shift(da)
        want = a.copy()
        want[1:] = a[:-1]
        assert np.array_equal(da.copy_to_host(), want)
        da = _dev(a)
        assert np.array_equal(rev(da).copy_to_host(), a[::-1] + 1)
        assert not da.copy_to_host().any()
        da = _dev(a)
        flip_in_place(da)
        assert np.array_equal(da.copy_to_host(), a[::-1])
    m = np.arange(37 * 64, dtype=np.float32).reshape(37, 64)
    dm = _dev(m)
    rows_down(dm)
    want = m.copy()
    want[1:, :] = m[:-1, :] * 2
    assert np.array_equal(dm.copy_to_host(), want)


def test_arguments_that_share_memory_get_their_own_plan(queue):
    """The same function called with disjoint and with overlapping views: the
    recorded plan of the first must not be replayed for the second."""
    import numba_mlir_b200 as nm

    @nm.njit
    def copy_to(dst, src):
        dst[:] = src + np.float32(1)

    a = np.arange(4096, dtype=np.float32)
    d1, d2 = _dev(a), _dev(a)
    copy_to(d1[1:], d2[:-1])
    want = a.copy()
    want[1:] = a[:-1] + 1
    assert np.array_equal(d1.copy_to_host(), want)
    d3 = _dev(a)
    copy_to(d3[1:], d3[:-1])
    assert np.array_equal(d3.copy_to_host(), want)
    assert len(copy_to._plans) == 2


def test_reduction_into_an_array_an_expression_still_reads(queue):
    import numba_mlir_b200 as nm

    @nm.njit
    def f(a, out, c):
        c[:] = out + np.float32(1)
        out[:] = np.sum(a, axis=1)

    rng = np.random.default_rng(9)
    a = rng.integers(-4, 5, (64, 128)).astype(np.float32)
    o = rng.integers(-4, 5, 64).astype(np.float32)
    for _ in range(2):
        do, dc = _dev(o), _dev(np.zeros_like(o))
        f(_dev(a), do, dc)
        assert np.array_equal(dc.copy_to_host(), o + 1)
        assert np.array_equal(do.copy_to_host(), a.sum(axis=1))


def test_plan_replays_on_the_queue_of_its_arguments(queue):
    """One njit function called with arrays of two queues of one device: the
    second call's kernels run on the second queue (its events order them)."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime

    @nm.njit
    def axpy(x, y, out):
        out[:] = x * np.float32(3) + y

    q2 = runtime.Queue(f"cuda:{queue.device}")
    rng = np.random.default_rng(10)
    x = rng.standard_normal(1 << 20).astype(np.float32)
    y = rng.standard_normal(1 << 20).astype(np.float32)
    out1 = nm.empty(x.size, np.float32, queue)
    axpy(nm.from_host(x, queue), nm.from_host(y, queue), out1)
    before = runtime.launch_count()
    out2 = nm.empty(x.size, np.float32, q2)
    axpy(nm.from_host(x, q2), nm.from_host(y, q2), out2)
    assert len(axpy._plans) == 1 and runtime.launch_count() == before + 1
    # synchronising the second queue alone is enough to read its result
    q2.synchronize()
    host = np.empty_like(x)
    q2.memcpy(host.ctypes.data, out2.ptr, host.nbytes, runtime.COPY_D2H, wait=True)
    assert np.array_equal(host, x * np.float32(3) + y)
    assert np.array_equal(out1.copy_to_host(), host)


def test_noncontiguous_device_copy(queue):
    a = np.arange(48, dtype=np.float32).reshape(6, 8)
    d = _dev(a)
    assert np.array_equal(d.T.copy().copy_to_host(), a.T)
    assert np.array_equal(d[::2, 1::3].copy_to_host(), a[::2, 1::3])


# ------------------------------------- producers fused into reductions --------
def _launches(fn, *args):
    from numba_mlir_b200 import runtime

    before = runtime.launch_count()
    out = fn(*args)
    return out, runtime.launch_count() - before


def test_reduction_of_an_elementwise_chain_is_one_pass(queue):
    """np.sqrt(np.square(a).sum(axis=1)) and friends read their inputs once:
    one reduction kernel over the chain (mlir/tests/test_gpu.py:2198-2224 is
    the reference's fused form), no temporary for the chain."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(12)
    a = rng.standard_normal((257, 1000)).astype(np.float32)
    b = rng.standard_normal((257, 1000)).astype(np.float32)
    da, db = _dev(a), _dev(b)

    norm = nm.njit(lambda x: np.sqrt(np.square(x).sum(axis=1)))
    norm(da)  # traced; the second call replays the plan
    got, n = _launches(norm, da)
    assert n == 1  # the reduction over the chain; the sqrt is applied to each row sum on its way out
    np.testing.assert_allclose(got.copy_to_host(), np.sqrt((a.astype(np.float64) ** 2).sum(1)), rtol=1e-5)

    rowsq = nm.njit(lambda x, out: out.__setitem__(slice(None), np.sum(x * x, axis=1)))
    out = nm.empty(257, np.float32)
    rowsq(da, out)
    _, n = _launches(rowsq, da, out)
    assert n == 1
    np.testing.assert_allclose(out.copy_to_host(), (a.astype(np.float64) ** 2).sum(1), rtol=1e-5)

    count = nm.njit(lambda x: (x > 0).sum())
    count(da)
    got, n = _launches(count, da)
    assert n == 1 and int(got.copy_to_host()) == int((a > 0).sum())

    mse = nm.njit(lambda x, y: np.mean((x - y) ** 2))
    mse(da, db)
    got, n = _launches(mse, da, db)
    assert n == 1  # the division by the element count rides on the reduction
    np.testing.assert_allclose(float(got.copy_to_host()), np.mean((a.astype(np.float64) - b) ** 2), rtol=1e-5)

    rms = nm.njit(lambda x, s: np.sqrt(np.sum(x, axis=1) * s + np.float32(1)))  # a plain array, a scalar argument
    rms(da, np.float32(0.0))
    got, n = _launches(rms, da, np.float32(0.0))
    assert n == 1 and np.array_equal(got.copy_to_host(), np.ones(257, np.float32))

    colmin = nm.njit(lambda x, y: np.min(x * y, axis=0))
    colmin(da, db)
    got, n = _launches(colmin, da, db)
    assert n == 1
    assert np.array_equal(got.copy_to_host(), (a * b).min(axis=0))

    # argmin / argmax of a chain along the last axis: one warp per row, first
    # occurrence on ties (quantised values make ties frequent)
    qa = np.round(a * 2).astype(np.float32)
    qb = np.round(b * 2).astype(np.float32)
    dqa, dqb = _dev(qa), _dev(qb)
    amin = nm.njit(lambda x, y: np.argmin(x * x - y, axis=1))
    amin(dqa, dqb)
    got, n = _launches(amin, dqa, dqb)
    assert n == 1 and got.dtype == np.int64
    assert np.array_equal(got.copy_to_host(), np.argmin(qa * qa - qb, axis=1))
    amax = nm.njit(lambda x, y: (np.abs(x) + y).argmax(axis=-1))
    amax(dqa, dqb)
    got, n = _launches(amax, dqa, dqb)
    assert n == 1 and np.array_equal(got.copy_to_host(), np.argmax(np.abs(qa) + qb, axis=1))
    ia = rng.integers(-50, 50, (300, 64)).astype(np.int32)
    imax = nm.njit(lambda x: np.argmax(x * x - 7, axis=1))
    got = imax(_dev(ia))
    assert np.array_equal(got.copy_to_host(), np.argmax(ia * ia - 7, axis=1))
    # three dimensions: rows are the leading axes flattened
    t3 = np.round(rng.standard_normal((5, 7, 32)) * 3).astype(np.float32)
    got = nm.njit(lambda x: np.argmin(x + 1, axis=2))(_dev(t3))
    assert got.shape == (5, 7) and np.array_equal(got.copy_to_host(), np.argmin(t3 + 1, axis=2))


@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (64, 63), (1000, 8), (5, 40000), (2, 3, 17), (1031,)])
@pytest.mark.parametrize("op", ["sum", "prod", "min", "max"])
def test_fused_reductions_match_numpy_on_every_axis(queue, shape, op):
    """reduce(f(a, b)) against NumPy for the row, column and full forms, ragged
    sizes, a broadcast operand, integer accumulation in int64."""
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(hash((shape, op)) % 2**32)
    fn = getattr(np, op)
    for dtype in (np.float32, np.int32):
        if dtype == np.int32:
            a = rng.integers(-3, 4, shape).astype(dtype)
            b = rng.integers(1, 3, shape[-1:]).astype(dtype)
        else:
            a = rng.uniform(0.5, 1.5, shape).astype(dtype)
            b = rng.uniform(0.9, 1.1, shape[-1:]).astype(dtype)
        if op == "prod":
            a = np.where(rng.random(shape) < 0.02, a, dtype(1)).astype(dtype)  # keep products in range
        for axis in [None] + list(range(len(shape))):
            got = nm.njit(lambda x, y: fn(x * y + dtype(1), axis=axis))(_dev(a), _dev(b)).copy_to_host()
            want = fn((a * b + dtype(1)).astype(np.int64 if dtype == np.int32 and op in ("sum", "prod") else dtype),
                      axis=axis)
            if dtype == np.int32 or op in ("min", "max"):
                assert np.array_equal(got, want), (shape, op, axis, dtype)
            else:
                np.testing.assert_allclose(got, want, rtol=2e-5)
    queue.check_status()


def test_fused_min_max_ignore_nans_like_the_library_reductions(queue):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import reduce_ops

    a = np.array([[3.0, np.nan, -1.0, 2.0], [np.nan, np.nan, 5.0, 4.0]], np.float32)
    da = _dev(a)
    for op in ("min", "max"):
        fused = nm.njit(lambda x: getattr(np, op)(x * np.float32(1), axis=1))(da).copy_to_host()
        plain = reduce_ops.reduce(da, op, 1).copy_to_host()
        assert np.array_equal(fused, plain)


def test_pairwise_distance_through_njit_is_one_contraction(queue):
    """Config 4 as a user writes it: np.dot inside njit with the norm
    expansion around it runs as the contraction's packing prepass plus one
    tensor-core launch (numpy/funcs.py:752-812 routes np.dot to the device
    gemm; the chain around it is the epilogue)."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import contraction, workloads
    from oracle import configs as O

    rng = np.random.default_rng(13)
    x = rng.uniform(0, 1, (1500, 64)).astype(np.float32)
    y = rng.uniform(0, 1, (700, 64)).astype(np.float32)
    dx, dy = _dev(x), _dev(y)
    d = nm.empty((1500, 700), np.float32)
    workloads.pairwise_distance(dx, dy, d)
    _, n = _launches(workloads.pairwise_distance, dx, dy, d)
    assert n == 2
    want = np.zeros((1500, 700), np.float32)
    O.pairwise(x, y, want)
    np.testing.assert_allclose(d.copy_to_host(), want, rtol=1e-5, atol=1e-6)
    assert np.array_equal(d.copy_to_host(), contraction.pairwise_distance(dx, dy).copy_to_host())


def test_product_with_bias_and_scale_epilogues(queue):
    import numba_mlir_b200 as nm

    rng = np.random.default_rng(14)
    a = rng.standard_normal((300, 40)).astype(np.float32)
    b = rng.standard_normal((40, 200)).astype(np.float32)
    bias = rng.standard_normal(200).astype(np.float32)
    rowb = rng.standard_normal((300, 1)).astype(np.float32)
    truth = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)

    f = nm.njit(lambda p, q, c: np.dot(p, q) + c)
    got, n = _launches(f, _dev(a), _dev(b), _dev(bias))
    assert np.all(np.abs(got.copy_to_host() - (truth + bias)) <= 1e-5 * (scale + np.abs(bias)))
    g = nm.njit(lambda p, q, r, c: r + c - np.float32(0.5) * np.dot(p, q))
    got = g(_dev(a), _dev(b), _dev(rowb), _dev(bias)).copy_to_host()
    assert np.all(np.abs(got - (rowb + bias - 0.5 * truth)) <= 1e-5 * (scale + np.abs(bias) + np.abs(rowb)))
    _, n = _launches(g, _dev(a), _dev(b), _dev(rowb), _dev(bias))
    assert n == 2  # prepass + contraction: the chain is the epilogue
    # a chain the epilogue does not cover still works (product, then a kernel)
    h = nm.njit(lambda p, q: np.exp(np.dot(p, q) * np.float32(0.01)))
    np.testing.assert_allclose(h(_dev(a), _dev(b)).copy_to_host(), np.exp(truth * 0.01), rtol=1e-4)
    queue.check_status()
