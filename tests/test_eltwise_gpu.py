"""Parity of the fused elementwise kernels against the CPU oracle, through the
C-ABI (gpuxModuleLoad/KernelGet/LaunchKernel with a GPUParamDesc array)."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2048, 2048), (205, 2048), (1, 4), (7, 13), (65, 127), (3, 1024)])
def test_bcast_add_bit_exact(queue, shape):
    # Odd sizes are the reference's own choices (mlir/tests/test_gpu.py:570-577).
    from numba_mlir_b200 import builtin_ops, from_host
    from oracle import configs as O

    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, shape).astype(np.float32)
    b = rng.uniform(-1, 1, (1, shape[1])).astype(np.float32)
    out = builtin_ops.bcast_add_f32(from_host(a), from_host(b)).copy_to_host()
    want = O.bcast_add(a, b)
    assert out.dtype == np.float32
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))


def test_bcast_add_unaligned_view(queue):
    from numba_mlir_b200 import builtin_ops, from_host

    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (9, 64)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 64)).astype(np.float32)
    da = from_host(a)
    sub = da[1:]  # starts 256 bytes in: still aligned; shift by one row of 65
    out = builtin_ops.bcast_add_f32(sub, from_host(b)).copy_to_host()
    assert np.array_equal(out, a[1:] + b)


def _ulp_diff(x, y):
    """Distance in float32 units in the last place."""
    xi = x.view(np.int32).astype(np.int64)
    yi = y.view(np.int32).astype(np.int64)
    xi = np.where(xi < 0, -(xi & 0x7FFFFFFF), xi)
    yi = np.where(yi < 0, -(yi & 0x7FFFFFFF), yi)
    return np.abs(xi - yi)


@pytest.mark.parametrize("n", [1, 7, 1000, 524288, 524288 + 3])
def test_black_scholes_matches_oracle(queue, n):
    """Tolerance: the chain ends in P*d1 - Se*d2, a difference of terms up to
    ~50 in magnitude, so the comparison is absolute: 2e-5 (about 5 ulp of 50)
    plus 1e-5 relative -- 50x tighter than the reference's own atol=1e-3
    (mlir/tests/test_numpy.py:2862-2863); and the GPU result must be as close
    to the float64 truth as the CPU oracle is, within a factor of two."""
    from numba_mlir_b200 import builtin_ops, empty, from_host
    from oracle import configs as O

    price, strike, t, rate, vol = O.make_inputs("black_scholes", n / 2**24, seed=777777)
    price, strike, t = price[:n], strike[:n], t[:n]
    call, put = empty(n), empty(n)
    builtin_ops.black_scholes_f32(from_host(price), from_host(strike), from_host(t), rate, vol, call, put)
    call, put = call.copy_to_host(), put.copy_to_host()
    ocall, oput = np.zeros(n, np.float32), np.zeros(n, np.float32)
    O.black_scholes(price, strike, t, rate, vol, ocall, oput)
    np.testing.assert_allclose(call, ocall, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(put, oput, rtol=1e-5, atol=2e-5)
    c64, p64 = O.black_scholes_f64(price, strike, t, rate, vol)
    for got, orc, truth in ((call, ocall, c64), (put, oput, p64)):
        gpu_err = np.abs(got - truth).max()
        cpu_err = np.abs(orc - truth).max()
        assert gpu_err <= 2 * cpu_err + 1e-6, (gpu_err, cpu_err)
