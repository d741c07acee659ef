"""`map_host`: host arrays in and out through the chunked three-queue pipeline
give the same bits as one whole-array call."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,chunk", [(1000, 4096), (4096, 4096), (4096 * 7, 4096), (4096 * 7 + 13, 4096),
                                     (1 << 20, 1 << 18)])
def test_map_host_black_scholes_matches_whole_array_call(queue, n, chunk):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import workloads
    from oracle import configs as O

    price, strike, t, rate, vol = O.make_inputs("black_scholes", max(n, 1 << 14) / 2**24, seed=5)
    price, strike, t = price[:n].copy(), strike[:n].copy(), t[:n].copy()
    ins = [nm.pinned_empty(n, np.float32, queue) for _ in range(3)]
    for dst, src in zip(ins, (price, strike, t)):
        dst[:] = src
    outs = [nm.pinned_empty(n, np.float32, queue) for _ in range(2)]
    for o in outs:
        o[:] = -1
    for _ in range(2):  # second pass reuses the pipeline, its slots and its events
        nm.map_host(workloads.black_scholes, ins, outs, scalars=(rate, vol), chunk=chunk, queue=queue)
    call, put = nm.empty(n), nm.empty(n)
    workloads.black_scholes(nm.from_host(price), nm.from_host(strike), nm.from_host(t), rate, vol, call, put)
    assert np.array_equal(np.asarray(outs[0]).view(np.uint32), call.copy_to_host().view(np.uint32))
    assert np.array_equal(np.asarray(outs[1]).view(np.uint32), put.copy_to_host().view(np.uint32))


def test_map_host_accepts_pageable_arrays_and_checks_arguments(queue):
    import numba_mlir_b200 as nm

    @nm.njit
    def twice(a, out):
        out[:] = a * 2

    a = np.arange(10000, dtype=np.int32)
    out = np.zeros_like(a)
    nm.map_host(twice, [a], [out], chunk=3000, queue=queue)
    assert np.array_equal(out, a * 2)
    with pytest.raises(ValueError):
        nm.map_host(twice, [a], [out[:5].copy()], chunk=3000, queue=queue)
    with pytest.raises(ValueError):  # 100 rows in, 10000 out
        nm.map_host(twice, [a.reshape(100, 100)], [out], chunk=3000, queue=queue)
    with pytest.raises(TypeError):   # not contiguous
        nm.map_host(twice, [a[::2]], [out[::2]], chunk=3000, queue=queue)


def test_map_host_row_chunks_of_a_matrix_and_a_resident_operand(queue):
    """Inputs and outputs cut along axis 0 with different row shapes (a row
    reduction; the distance rows of a block of points against a second operand
    that stays whole on the device)."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import contraction, workloads
    from oracle import configs as O

    rng = np.random.default_rng(3)
    a = rng.standard_normal((1000, 512)).astype(np.float32)
    out = np.zeros(1000, np.float32)
    for _ in range(2):
        nm.map_host(workloads.sum_axis1, [a], [out], chunk=192, queue=queue)
    whole = nm.empty(1000, np.float32)
    workloads.sum_axis1(nm.from_host(a), whole)
    assert np.array_equal(out.view(np.uint32), whole.copy_to_host().view(np.uint32))

    x = rng.uniform(0, 1, (700, 64)).astype(np.float32)
    y = rng.uniform(0, 1, (300, 64)).astype(np.float32)
    d = np.zeros((700, 300), np.float32)

    def rows(xc, yw, dc):
        contraction.pairwise_distance(xc, yw, dc)

    nm.map_host(rows, [x], [d], resident=[y], chunk=256, queue=queue)
    want = np.zeros_like(d)
    O.pairwise(x, y, want)
    np.testing.assert_allclose(d, want, rtol=1e-5, atol=1e-6)
