"""gpuxSumInt32NoAlloc: the entry point for callers that cannot allocate.

Some callers of the runtime must not trigger a device allocation: a monitoring
or real-time thread that may not wait on the CUDA allocator, a process whose
device memory was all handed out at start-up.  This
entry point keeps its scratch in a fixed array inside the library, so it can
be called from there.  It is checked here through the C-ABI against the
regular full-sum path (per-queue scratch), bit-exactly (integer sums), on two
calls in a row because the second call meets whatever the first one left in
the shared array.  Collected last on purpose: a failure here stops nothing else.
"""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sum_no_alloc(lib, queue, dev_in, dev_out):
    rc = lib.gpuxSumInt32NoAlloc(queue.handle, dev_in.ptr, dev_in.size, dev_out.ptr)
    from numba_mlir_b200 import runtime

    if rc != 0:
        runtime.check()
        raise AssertionError("gpuxSumInt32NoAlloc failed without an error message")


def test_no_alloc_sum_matches_regular_entry_point_twice(queue, runtime_lib):
    from numba_mlir_b200 import empty, from_host, reduce_ops

    rng = np.random.default_rng(11)
    out_a, out_b = empty((), np.int64), empty((), np.int64)
    for n in ((1 << 22) + 3, 12345):  # second call: smaller grid, stale partials behind it
        host = rng.integers(-1000, 1001, n, dtype=np.int32)
        d = from_host(host)
        _sum_no_alloc(runtime_lib, queue, d, out_a)
        reduce_ops.reduce(d, "sum", None, out=out_b)
        queue.synchronize()
        got, want = int(out_a.copy_to_host()), int(out_b.copy_to_host())
        assert got == want == int(host.sum(dtype=np.int64))
        # the entry point's own failure report: no bounded wait ran out
        assert runtime_lib.gpuxSumInt32NoAllocStatus(queue.handle) == 0
    queue.check_status()


def test_no_alloc_sum_rejects_what_it_cannot_handle(queue, runtime_lib):
    from numba_mlir_b200 import empty, from_host, runtime

    d = from_host(np.arange(64, dtype=np.int32))
    out = empty((), np.int64)
    # empty input
    assert runtime_lib.gpuxSumInt32NoAlloc(queue.handle, d.ptr, 0, out.ptr) != 0
    with pytest.raises(runtime.GpuRuntimeError, match="outside 1 .. 2\\^32"):
        runtime.check()
    # beyond the stated maximum
    assert runtime_lib.gpuxSumInt32NoAlloc(queue.handle, d.ptr, (1 << 32) + 1, out.ptr) != 0
    with pytest.raises(runtime.GpuRuntimeError, match="outside 1 .. 2\\^32"):
        runtime.check()
    # misaligned input
    assert runtime_lib.gpuxSumInt32NoAlloc(queue.handle, d.ptr + 4, 8, out.ptr) != 0
    with pytest.raises(runtime.GpuRuntimeError, match="16-byte aligned"):
        runtime.check()
