"""GPU checks of the gpux* runtime itself, through the C-ABI."""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_queue_refcount_outlives_buffers_and_events(runtime_lib):
    # Buffers and events retain the queue (GpuRuntime.cpp:248-260,287-300).
    from numba_mlir_b200 import runtime as rt

    q = runtime_lib.gpuxQueueCreate(b"cuda:0")
    assert q
    res = rt.GPUAllocResult()
    runtime_lib.gpuxAlloc(q, 1024, 64, rt.ALLOC_DEVICE, None, ctypes.byref(res))
    assert res.ptr and res.event
    runtime_lib.gpuxQueueDestroy(q)  # queue handle released by its creator
    runtime_lib.gpuxWait(q, res.event)  # ...but still alive through the event
    runtime_lib.gpuxDestroyEvent(q, res.event)
    runtime_lib.gpuxDeAlloc(q, res.ptr)  # last reference: queue dies here
    rt.check()


@pytest.mark.parametrize("kind", ["device", "shared", "host"])
def test_alloc_kinds_roundtrip(queue, kind):
    from numba_mlir_b200 import runtime as rt

    k = {"device": rt.ALLOC_DEVICE, "shared": rt.ALLOC_SHARED, "host": rt.ALLOC_HOST}[kind]
    host = np.arange(1000, dtype=np.int32)
    back = np.zeros_like(host)
    p = queue.alloc(host.nbytes, k)
    assert p % 64 == 0
    queue.memcpy(p, host.ctypes.data, host.nbytes, rt.COPY_DEFAULT, wait=True)
    queue.memcpy(back.ctypes.data, p, host.nbytes, rt.COPY_DEFAULT, wait=True)
    queue.free(p)
    assert (back == host).all()


def test_local_alloc_has_no_pointer(queue):
    from numba_mlir_b200 import runtime as rt

    assert queue.alloc(256, rt.ALLOC_LOCAL) is None
    queue.lib.gpuxDeAlloc(queue.handle, None)  # balances the retain
    rt.check()


def test_unknown_builtin_and_bad_blob_are_errors(queue):
    from numba_mlir_b200 import runtime as rt

    with pytest.raises(rt.GpuRuntimeError, match="no builtin kernel"):
        queue.builtin("no_such_kernel")
    with pytest.raises(rt.GpuRuntimeError):
        queue.load_module(b"\x7fELFgarbage-not-a-cubin")


def test_bad_param_type_is_rejected(queue):
    from numba_mlir_b200 import runtime as rt

    k = queue.builtin("nmb_bcast_add_f32_v1")
    descs = (rt.GPUParamDesc * 2)()
    slot = ctypes.c_int64(0)
    descs[0].data = ctypes.cast(ctypes.pointer(slot), ctypes.c_void_p)
    descs[0].size = 8
    descs[0].type = 42
    ev = queue.lib.gpuxLaunchKernel(queue.handle, k, 1, 1, 1, 1, 1, 1, None,
                                    ctypes.cast(descs, ctypes.c_void_p))
    assert not ev
    with pytest.raises(rt.GpuRuntimeError, match="Unhandled param type"):
        rt.check()


def test_nvrtc_module_launch_with_local_memory(queue):
    """CUDA C blob -> gpuxModuleLoad -> gpuxKernelGet -> gpuxLaunchKernel with a
    work-group-local parameter ({NULL, size, ptr}, GpuRuntime.cpp:318-324)."""
    from numba_mlir_b200 import from_host, runtime as rt

    src = (
        "//NMB200:CUDA-SOURCE\n"
        '#include "nmb_device.cuh"\n'
        "extern __shared__ __align__(16) unsigned char nmb_smem[];\n"
        'extern "C" __global__ void rev(const int* in, int* out, uint64_t loc) {\n'
        "  int* tile = reinterpret_cast<int*>(nmb_smem + loc);\n"
        "  int i = blockIdx.x * blockDim.x + threadIdx.x;\n"
        "  tile[threadIdx.x] = in[i];\n"
        "  __syncthreads();\n"
        "  out[i] = tile[blockDim.x - 1 - threadIdx.x];\n}\n"
    ).encode()
    mod = queue.load_module(src)
    k = queue.get_kernel(mod, "rev")
    host = np.arange(256, dtype=np.int32)
    a = from_host(host)
    b = from_host(np.zeros_like(host))
    queue.launch(k, (4,), (64,), [("ptr", a.ptr), ("ptr", b.ptr), rt.LocalMem(64 * 4)], wait=True)
    want = host.reshape(4, 64)[:, ::-1].reshape(-1)
    assert (b.copy_to_host() == want).all()


def test_suggest_block_size_rules(queue):
    # GpuModule.cpp:499-507: dims of size <= 1 get 1; others a power-of-two
    # share of the work-group budget.
    k = queue.builtin("nmb_bcast_add_f32_v1")
    assert queue.suggest_block_size(k, (1,)) == (1,)
    bx, by = queue.suggest_block_size(k, (1 << 20, 1))
    assert by == 1 and bx >= 32 and bx & (bx - 1) == 0
    bx, by, bz = queue.suggest_block_size(k, (7, 1000, 1000))
    assert bx == 7 and bx * by * bz <= 1024


def test_events_time_the_stream(queue):
    from numba_mlir_b200 import zeros

    a = zeros(1 << 24, np.float32)
    e0 = queue.record()
    queue.memset(a.ptr, 0, a.nbytes)
    e1 = queue.record()
    queue.wait(e1)
    ms = queue.elapsed_ms(e0, e1)
    assert 0 < ms < 1000
    queue.destroy_event(e0)
    queue.destroy_event(e1)


def test_cuda_array_interface_interop_with_torch(queue):
    import torch

    from numba_mlir_b200 import as_device_array, from_host

    host = np.arange(12, dtype=np.float32).reshape(3, 4)
    d = from_host(host)
    t = torch.as_tensor(d, device="cuda")
    assert t.shape == (3, 4) and t.data_ptr() == d.ptr
    assert np.array_equal(t.cpu().numpy(), host)
    back = as_device_array(t * 2)
    queue.synchronize()
    torch.cuda.synchronize()
    assert np.array_equal(back.copy_to_host(), host * 2)


class _StreamedExport:
    """Exporter of version 3 of the CUDA array interface: names the stream the
    data is ready on, as cupy and numba.cuda do."""

    def __init__(self, tensor, stream):
        self._tensor = tensor
        iface = dict(tensor.__cuda_array_interface__)
        iface["version"] = 3
        iface["stream"] = stream
        self.__cuda_array_interface__ = iface


def test_import_orders_queue_after_producer_stream(queue):
    import torch

    import numba_mlir_b200 as nm

    n = 1 << 24
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        t = torch.zeros(n, dtype=torch.float32, device="cuda")
        for k in range(1, 41):  # enough queued work that a missing dependency shows
            t.add_(float(k) - float(k - 1))
    d = nm.as_device_array(_StreamedExport(t, side.cuda_stream))

    @nm.njit(parallel=True)
    def twice(x):
        return x + x

    got = twice(d).copy_to_host()
    side.synchronize()
    assert got.min() == 80.0 and got.max() == 80.0


def test_wait_stream_accepts_default_stream_names(queue):
    # 1 and 2 name the legacy and the per-thread default streams
    queue.wait_stream(1)
    queue.wait_stream(2)
    queue.wait_stream(queue.stream or 0)
    queue.synchronize()


def test_duplicate_queue_wraps_a_foreign_stream_in_order(queue, runtime_lib):
    """gpuxDuplicateQueue (GpuRuntime.cpp:455-463 hands generated code a queue
    over a stream it did not create): work launched on the duplicate runs on
    torch's current stream, in order with torch's own work on it."""
    import ctypes

    import torch

    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime

    stream = torch.cuda.Stream()
    n = 1 << 22
    with torch.cuda.stream(stream):
        t = torch.zeros(n, dtype=torch.float32, device="cuda")
        for _ in range(20):
            t += 1.0  # torch work queued on the stream first
        q2 = runtime.Queue.from_stream(stream.cuda_stream)
        assert q2.stream == stream.cuda_stream and q2.device == queue.device
        arr = nm.as_device_array(t, queue=q2)
        out = nm.empty((), np.float32, q2)
        from numba_mlir_b200 import reduce_ops

        reduce_ops.reduce(arr, "sum", None, out=out)  # launched through the duplicate: after the adds
        t += 1.0  # and torch work after it
        stream.synchronize()
    assert float(out.copy_to_host()) == 20.0 * n
    assert float(t[0]) == 21.0
    del ctypes


def test_wait_gives_up_after_the_configured_time(queue, runtime_lib, monkeypatch):
    """NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS bounds gpuxWait on the host.  The event
    waited on sits behind a few hundred milliseconds of ordinary work (nothing
    hangs): with a 1 ms bound the call returns with the error set while the
    work goes on; without the bound the same wait completes."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import reduce_ops, runtime

    a = nm.zeros(1 << 28, np.int32, queue)  # 1 GiB: about 0.17 ms per reduction
    out = nm.empty((), np.int64, queue)
    reduce_ops.reduce(a, "sum", None, out=out)
    queue.synchronize()
    for _ in range(1500):
        reduce_ops.reduce(a, "sum", None, out=out)
    ev = queue.record()
    monkeypatch.setenv("NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS", "1")
    runtime_lib.gpuxWait(queue.handle, ev)
    with pytest.raises(runtime.GpuRuntimeError, match="not reached within 1 ms"):
        runtime.check()
    monkeypatch.setenv("NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS", "60000")
    queue.wait(ev)  # bounded, long enough
    monkeypatch.delenv("NUMBA_MLIR_GPU_WAIT_TIMEOUT_MS")
    queue.wait(ev)
    queue.destroy_event(ev)
    assert int(out.copy_to_host()) == 0
    queue.check_status()


def test_injected_driver_faults_are_reported_and_leave_the_queue_usable(queue, runtime_lib):
    """Host-side failure injection: a driver call made to return CUDA_ERROR_*
    surfaces as an error of the gpux* call (NULL result + message); the next
    call works."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import runtime

    CUDA_ERROR_LAUNCH_OUT_OF_RESOURCES, CUDA_ERROR_INVALID_IMAGE, CUDA_ERROR_NOT_FOUND = 701, 200, 500
    add = nm.njit(lambda a, out: out.__setitem__(slice(None), a + np.float32(1)))
    a, out = nm.zeros(1000, np.float32, queue), nm.zeros(1000, np.float32, queue)
    add(a, out)  # compiled and loaded
    runtime_lib.gpuxTestInjectDriverFault(b"cuLaunchKernel", CUDA_ERROR_LAUNCH_OUT_OF_RESOURCES, 1)
    with pytest.raises(runtime.GpuRuntimeError, match="too many resources|LaunchKernel"):
        add(a, out)
    add(a, out)
    assert np.all(out.copy_to_host() == 1)
    src = b"//NMB200:CUDA-SOURCE\nextern \"C\" __global__ void probe_k(int *p) { p[0] = 1; }\n"
    runtime_lib.gpuxTestInjectDriverFault(b"cuModuleLoadDataEx", CUDA_ERROR_INVALID_IMAGE, 1)
    q2 = runtime.Queue(f"cuda:{queue.device}")
    with pytest.raises(runtime.GpuRuntimeError):
        q2.load_module(src)
    mod = q2.load_module(src)
    runtime_lib.gpuxTestInjectDriverFault(b"cuModuleGetFunction", CUDA_ERROR_NOT_FOUND, 1)
    with pytest.raises(runtime.GpuRuntimeError):
        q2.get_kernel(mod, "probe_k")
    assert q2.get_kernel(mod, "probe_k")
    runtime_lib.gpuxTestInjectDriverFault(None, 0, 0)
    queue.check_status()


def test_double_dealloc_keeps_the_queue_alive(queue, runtime_lib):
    """A pointer freed twice (or never allocated here) is reported and does not
    drop a second reference of the queue."""
    from numba_mlir_b200 import runtime

    q2 = runtime.Queue(f"cuda:{queue.device}")
    p = q2.alloc(4096)
    keep = q2.alloc(4096)
    q2.free(p)
    q2.free(p)
    with pytest.raises(runtime.GpuRuntimeError, match="not allocated by this queue"):
        runtime.check()
    # the queue still works and still owns `keep`
    q2.memset(keep, 0, 4096)
    q2.synchronize()
    q2.free(keep)
    assert queue.sm_count >= 1
