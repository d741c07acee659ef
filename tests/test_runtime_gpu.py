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
