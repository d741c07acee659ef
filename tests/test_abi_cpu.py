"""CPU checks of the drop-in boundary: the library builds for sm_100a, loads
without a GPU, and exports every symbol include/*.h declares."""

import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "numba_mlir_gpu_runtime_cuda.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(n for n in names if n.startswith(("gpux", "_mlir_ciface", "mkl_"))))


def test_header_declares_the_13_reference_exports():
    # numba_mlir_gpu_runtime_sycl/lib/GpuRuntime.cpp:361-463
    ref = {
        "gpuxQueueCreate", "gpuxQueueDestroy", "gpuxModuleLoad", "gpuxModuleDestroy",
        "gpuxKernelGet", "gpuxKernelDestroy", "gpuxLaunchKernel", "gpuxWait",
        "gpuxDestroyEvent", "gpuxAlloc", "gpuxDeAlloc", "gpuxSuggestBlockSize",
        "gpuxDuplicateQueue",
    }
    assert ref <= set(declared_functions())


def test_library_exports_every_declared_symbol(runtime_lib):
    from numba_mlir_b200 import runtime

    for name in declared_functions():
        assert hasattr(runtime_lib, name), name
        assert name in runtime.SIGNATURES, f"{name} has no ctypes signature"


def test_only_c_abi_symbols_are_visible():
    # numba_mlir_gpu_common/export.txt:1-4 exports gpux* only.
    import subprocess

    from numba_mlir_b200 import runtime

    out = subprocess.run(["nm", "-D", "--defined-only", runtime.lib_path()],
                         capture_output=True, text=True, check=True).stdout
    syms = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert syms, "no exported functions"
    for s in syms:
        assert s.startswith(("gpux", "_mlir_ciface_", "mkl_gemm_")), s


def test_param_desc_layout():
    from numba_mlir_b200 import runtime

    # {ptr, i32, i32}: mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:87-93
    assert ctypes.sizeof(runtime.GPUParamDesc) == 16
    assert runtime.GPUParamDesc.size.offset == 8
    assert runtime.GPUParamDesc.type.offset == 12
    assert ctypes.sizeof(runtime.GPUAllocResult) == 16
    assert ctypes.sizeof(runtime.Memref2f) == 56


def test_pack_params_terminator_and_types():
    from numba_mlir_b200 import runtime

    descs, keep = runtime.pack_params(
        [("ptr", 0x1000), np.int64(7), np.float32(1.5), np.bool_(True), runtime.LocalMem(256)]
    )
    assert [d.type for d in descs] == [runtime.P_PTR, runtime.P_INT64, runtime.P_FLOAT32,
                                       runtime.P_BOOL, runtime.P_PTR, runtime.P_NULL]
    assert [d.size for d in descs] == [8, 8, 4, 1, 256, 0]
    assert descs[4].data is None and descs[5].data is None
    assert ctypes.cast(descs[1].data, ctypes.POINTER(ctypes.c_int64))[0] == 7
    assert ctypes.cast(descs[2].data, ctypes.POINTER(ctypes.c_float))[0] == 1.5


def test_no_device_means_loud_failure(runtime_lib):
    """Without a CUDA device the queue cannot be created and the error is
    reported, not papered over by a fallback."""
    import pytest

    from numba_mlir_b200 import runtime

    q = runtime_lib.gpuxQueueCreate(None)
    if q:  # a GPU is present: nothing to check here
        runtime_lib.gpuxQueueDestroy(q)
        return
    assert runtime_lib.gpuxGetLastError() is not None
    with pytest.raises(runtime.GpuRuntimeError):
        runtime.check()
    assert runtime_lib.gpuxGetLastError() is None


def test_bad_device_name_is_rejected(runtime_lib):
    import pytest

    from numba_mlir_b200 import runtime

    assert not runtime_lib.gpuxQueueCreate(b"level_zero:gpu:0")
    with pytest.raises(runtime.GpuRuntimeError, match="unknown device name"):
        runtime.check()


def test_builtin_kernel_table(runtime_lib):
    names = runtime_lib.gpuxBuiltinKernelNames().decode().split()
    for n in ("nmb_bcast_add_f32", "nmb_black_scholes_f32"):
        assert n in names


def test_nvrtc_compiles_generated_source_for_sm100a_without_gpu(runtime_lib):
    from numba_mlir_b200 import runtime

    src = (
        "//NMB200:CUDA-SOURCE\n//NMB200:OPTIONS --fmad=false\n"
        '#include "nmb_device.cuh"\n'
        'extern "C" __global__ void k(float* a, int64_t n) {\n'
        "  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;\n"
        "  if (i < n) a[i] = nmb::f_erf(a[i]);\n}\n"
    )
    cubin = runtime.compile_to_cubin(src)
    assert cubin[:4] == b"\x7fELF"


def test_nvrtc_error_is_reported(runtime_lib):
    import pytest

    from numba_mlir_b200 import runtime

    with pytest.raises(runtime.GpuRuntimeError, match="NVRTC compilation failed"):
        runtime.compile_to_cubin("//NMB200:CUDA-SOURCE\nthis is not CUDA\n")


def test_native_launch_path_builds_the_param_desc_array(runtime_lib):
    """The `_fastcall` extension unboxes arguments and builds the GPUParamDesc
    array the generated host code would build
    (mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:444-628): here its launch goes to
    a recording stand-in for gpuxLaunchKernel."""
    import ctypes

    from numba_mlir_b200 import lazy, runtime
    from numba_mlir_b200.device_array import DeviceArray

    fast = runtime.fastcall()
    seen = []

    LAUNCH = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t,
                              ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p,
                              ctypes.c_void_p)
    DESTROY = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p)

    def fake_launch(queue, kernel, gx, gy, gz, bx, by, bz, events, params):
        descs = ctypes.cast(params, ctypes.POINTER(runtime.GPUParamDesc))
        out, i = [], 0
        while descs[i].type != runtime.P_NULL or descs[i].size != 0:
            d = descs[i]
            raw = ctypes.string_at(d.data, d.size) if d.data else None
            out.append((d.type, d.size, raw))
            i += 1
        seen.append(((queue, kernel), (gx, gy, gz), (bx, by, bz), out))
        return 0x1234

    launch_cb, destroy_cb = LAUNCH(fake_launch), DESTROY(lambda q, e: None)
    fast.init(ctypes.cast(launch_cb, ctypes.c_void_p).value, ctypes.cast(destroy_cb, ctypes.c_void_p).value)
    try:
        a = lazy.fake_array((6, 8), np.float32, ptr=0x7000_0000_1000)
        v = a.T  # not C-contiguous: strides follow the shape
        fast.launch_kernel(11, 22, (3, 2), (64,), b"A\x02C" + b"A\x02S" + b"f" + b"q" + b"b", (a, v, 1.5, -7, True),
                           (6, 8, 1, -4096))
        (_qk, grid, block, descs) = seen[-1]
        assert _qk == (11, 22) and grid == (3, 2, 1) and block == (64, 1, 1)
        i64 = lambda x: np.int64(x).tobytes()  # noqa: E731
        assert descs[0] == (runtime.P_PTR, 8, np.uint64(0x7000_0000_1000).tobytes())
        assert [d[2] for d in descs[1:3]] == [i64(6), i64(8)]
        assert descs[3] == (runtime.P_PTR, 8, np.uint64(0x7000_0000_1000).tobytes())
        assert [d[2] for d in descs[4:8]] == [i64(8), i64(6), i64(1), i64(8)]  # shape, then element strides
        assert descs[8] == (runtime.P_FLOAT32, 4, np.float32(1.5).tobytes())
        assert descs[9] == (runtime.P_INT64, 8, i64(-7))
        assert descs[10] == (runtime.P_BOOL, 1, b"\x01")
        assert [d[2] for d in descs[11:14]] == [i64(6), i64(8), i64(1)]
        assert descs[14] == (runtime.P_PTR, 4096, None)  # the local-memory request
        # a recorded plan: two launches over the call's arguments
        b = lazy.fake_array((48,), np.float32, ptr=0x7000_0000_9000)
        fast.replay(5, ((31, (1,), (256,), b"ppkf", (0, 1, 48, 2)), (32, (2,), (256,), b"pk", (1, 48))), (a, b, 0.25))
        first, second = seen[-2], seen[-1]
        assert first[0] == (5, 31) and [d[0] for d in first[3]] == [runtime.P_PTR, runtime.P_PTR, runtime.P_INT64,
                                                                    runtime.P_FLOAT32]
        assert first[3][1][2] == np.uint64(0x7000_0000_9000).tobytes() and first[3][3][2] == np.float32(0.25).tobytes()
        assert second[0] == (5, 32) and second[1] == (2, 1, 1)
        with pytest.raises(IndexError):
            fast.replay(5, ((31, (1,), (256,), b"p", (7,)),), (a,))
        # the plan key computed natively equals the Python one
        for args in ((a, b), (a, a), (a[1:], a[:-1]), (a, 2, 0.5, True)):
            for x in args:
                if isinstance(x, DeviceArray):
                    x.trace_sig, x.extent
            assert fast.signature(args, DeviceArray) == lazy.signature_of(args)
        assert fast.signature((a, np.float32(1)), DeviceArray) is None  # NumPy scalars: typed in Python
    finally:
        lib = runtime.load()
        fast.init(ctypes.cast(lib.gpuxLaunchKernel, ctypes.c_void_p).value,
                  ctypes.cast(lib.gpuxDestroyEvent, ctypes.c_void_p).value)
