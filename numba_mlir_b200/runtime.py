"""ctypes binding of the gpux* C-ABI in libnumba_mlir_gpu_runtime_cuda.so.

Counterpart of numba_mlir/numba_mlir/mlir/gpu_runtime.py:14-82, which loads the
runtime named by NUMBA_MLIR_GPU_RUNTIME and registers its symbols.  Here the
only accepted runtime name is "cuda".  There is no fallback of any kind: a
missing library or symbol raises.
"""

import ctypes
import os
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libnumba_mlir_gpu_runtime_cuda.so"

# GpuAllocType / GpuParamType, numba_mlir_gpu_common/GpuCommon.hpp:30-42
ALLOC_DEVICE, ALLOC_SHARED, ALLOC_LOCAL, ALLOC_HOST = 0, 1, 2, 3
(P_NULL, P_BOOL, P_INT8, P_INT16, P_INT32, P_INT64, P_FLOAT32, P_FLOAT64, P_PTR) = range(9)
COPY_H2D, COPY_D2H, COPY_D2D, COPY_DEFAULT = 0, 1, 2, 3


class GPUParamDesc(ctypes.Structure):
    """{const void* data; int32 size; int32 type} (GpuCommon.hpp:45-55)."""

    _fields_ = [("data", ctypes.c_void_p), ("size", ctypes.c_int32), ("type", ctypes.c_int32)]


class GPUAllocResult(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("event", ctypes.c_void_p)]


class Memref2f(ctypes.Structure):
    """Memref<2,float>, math_runtime/include/Common.hpp:17-23 (element units)."""

    _fields_ = [
        ("userData", ctypes.c_void_p),
        ("data", ctypes.c_void_p),
        ("offset", ctypes.c_size_t),
        ("dims", ctypes.c_size_t * 2),
        ("strides", ctypes.c_size_t * 2),
    ]


# Every symbol the header include/numba_mlir_gpu_runtime_cuda.h declares.
_vp, _sz, _i, _cp = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_char_p
SIGNATURES = {
    "gpuxQueueCreate": (_vp, [_cp]),
    "gpuxQueueDestroy": (None, [_vp]),
    "gpuxModuleLoad": (_vp, [_vp, _vp, _sz]),
    "gpuxModuleDestroy": (None, [_vp]),
    "gpuxKernelGet": (_vp, [_vp, _cp]),
    "gpuxKernelDestroy": (None, [_vp]),
    "gpuxLaunchKernel": (_vp, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp]),
    "gpuxLaunchKernelNoEvent": (ctypes.c_int, [_vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp]),
    "gpuxWait": (None, [_vp, _vp]),
    "gpuxDestroyEvent": (None, [_vp, _vp]),
    "gpuxAlloc": (None, [_vp, _sz, _sz, _i, _vp, ctypes.POINTER(GPUAllocResult)]),
    "gpuxDeAlloc": (None, [_vp, _vp]),
    "gpuxSuggestBlockSize": (
        None,
        [_vp, _vp, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32), _sz],
    ),
    "gpuxDuplicateQueue": (_vp, [_vp]),
    "_mlir_ciface_mkl_gemm_float32_device": (
        None,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_float, ctypes.c_float,
         ctypes.POINTER(Memref2f)],
    ),
    "mkl_gemm_float32_device": (
        None,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_float, ctypes.c_float,
         ctypes.POINTER(Memref2f)],
    ),
    "_mlir_ciface_nmb_gemm_float32_device_async": (
        _vp,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_float, ctypes.c_float,
         ctypes.POINTER(Memref2f)],
    ),
    # Memref<2,double> has the same layout (the data pointer is passed as void*)
    "_mlir_ciface_mkl_gemm_float64_device": (
        None,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_double, ctypes.c_double,
         ctypes.POINTER(Memref2f)],
    ),
    "mkl_gemm_float64_device": (
        None,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_double, ctypes.c_double,
         ctypes.POINTER(Memref2f)],
    ),
    "_mlir_ciface_nmb_gemm_float64_device_async": (
        _vp,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_double, ctypes.c_double,
         ctypes.POINTER(Memref2f)],
    ),
    "_mlir_ciface_nmb_contract_rowcol_float32_device": (
        _vp,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.c_float, _i, _vp, _i, _vp, _i,
         ctypes.POINTER(Memref2f)],
    ),
    "gpuxMemcpy": (_vp, [_vp, _vp, _vp, _sz, _i, _vp]),
    "gpuxMemset": (_vp, [_vp, _vp, _i, _sz, _vp]),
    "gpuxRecordEvent": (_vp, [_vp]),
    "gpuxQueueWaitEvents": (_i, [_vp, _vp]),
    "gpuxQueueWaitStream": (_i, [_vp, _vp]),
    "gpuxPeerAlloc": (_vp, [_vp, ctypes.c_size_t]),
    "gpuxPeerFree": (None, [_vp, _vp]),
    "gpuxPeerExport": (_i, [_vp, _vp]),
    "gpuxPeerOpen": (_vp, [_vp, _vp]),
    "gpuxPeerClose": (None, [_vp, _vp]),
    "gpuxEventElapsedMs": (ctypes.c_float, [_vp, _vp]),
    "gpuxQueueSynchronize": (None, [_vp]),
    "gpuxQueueGetStream": (_vp, [_vp]),
    "gpuxQueueGetDevice": (_i, [_vp]),
    "gpuxQueueGetSmCount": (_i, [_vp]),
    "gpuxTestInjectDriverFault": (None, [_cp, _i, _i]),
    "gpuxQueueStatusPtr": (_vp, [_vp]),
    "gpuxGetLastError": (_cp, []),
    "gpuxClearLastError": (None, []),
    "gpuxLaunchCount": (ctypes.c_uint64, []),
    "gpuxGraphBegin": (None, [_vp]),
    "gpuxGraphEnd": (_vp, [_vp]),
    "gpuxGraphLaunch": (_vp, [_vp, _vp]),
    "gpuxGraphDestroy": (None, [_vp]),
    "gpuxCompileToCubin": (_vp, [_vp, _sz, ctypes.POINTER(_sz)]),
    "gpuxFreeHostBlob": (None, [_vp]),
    "gpuxBuiltinKernelNames": (_cp, []),
    "gpuxSumInt32NoAlloc": (_i, [_vp, _vp, _sz, _vp]),
    "gpuxSumInt32NoAllocStatus": (_i, [_vp]),
    "_mlir_ciface_nmb_pairwise_distance_float32_device": (
        _vp,
        [_vp, ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f), ctypes.POINTER(Memref2f)],
    ),
}


class GpuRuntimeError(RuntimeError):
    """A gpux* call failed (the reference aborts the process instead,
    numba_mlir_gpu_runtime_sycl/lib/Utils.hpp:8-21)."""


_lib = None
_lib_lock = threading.Lock()


def lib_path():
    name = os.environ.get("NUMBA_MLIR_GPU_RUNTIME", "cuda")
    if name != "cuda":
        raise ValueError(f"Invalid GPU runtime type: {name}; only 'cuda' is built")
    return os.path.join(_HERE, LIB_NAME)


def load(optional_symbols=()):
    """Loads the runtime library and binds every declared symbol."""
    global _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path):
            raise GpuRuntimeError(
                f"{path} is missing: build it with `python -m numba_mlir_b200.build` "
                "(there is no CPU or eager fallback)"
            )
        # libnvrtc is looked up by soname; point at the toolkit copy when the
        # loader path does not have it.
        if "NUMBA_MLIR_NVRTC_PATH" not in os.environ:
            for cand in ("/usr/local/cuda/lib64/libnvrtc.so.12",):
                if os.path.exists(cand):
                    os.environ["NUMBA_MLIR_NVRTC_PATH"] = cand
                    break
        lib = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            if not hasattr(lib, name):
                if name in optional_symbols:
                    continue
                raise GpuRuntimeError(f"{path} does not export {name}")
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


_fast = None


def fastcall():
    """The native launch path (`_fastcall` extension: argument unboxing,
    GPUParamDesc building and the launch in C++), bound to this library's
    gpuxLaunchKernelNoEvent (the front end orders its work by the queue and
    needs no event per launch).  Built by numba_mlir_b200.build."""
    global _fast
    if _fast is None:
        lib = load()
        try:
            from . import _fastcall
        except ImportError as e:
            raise GpuRuntimeError(
                f"the native launch path is missing ({e}): build it with `python -m numba_mlir_b200.build`"
            ) from None
        _fastcall.init(ctypes.cast(lib.gpuxLaunchKernel, ctypes.c_void_p).value,
                       ctypes.cast(lib.gpuxDestroyEvent, ctypes.c_void_p).value,
                       ctypes.cast(lib.gpuxLaunchKernelNoEvent, ctypes.c_void_p).value)
        _fast = _fastcall
    return _fast


_CODE_OF_DTYPE = {"bool": b"b", "int8": b"c", "uint8": b"C", "int16": b"h", "uint16": b"H", "int32": b"i",
                  "uint32": b"I", "int64": b"q", "uint64": b"Q", "float32": b"f", "float64": b"d"}


def param_code(dtype):
    """One-letter parameter code of the native launch path for a scalar dtype."""
    try:
        return _CODE_OF_DTYPE[np.dtype(dtype).name]
    except KeyError:
        raise TypeError(f"unsupported kernel argument type {dtype}") from None


def check():
    """Raises GpuRuntimeError if the library recorded an error."""
    lib = load()
    msg = lib.gpuxGetLastError()
    if msg is not None:
        text = msg.decode("utf-8", "replace")
        lib.gpuxClearLastError()
        raise GpuRuntimeError(text)


_PARAM_OF_DTYPE = {
    np.dtype(np.bool_): (P_BOOL, ctypes.c_bool),
    np.dtype(np.int8): (P_INT8, ctypes.c_int8),
    np.dtype(np.int16): (P_INT16, ctypes.c_int16),
    np.dtype(np.int32): (P_INT32, ctypes.c_int32),
    np.dtype(np.int64): (P_INT64, ctypes.c_int64),
    np.dtype(np.uint8): (P_INT8, ctypes.c_uint8),
    np.dtype(np.uint16): (P_INT16, ctypes.c_uint16),
    np.dtype(np.uint32): (P_INT32, ctypes.c_uint32),
    np.dtype(np.uint64): (P_INT64, ctypes.c_uint64),
    np.dtype(np.float32): (P_FLOAT32, ctypes.c_float),
    np.dtype(np.float64): (P_FLOAT64, ctypes.c_double),
}


class LocalMem:
    """Launch argument asking for `nbytes` of work-group-local memory
    ({data=NULL, size, ptr}, GpuRuntimeToLlvm.cpp:514-528)."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)


def pack_params(args):
    """Builds the GPUParamDesc[] the generated host code would build
    (mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:444-628): one slot per operand,
    `data` pointing at the value, terminated by {NULL, 0, null}.

    `args` items: int (device pointer) wrapped as ("ptr", value), NumPy scalars
    (typed), LocalMem.  Returns (desc_array, keepalive)."""
    n = len(args)
    descs = (GPUParamDesc * (n + 1))()
    keep = []
    for i, a in enumerate(args):
        if isinstance(a, LocalMem):
            descs[i].data = None
            descs[i].size = a.nbytes
            descs[i].type = P_PTR
            continue
        if isinstance(a, tuple) and a[0] == "ptr":
            slot = ctypes.c_void_p(a[1])
            ptype, size = P_PTR, 8
        else:
            dt = np.asarray(a).dtype
            if dt not in _PARAM_OF_DTYPE:
                raise TypeError(f"unsupported kernel argument type {dt}")
            ptype, ctype = _PARAM_OF_DTYPE[dt]
            slot = ctype(a.item() if hasattr(a, "item") else a)
            size = ctypes.sizeof(ctype)
        keep.append(slot)
        descs[i].data = ctypes.cast(ctypes.pointer(slot), ctypes.c_void_p)
        descs[i].size = size
        descs[i].type = ptype
    descs[n].data = None
    descs[n].size = 0
    descs[n].type = P_NULL
    return descs, keep


def _arg_kind(a):
    if type(a) is tuple:
        return "ptr"
    if isinstance(a, LocalMem):
        return "local"
    return a.dtype if isinstance(a, np.generic) else np.asarray(a).dtype


class _PreparedParams:
    """A GPUParamDesc array with reusable value slots."""

    def __init__(self, kinds):
        n = len(kinds)
        self.descs = (GPUParamDesc * (n + 1))()
        self.slots = []
        for i, k in enumerate(kinds):
            if k == "local" or (type(k) is tuple and k[0] == "local"):
                # ("local", nbytes): a size fixed for the kernel; "local": set by fill()
                self.descs[i].data = None
                self.descs[i].type = P_PTR
                if type(k) is tuple:
                    self.descs[i].size = int(k[1])
                self.slots.append(None)
                continue
            if k == "ptr":
                slot, ptype, size = ctypes.c_void_p(0), P_PTR, 8
            else:
                if k not in _PARAM_OF_DTYPE:
                    raise TypeError(f"unsupported kernel argument type {k}")
                ptype, ctype = _PARAM_OF_DTYPE[k]
                slot, size = ctype(0), ctypes.sizeof(ctype)
            self.slots.append(slot)
            self.descs[i].data = ctypes.cast(ctypes.pointer(slot), ctypes.c_void_p)
            self.descs[i].size = size
            self.descs[i].type = ptype
        self.descs[n].data = None
        self.descs[n].size = 0
        self.descs[n].type = P_NULL
        self.descs_ptr = ctypes.cast(self.descs, ctypes.c_void_p)

    def fill(self, args):
        descs = self.descs
        for i, (slot, a) in enumerate(zip(self.slots, args)):
            if slot is None:
                descs[i].size = a.nbytes
            elif type(a) is tuple:
                slot.value = a[1]
            else:
                slot.value = a.item() if hasattr(a, "item") else a


def _event_list(events):
    """NULL-terminated Event*[] (GpuRuntimeToLlvm.cpp:196-225) or None."""
    events = [e for e in (events or ()) if e]
    if not events:
        return None
    arr = (ctypes.c_void_p * (len(events) + 1))(*events, None)
    return ctypes.cast(arr, ctypes.c_void_p)


class Queue:
    """Owning wrapper of a gpux queue handle plus the handles created from it.

    Mirrors what the reference's generated host code keeps in its per-function
    context (queue, module, kernel handles created once and cached:
    numba_mlir/mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940)."""

    def __init__(self, device=None):
        self.lib = load()
        name = None if device is None else str(device).encode()
        self.handle = self.lib.gpuxQueueCreate(name)
        if not self.handle:
            check()
            raise GpuRuntimeError("gpuxQueueCreate returned NULL")
        self.device = self.lib.gpuxQueueGetDevice(self.handle)
        self._sm_count = None
        self._modules = {}
        self._kernels = {}
        self._builtin = None
        self._prepared = {}
        self._scratch = None
        self._scratch_bytes = 0
        self._status = None

    @classmethod
    def from_stream(cls, stream):
        """Queue over an existing CUDA stream (an integer cudaStream_t handle,
        e.g. `torch.cuda.current_stream().cuda_stream`) of the current device:
        gpuxDuplicateQueue, what generated code gets for a queue it did not
        create (GpuRuntime.cpp:455-463).  The stream stays the caller's."""
        self = cls.__new__(cls)
        self.lib = load()
        self.handle = self.lib.gpuxDuplicateQueue(ctypes.c_void_p(int(stream)))
        if not self.handle:
            check()
            raise GpuRuntimeError("gpuxDuplicateQueue returned NULL")
        self.device = self.lib.gpuxQueueGetDevice(self.handle)
        self._sm_count = None
        self._modules = {}
        self._kernels = {}
        self._builtin = None
        self._prepared = {}
        self._scratch = None
        self._scratch_bytes = 0
        self._status = None
        return self

    @property
    def sm_count(self):
        """Multiprocessors of the queue's device; launch shapes are sized by it."""
        n = self._sm_count
        if n is None:
            n = self.lib.gpuxQueueGetSmCount(self.handle)
            if n <= 0:
                check()
                raise GpuRuntimeError("gpuxQueueGetSmCount failed")
            self._sm_count = n
        return n

    # -- modules / kernels ---------------------------------------------------
    def load_module(self, blob):
        key = hash(blob)
        mod = self._modules.get(key)
        if mod is None:
            buf = ctypes.create_string_buffer(blob, len(blob))
            mod = self.lib.gpuxModuleLoad(self.handle, ctypes.cast(buf, ctypes.c_void_p), len(blob))
            if not mod:
                check()
                raise GpuRuntimeError("gpuxModuleLoad returned NULL")
            self._modules[key] = mod
        return mod

    def get_kernel(self, module, name):
        key = (module, name)
        k = self._kernels.get(key)
        if k is None:
            k = self.lib.gpuxKernelGet(module, name.encode())
            if not k:
                check()
                raise GpuRuntimeError(f"gpuxKernelGet({name}) returned NULL")
            self._kernels[key] = k
        return k

    def builtin(self, name):
        if self._builtin is None:
            self._builtin = self.load_module(b"NMB200:BUILTIN")
        return self.get_kernel(self._builtin, name)

    def suggest_block_size(self, kernel, global_size):
        n = len(global_size)
        g = (ctypes.c_uint32 * 3)(*[min(int(x), 0xFFFFFFFF) for x in global_size])
        b = (ctypes.c_uint32 * 3)(1, 1, 1)
        self.lib.gpuxSuggestBlockSize(self.handle, kernel, g, b, n)
        check()
        return tuple(b[i] for i in range(n))

    # -- launches --------------------------------------------------------------
    def launch(self, kernel, grid, block, args, wait=False):
        """gpuxLaunchKernel; returns nothing (the event is waited on when
        `wait`, as the reference does after every launch,
        GpuRuntimeToLlvm.cpp:619-622, and destroyed either way).

        The GPUParamDesc array and its value slots are built once per
        (kernel, argument kinds) and refilled in place on later launches: the
        driver copies the values during the call, so reuse is safe."""
        kinds = tuple(_arg_kind(a) for a in args)
        key = (kernel, kinds)
        prepared = self._prepared.get(key)
        if prepared is None:
            prepared = _PreparedParams(kinds)
            self._prepared[key] = prepared
        prepared.fill(args)
        ng, nb = len(grid), len(block)
        ev = self.lib.gpuxLaunchKernel(
            self.handle, kernel, grid[0], grid[1] if ng > 1 else 1, grid[2] if ng > 2 else 1,
            block[0], block[1] if nb > 1 else 1, block[2] if nb > 2 else 1,
            None, prepared.descs_ptr,
        )
        if not ev:
            check()
            raise GpuRuntimeError("gpuxLaunchKernel returned NULL")
        if wait:
            self.lib.gpuxWait(self.handle, ev)
        self.lib.gpuxDestroyEvent(self.handle, ev)

    def launch_values(self, kernel, grid, block, kinds, values):
        """`launch` for callers that know the parameter kinds beforehand
        (`kinds`: a hashable tuple of "ptr" / NumPy dtypes) and pass plain
        Python numbers: skips the per-argument type discovery."""
        key = (kernel, kinds)
        prepared = self._prepared.get(key)
        if prepared is None:
            prepared = _PreparedParams(kinds)
            self._prepared[key] = prepared
        for slot, v in zip(prepared.slots, values):
            slot.value = v
        ng, nb = len(grid), len(block)
        ev = self.lib.gpuxLaunchKernel(
            self.handle, kernel, grid[0], grid[1] if ng > 1 else 1, grid[2] if ng > 2 else 1,
            block[0], block[1] if nb > 1 else 1, block[2] if nb > 2 else 1,
            None, prepared.descs_ptr,
        )
        if not ev:
            check()
            raise GpuRuntimeError("gpuxLaunchKernel returned NULL")
        self.lib.gpuxDestroyEvent(self.handle, ev)

    # -- CUDA graphs -----------------------------------------------------------
    def graph_begin(self):
        """Starts recording the queue's launches into a CUDA graph."""
        self.lib.gpuxGraphBegin(self.handle)
        check()

    def graph_end(self):
        g = self.lib.gpuxGraphEnd(self.handle)
        if not g:
            check()
            raise GpuRuntimeError("gpuxGraphEnd returned NULL")
        return g

    def graph_launch(self, graph):
        ev = self.lib.gpuxGraphLaunch(self.handle, graph)
        if not ev:
            check()
            raise GpuRuntimeError("gpuxGraphLaunch returned NULL")
        self.lib.gpuxDestroyEvent(self.handle, ev)

    def graph_destroy(self, graph):
        self.lib.gpuxGraphDestroy(graph)

    # -- memory ----------------------------------------------------------------
    def alloc(self, nbytes, kind=ALLOC_DEVICE):
        res = GPUAllocResult()
        # Alignment is always 64 in generated code (GpuRuntimeToLlvm.cpp:670-672).
        self.lib.gpuxAlloc(self.handle, int(nbytes), 64, kind, None, ctypes.byref(res))
        if res.event:
            self.lib.gpuxDestroyEvent(self.handle, res.event)
        if not res.ptr and kind != ALLOC_LOCAL:
            check()
            raise GpuRuntimeError("gpuxAlloc returned NULL")
        return res.ptr

    def free(self, ptr):
        self.lib.gpuxDeAlloc(self.handle, ptr)

    def memcpy(self, dst, src, nbytes, kind=COPY_DEFAULT, wait=False, deps=None):
        """Asynchronous copy on the queue's stream, after the events in `deps`."""
        ev = self.lib.gpuxMemcpy(self.handle, dst, src, int(nbytes), kind, _event_list(deps))
        if not ev:
            check()
            raise GpuRuntimeError("gpuxMemcpy returned NULL")
        if wait:
            self.lib.gpuxWait(self.handle, ev)
        self.lib.gpuxDestroyEvent(self.handle, ev)

    def wait_events(self, events):
        """Later submissions to this queue run after `events` (events of other
        queues of the device included); the host does not block."""
        if events and self.lib.gpuxQueueWaitEvents(self.handle, _event_list(events)):
            check()
            raise GpuRuntimeError("gpuxQueueWaitEvents failed")

    def wait_stream(self, stream):
        """Later submissions to this queue run after the work already submitted
        to the CUDA stream `stream` (an integer handle; 1 and 2 are the legacy
        and per-thread default streams)."""
        if self.lib.gpuxQueueWaitStream(self.handle, ctypes.c_void_p(int(stream))):
            check()
            raise GpuRuntimeError("gpuxQueueWaitStream failed")

    def memset(self, dst, value, nbytes):
        ev = self.lib.gpuxMemset(self.handle, dst, int(value), int(nbytes), None)
        if not ev:
            check()
            raise GpuRuntimeError("gpuxMemset returned NULL")
        self.lib.gpuxDestroyEvent(self.handle, ev)

    def record(self):
        ev = self.lib.gpuxRecordEvent(self.handle)
        if not ev:
            check()
            raise GpuRuntimeError("gpuxRecordEvent returned NULL")
        return ev

    def elapsed_ms(self, start, end):
        ms = self.lib.gpuxEventElapsedMs(start, end)
        if ms < 0:
            check()
        return ms

    def wait(self, ev):
        self.lib.gpuxWait(self.handle, ev)
        check()

    def destroy_event(self, ev):
        self.lib.gpuxDestroyEvent(self.handle, ev)

    def synchronize(self):
        self.lib.gpuxQueueSynchronize(self.handle)
        check()

    @property
    def stream(self):
        return self.lib.gpuxQueueGetStream(self.handle) or 0

    # -- kernel scratch and status ---------------------------------------------
    COUNTER_BYTES = 65536

    def scratch(self, nbytes):
        """Grow-only device scratch shared by the kernels of this queue (stream
        order keeps consecutive users apart).  The first COUNTER_BYTES hold
        ticket counters that start at zero and that every kernel leaves at
        zero; the rest is uninitialised.  Returns (counters_ptr, data_ptr)."""
        need = self.COUNTER_BYTES + int(nbytes)
        if need > self._scratch_bytes:
            if self._scratch:
                self.free(self._scratch)
            size = max(need, 1 << 20)
            self._scratch = self.alloc(size)
            self._scratch_bytes = size
            self.memset(self._scratch, 0, self.COUNTER_BYTES)
        return self._scratch, self._scratch + self.COUNTER_BYTES

    @property
    def status_ptr(self):
        """Device word kernels with bounded waits set when a wait ran out."""
        if self._status is None:
            self._status = self.lib.gpuxQueueStatusPtr(self.handle)
            if not self._status:
                check()
                raise GpuRuntimeError("gpuxQueueStatusPtr returned NULL")
        return self._status

    def check_status(self):
        """Synchronises and raises if any kernel reported a timed-out wait."""
        word = ctypes.c_uint32(0)
        self.status_ptr
        self.memcpy(ctypes.addressof(word), self._status, 4, COPY_D2H, wait=True)
        check()
        if word.value:
            self.memset(self._status, 0, 64)
            raise GpuRuntimeError(f"a device-side wait timed out (status {word.value})")


_default_queues = {}
_queue_lock = threading.Lock()


def default_device_name():
    """NUMBA_MLIR_DEFAULT_DEVICE, as numba_mlir/mlir/dpctl_interop.py:9; under a
    multi-process launcher each rank defaults to its LOCAL_RANK's GPU."""
    name = os.environ.get("NUMBA_MLIR_DEFAULT_DEVICE")
    if name:
        return name
    rank = os.environ.get("LOCAL_RANK")
    return f"cuda:{rank}" if rank is not None else "cuda:0"


def get_queue(device=None):
    """One shared queue per device string (the reference creates one queue per
    device per function: mlir/lib/Conversion/GpuToGpuRuntime.cpp:169-197)."""
    name = str(device) if device is not None else default_device_name()
    with _queue_lock:
        q = _default_queues.get(name)
        if q is None:
            q = Queue(name)
            _default_queues[name] = q
        return q


def launch_count():
    return int(load().gpuxLaunchCount())


def compile_to_cubin(source):
    """NVRTC-compiles a tagged CUDA C blob for sm_100a on the host (no GPU)."""
    lib = load()
    if isinstance(source, str):
        source = source.encode()
    out = ctypes.c_size_t()
    buf = ctypes.create_string_buffer(source, len(source))
    p = lib.gpuxCompileToCubin(ctypes.cast(buf, ctypes.c_void_p), len(source), ctypes.byref(out))
    if not p:
        check()
        raise GpuRuntimeError("gpuxCompileToCubin returned NULL")
    data = ctypes.string_at(p, out.value)
    lib.gpuxFreeHostBlob(p)
    return data
