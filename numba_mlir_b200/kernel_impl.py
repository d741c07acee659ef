"""`@kernel` API: get_global_id & co, atomics, barriers, local/private arrays,
group reductions, and the launcher.

User-facing names and call forms are those of numba_mlir/numba_mlir/kernel.py
and mlir/kernel_impl.py:97-482; `kernel[global_size, local_size](*args)` as in
mlir/kernel_base.py:24-58.  The functions below are stubs that only mean
something inside a kernel body; their typing is registered with Numba so that
the body can be type-inferred, and codegen_ir lowers them to CUDA.
"""

import copy

import numpy as np

from . import runtime as _rt
from numba.core import types
from numba.core.typing.templates import AbstractTemplate, ConcreteTemplate, infer_global, signature

from .decorators import _wrap_arg, check_device_args
from .device_array import DeviceArray


def _stub_error():
    raise NotImplementedError("This is a stub: it can only be called inside a @kernel function")


# --- ids and sizes (kernel_impl.py:214-248) -----------------------------------
def get_global_id(axis):
    _stub_error()


def get_local_id(axis):
    _stub_error()


def get_group_id(axis):
    _stub_error()


def get_global_size(axis):
    _stub_error()


def get_local_size(axis):
    _stub_error()


ID_FUNCS = (get_global_id, get_local_id, get_group_id, get_global_size, get_local_size)


class _IdTemplate(ConcreteTemplate):
    cases = [signature(types.int64, types.int64)]


for _f in ID_FUNCS:
    infer_global(_f)(_IdTemplate)


class Stub:
    """Namespace object that is meaningless outside a kernel."""

    __slots__ = ()

    def __new__(cls):
        raise NotImplementedError("%s is not instantiable" % cls)


# --- atomics (kernel_impl.py:267-322) -------------------------------------------
def atomic_add(arr, idx, val):
    _stub_error()


def atomic_sub(arr, idx, val):
    _stub_error()


class atomic(Stub):
    add = staticmethod(atomic_add)
    sub = staticmethod(atomic_sub)


class _AtomicTemplate(AbstractTemplate):
    def generic(self, args, kws):
        assert not kws
        ary, idx, val = args
        if not isinstance(ary, types.Array):
            return None
        if ary.ndim == 1:
            return signature(ary.dtype, ary, types.intp, ary.dtype)
        return signature(ary.dtype, ary, idx, ary.dtype)


infer_global(atomic_add)(_AtomicTemplate)
infer_global(atomic_sub)(_AtomicTemplate)

# --- barriers (kernel_impl.py:325-363) ---------------------------------------------
LOCAL_MEM_FENCE = 0x1
GLOBAL_MEM_FENCE = 0x2


def barrier(flags=None):
    _stub_error()


def mem_fence(flags=None):
    _stub_error()


class _FenceTemplate(ConcreteTemplate):
    cases = [signature(types.none), signature(types.none, types.int64), signature(types.none, types.none)]


infer_global(barrier)(_FenceTemplate)
infer_global(mem_fence)(_FenceTemplate)


# --- local / private arrays (kernel_impl.py:366-437) --------------------------------
def local_array(shape, dtype):
    _stub_error()


def private_array(shape, dtype):
    _stub_error()


class local(Stub):
    array = staticmethod(local_array)


class private(Stub):
    array = staticmethod(private_array)


def _parse_dtype(dtype):
    if isinstance(dtype, types.DType):
        return dtype.dtype
    if isinstance(dtype, types.NumberClass):
        return dtype.dtype
    if isinstance(dtype, types.TypeRef):
        return dtype.instance_type
    return None


def _array_pysig(shape, dtype):
    pass


class _ArrayTemplate(AbstractTemplate):
    def generic(self, args, kws):
        # positional or keyword form (local.array(shape=..., dtype=...),
        # numba_mlir/mlir/tests/test_gpu.py:1140-1142)
        kws = dict(kws)
        args = list(args)
        for name in ("shape", "dtype")[len(args):]:
            if name not in kws:
                return None
            args.append(kws.pop(name))
        if kws or len(args) != 2:
            return None
        shape, dtype = args
        if isinstance(shape, types.Integer):
            ndim = 1
        elif isinstance(shape, (types.Tuple, types.UniTuple)) and all(
                isinstance(s, types.Integer) for s in shape.types):
            ndim = len(shape)
        else:
            return None
        nb_dtype = _parse_dtype(dtype)
        if nb_dtype is None:
            return None
        from numba.core.utils import pysignature

        return signature(types.Array(nb_dtype, ndim, "C"), shape, dtype).replace(
            pysig=pysignature(_array_pysig))


infer_global(local_array)(_ArrayTemplate)
infer_global(private_array)(_ArrayTemplate)


# --- group reductions (kernel_impl.py:440-482) ---------------------------------------
def group_reduce_add(value):
    _stub_error()


def group_reduce_mul(value):
    _stub_error()


def group_reduce_min(value):
    _stub_error()


def group_reduce_max(value):
    _stub_error()


class group(Stub):
    reduce_add = staticmethod(group_reduce_add)
    reduce_mul = staticmethod(group_reduce_mul)
    reduce_min = staticmethod(group_reduce_min)
    reduce_max = staticmethod(group_reduce_max)


GROUP_REDUCE = {
    group_reduce_add: ("OpAdd", "add"), group_reduce_mul: ("OpMul", "mul"),
    group_reduce_min: ("OpMin", "min"), group_reduce_max: ("OpMax", "max"),
}


class _GroupTemplate(AbstractTemplate):
    def generic(self, args, kws):
        assert not kws
        (val,) = args
        val = types.unliteral(val)
        if isinstance(val, (types.Integer, types.Float)):
            return signature(val, val)
        return None


for _f in GROUP_REDUCE:
    infer_global(_f)(_GroupTemplate)

# (namespace object, attribute) -> stub, for inline `atomic.add(...)` forms
API_ATTRS = {
    (atomic, "add"): atomic_add, (atomic, "sub"): atomic_sub,
    (local, "array"): local_array, (private, "array"): private_array,
    (group, "reduce_add"): group_reduce_add, (group, "reduce_mul"): group_reduce_mul,
    (group, "reduce_min"): group_reduce_min, (group, "reduce_max"): group_reduce_max,
}

DEFAULT_LOCAL_SIZE = ()


# --- launcher ----------------------------------------------------------------------------
def _raise_error(desc):
    raise ValueError(desc)


def _process_dims(dims):
    if isinstance(dims, (int, np.integer)):
        return (int(dims),)
    if isinstance(dims, (list, tuple)):
        n = len(dims)
        if n > 3:
            _raise_error(f"Invalid dimentions count: {n}")
        return tuple(int(d) for d in dims)
    _raise_error(f"Invalid dimentions type: {type(dims)}")


def call_signature(args):
    """Cache key of a compiled kernel: what its code depends on."""
    sig = []
    for a in args:
        if isinstance(a, DeviceArray):
            sig.append(a.call_sig)
        else:
            sig.append(("scalar", type(a).__name__, getattr(a, "dtype", None) and a.dtype.name))
    return tuple(sig)


def marshal_params(args, param_layout):
    """Python arguments -> launch parameter list: an array is its pointer,
    its shape and, unless C-contiguous, its element strides (the flattened
    memref form of numba_mlir/mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:507-536)."""
    params = []
    for a, lay in zip(args, param_layout):
        if lay[0] == "array":
            params.append(("ptr", a.ptr))
            params += [np.int64(s) for s in a.shape]
            if lay[2] != "C":
                params += [np.int64(st // a.dtype.itemsize) for st in a.strides]
        else:
            params.append(lay[1].type(a))
    return params


_I64 = np.dtype(np.int64)


def param_kinds(param_layout, trailing_int64=0):
    """Parameter kinds of a compiled kernel in launch order (see marshal_values)."""
    kinds = []
    for lay in param_layout:
        if lay[0] == "array":
            kinds.append("ptr")
            kinds += [_I64] * (lay[1] * (1 if lay[2] == "C" else 2))
        else:
            kinds.append(lay[1])
    return tuple(kinds + [_I64] * trailing_int64)


def marshal_values(args, param_layout):
    """Like marshal_params, as plain Python numbers for Queue.launch_values."""
    vals = []
    for a, lay in zip(args, param_layout):
        if lay[0] == "array":
            vals.append(a.ptr)
            vals.extend(a.shape)
            if lay[2] != "C":
                it = a.dtype.itemsize
                vals.extend(st // it for st in a.strides)
        else:
            vals.append(a.item() if isinstance(a, np.generic) else a)
    return vals


class Kernel:
    """`kernel(func)`; configure with `k[global_size, local_size]`, then call."""

    def __init__(self, func, kwargs):
        self.py_func = func
        self.options = dict(kwargs)
        self.global_size = ()
        self.local_size = ()
        self._compiled = {}
        self._launchers = {}  # (argument kinds, rank of the launch) -> (compiled kernel, index of an array argument)

    def copy(self):
        return copy.copy(self)

    def configure(self, global_size, local_size):
        global_dim_count = len(global_size)
        local_dim_count = len(local_size)
        assert local_dim_count <= global_dim_count
        if local_dim_count != 0 and local_dim_count < global_dim_count:
            local_size = tuple(local_size[i] if i < local_dim_count else 1
                               for i in range(global_dim_count))
        ret = self.copy()
        ret.global_size = tuple(global_size)
        ret.local_size = tuple(local_size)
        return ret

    def __getitem__(self, args):
        if not isinstance(args, tuple):
            args = (args,)
        nargs = len(args)
        if nargs < 1 or nargs > 2:
            _raise_error(f"Invalid kernel arguments count: {nargs}")
        gs = _process_dims(args[0])
        ls = _process_dims(args[1]) if nargs > 1 else ()
        return self.configure(gs, ls)

    def _signature(self, args):
        return call_signature(args)

    def __call__(self, *args, **kwargs):
        if kwargs:
            _raise_error("kwargs not supported")
        # A call like one seen before (same argument kinds): straight to the
        # native launch path, which reads pointers, shapes and scalars out of
        # the argument objects and builds the GPUParamDesc array.
        try:
            key = tuple([a._call_sig if type(a) is DeviceArray else type(a) for a in args])
        except AttributeError:
            key = None
        entry = self._launchers.get((key, len(self.global_size))) if key is not None else None
        if entry is not None:
            ck, first = entry
            queue = args[first]._buf.queue
            for a in args:
                if type(a) is DeviceArray and a._buf.queue is not queue and a._buf.queue.device != queue.device:
                    check_device_args(args)
            kernel = ck._handles.get(queue) or ck.handle_on(queue)
            gs = self.global_size
            local = self.local_size or ck.block_size_on(queue, kernel, gs)
            if 0 in gs:
                return
            grid = tuple([(g + l - 1) // l for g, l in zip(gs, local)])
            tail = gs + (1,) * (3 - len(gs))
            if ck.local_bytes:
                tail += (-ck.local_bytes,)
            try:
                _rt.fastcall().launch_kernel(queue.handle, kernel, grid, local, ck.layout_code(), args, tail)
            except RuntimeError:
                _rt.check()
                raise
            return
        self._call_slow(args)

    def _call_slow(self, args):
        """First call with these argument kinds: wraps foreign arrays, checks the
        devices, compiles, and remembers the compiled kernel for the fast path."""
        args = tuple(_wrap_arg(a) for a in args)
        if not check_device_args(args):
            raise TypeError("kernel launch needs at least one device array argument")
        ndim = len(self.global_size)
        if not 1 <= ndim <= 3:
            _raise_error(f"Invalid dim count: {ndim}")
        from . import codegen_ir

        key = (self._signature(args), ndim)
        ck = self._compiled.get(key)
        if ck is None:
            ck = codegen_ir.compile_kernel(self.py_func, args, ndim,
                                           fastmath=bool(self.options.get("fastmath", False)),
                                           index32=not self.options.get("gpu_use_64bit_index", True))
            self._compiled[key] = ck
        fast_key = tuple([a.call_sig if type(a) is DeviceArray else type(a) for a in args])
        first = next(i for i, a in enumerate(args) if isinstance(a, DeviceArray))
        self._launchers[(fast_key, ndim)] = (ck, first)
        queue = args[first].queue
        kernel = ck.handle_on(queue)
        if self.local_size:
            local = tuple(self.local_size)
        else:
            local = ck.block_size_on(queue, kernel, tuple(self.global_size))
        grid = tuple((g + l - 1) // l for g, l in zip(self.global_size, local))
        if any(g == 0 for g in self.global_size):
            return
        # pointers, shapes and scalars go from the argument objects into the
        # GPUParamDesc array in the native launch path
        tail = tuple(self.global_size) + (1,) * (3 - ndim)
        if ck.local_bytes:
            tail += (-ck.local_bytes,)
        try:
            _rt.fastcall().launch_kernel(queue.handle, kernel, grid, local, ck.layout_code(), args, tail)
        except RuntimeError:
            _rt.check()
            raise


def kernel(func=None, **kwargs):
    if func is None:
        def wrapper(f):
            return Kernel(f, kwargs)

        return wrapper
    return Kernel(func, kwargs)


def kernel_func(func=None, **kwargs):
    """Device function callable from kernels: inlined into the caller at the IR
    level, like the reference's force-inlined njit (kernel_impl.py:211)."""
    import numba

    if func is None:
        return lambda f: numba.njit(inline="always")(f)
    return numba.njit(inline="always")(func)
