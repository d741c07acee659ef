"""`njit` / `jit` / `vectorize` / `njit_replace_parfors` for the CUDA offload path.

Same names and call forms as numba_mlir/numba_mlir/decorators.py:25-107.  In the
reference, offload is selected by argument type: a function compiled by `njit`
goes to the GPU when its array arguments are device (USM) arrays
(numba_mlir/mlir/dpctl_interop.py:210-234).  Here device arrays are
`DeviceArray`s (anything exposing `__cuda_array_interface__` is accepted and
wrapped).  There is no CPU path in this package: calling a decorated function
without any device array raises instead of silently running on the host.
"""

import functools

import numpy as np

from . import lazy
from . import runtime as _rt
from .device_array import DeviceArray, as_device_array

# Keyword options accepted for compatibility (numba_mlir/mlir/target.py:176-203):
# parallel, fastmath, gpu_fp64_truncate, gpu_use_64bit_index,
# enable_gpu_pipeline, mlir_force_inline, mlir_vectorize, cache, inline,
# boundscheck, nogil, locals, nopython, forceobj.  B200 has native fp64, so
# gpu_fp64_truncate has nothing to do.  gpu_use_64bit_index=False makes the
# index arithmetic of `prange` and `@kernel` code 32-bit (codegen_ir.index_like_vars).


def _wrap_arg(a):
    if isinstance(a, DeviceArray):
        return a
    if hasattr(a, "__cuda_array_interface__"):
        return as_device_array(a)
    return a


def check_device_args(args):
    """All device arrays of one call must live on one device
    (check_usm_ndarray_args, numba_mlir/mlir/dpctl_interop.py:270-275)."""
    devs = {a.queue.device for a in args if isinstance(a, DeviceArray)}
    if len(devs) > 1:
        raise ValueError(f"Device arrays have different devices: {sorted(devs)}")
    return devs


def parfor_launch_shape(extents, inner_parallel, sms=148):
    """Launch shape of a prange kernel from the trip counts the host knows
    (None = unknown) and the device's multiprocessor count.  Returns
    (None, None) for an empty loop."""
    def ceil_div(a, b):
        return (a + b - 1) // b

    # the loops are grid-strided: more blocks than this only add launch cost
    _MAX_PARFOR_BLOCKS = sms * 32

    n = extents[0]
    if n == 0:
        return None, None
    if not inner_parallel:
        blocks = sms * 8 if n is None else min(ceil_div(n, 256), _MAX_PARFOR_BLOCKS)
        return (blocks,), (256,)
    m = extents[1]
    if m == 0:
        return None, None
    bx = 32 if m is None else min(256, 1 << max(0, (m - 1).bit_length()))
    by = 256 // bx
    gx = 8 if m is None else min(ceil_div(m, bx), 1024)
    gy = sms if n is None else ceil_div(n, by)
    gy = max(1, min(gy, _MAX_PARFOR_BLOCKS // gx, 65535))
    return (gx, gy), (bx, by)


class Dispatcher:
    """Callable returned by `njit`: traces the function on its first call per
    argument signature, then replays the recorded launches."""

    def __init__(self, py_func, options):
        functools.update_wrapper(self, py_func)
        self.py_func = py_func
        self.options = dict(options)
        self._plans = {}
        self._native_plans = {}
        self._parfor = None
        self._parfor_kernels = {}
        self._split = True if options.get("split_parfors") else None
        self._split_func = None

    def __call__(self, *args, **kwargs):
        if kwargs:
            raise TypeError("keyword arguments are not supported in offloaded calls")
        if self._native_plans and lazy.current_trace() is None:
            # a call seen before whose plan is launches over its own arguments: the
            # key, the pointers and the launches are all handled natively
            key = _rt.fastcall().signature(args, DeviceArray)
            if key is not None:
                plan = self._native_plans.get(key)
                if plan is not None:
                    return plan.replay_native(args, next(a for a in args if type(a) is DeviceArray).queue)
        if lazy.current_trace() is not None:
            # called from another offloaded function that is being traced: the
            # body joins the caller's trace (the reference inlines nested njit
            # calls into one module, mlir/tests/test_gpu.py:1673-1702)
            from . import codegen_ir

            if codegen_ir.uses_prange(self.py_func):
                return self._call_parfor_in_trace(lazy.current_trace(), args)
            return lazy.with_device_creators(self.py_func)(*args)
        args = tuple(_wrap_arg(a) for a in args)
        devs = check_device_args(args)
        if not devs:
            raise TypeError(
                f"{self.py_func.__name__}: no device array among the arguments; this package "
                "only implements the GPU offload path (there is no CPU fallback) -- copy the "
                "inputs with numba_mlir_b200.from_host first"
            )
        for a in args:
            if isinstance(a, np.ndarray):
                raise TypeError("host NumPy arrays cannot be mixed with device arrays")
        if self._parfor is None:
            from . import codegen_ir

            self._parfor = codegen_ir.uses_prange(self.py_func)
        if self._parfor:
            from . import codegen_ir, parfor_split

            if self._split is None:
                self._split = parfor_split.count_outer_prange_loops(self.py_func) > 1
            if not self._split:
                try:
                    return self._call_parfor(args)
                except codegen_ir.UnsupportedError:
                    # loops mixed with array expressions or host-side code: cut the
                    # loops out and run the rest as a traced function
                    if parfor_split.count_outer_prange_loops(self.py_func) < 1:
                        raise
                    self._split = True
            return self._call_split(args)
        key = lazy.signature_of(args)
        plan = self._plans.get(key) if key is not None else None
        queue = next(a.queue for a in args if isinstance(a, DeviceArray))
        if plan is not None:
            return plan.replay(args, queue)
        result, plan = lazy.trace_call(self.py_func, args, queue,
                                        fastmath=bool(self.options.get("fastmath", False)))
        if plan is not None and key is not None:
            self._plans[key] = plan
            if plan.native_ok:
                self._native_plans[key] = plan
        return result

    def _call_parfor(self, args):
        """Functions written as `prange` loop nests are compiled as a whole:
        the outermost parallel loop becomes the grid
        (numba_mlir/mlir/tests/test_gpu.py:1523-1613)."""
        from . import codegen_ir, kernel_impl

        key = kernel_impl.call_signature(args)
        ck = self._parfor_kernels.get(key)
        if ck is None:
            ck = codegen_ir.compile_parfor(self.py_func, args,
                                           fastmath=bool(self.options.get("fastmath", False)),
                                           index32=not self.options.get("gpu_use_64bit_index", True))
            self._parfor_kernels[key] = ck
        queue = next(a.queue for a in args if isinstance(a, DeviceArray))
        kernel = ck.handle_on(queue)
        grid, block = parfor_launch_shape(ck.extents(args), ck.inner_parallel, queue.sm_count)
        values = kernel_impl.marshal_values(args, ck.param_layout)
        if ck.epilogue is None:
            if grid is not None:
                queue.launch_values(kernel, grid, block, ck.kinds(), values)
            return None
        # Reductions, code after the loop, a scalar result: the kernel needs room
        # for one partial per block and reduction, a ticket and the result cell;
        # an empty loop still runs (one block) for what follows it.
        if grid is None:
            grid, block = (1,), (256,)
        counters, data = queue.scratch(ck.epilogue * grid[0] + 16)
        ret = data + ck.epilogue * grid[0]
        ret += -ret % 8
        queue.launch_values(kernel, grid, block, ck.kinds() + ("ptr", "ptr", "ptr"), values + [data, counters, ret])
        if ck.return_dtype is None:
            return None
        host = np.zeros(1, ck.return_dtype)
        queue.memcpy(host.ctypes.data, ret, host.nbytes, _rt.COPY_D2H, wait=True)
        return host[0]

    def _call_split(self, args):
        """Several parallel loops, or loops next to array expressions: every
        outermost `prange` loop is its own kernel, the code between them runs
        here on the host (mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940
        makes one `gpu.launch` per loop nest)."""
        from . import parfor_split

        if self._split_func is None:
            opts = {k: v for k, v in self.options.items() if k != "split_parfors"}
            try:
                self._split_func, _n = parfor_split.split(self.py_func, lambda f: Dispatcher(f, opts))
            except parfor_split.SplitError as e:
                raise TypeError(str(e)) from None
        queue = next(a.queue for a in args if isinstance(a, DeviceArray))
        key = lazy.signature_of(args)
        plan = self._plans.get(key) if key is not None else None
        if plan is not None:
            return plan.replay(args, queue)
        result, plan = lazy.trace_call(self._split_func, args, queue,
                                       fastmath=bool(self.options.get("fastmath", False)))
        if plan is not None and key is not None:
            # loops that hand no scalar back to the host code are steps of the
            # plan like the kernels of the array expressions around them
            self._plans[key] = plan
        return result

    def _call_parfor_in_trace(self, trace, args):
        """A loop function called while an array-expression function is being
        traced: its operands are evaluated, the loop's kernel is launched, and
        its scalar result (if any) comes back as a host value."""
        if trace.dry:
            raise TypeError("prange loops cannot be traced without a device")
        real, specs, replayable = [], [], True
        for a in args:
            if isinstance(a, lazy.LazyArray):
                if a.shape == () and a.concrete is not None and a.node.kind != "leaf":
                    real.append(a.concrete)
                    if a.node.kind == "arg":
                        specs.append(("arg", a.node.value))   # a scalar argument of the call
                    elif a.node.kind == "const":
                        specs.append(("const", a.concrete))
                    else:
                        replayable = False                     # computed from argument values
                    continue
                slot = trace.materialize(a)
                arr = trace.arrays[slot]
                if a.shape == ():
                    real.append(arr.copy_to_host()[()])  # a device scalar: the loop takes its value
                    replayable = False
                else:
                    trace.before_direct_write(slot)  # the loop may write it
                    real.append(arr)
                    specs.append(("slot", slot))
            else:
                real.append(a)
                specs.append(("const", a))  # a shape or a literal: fixed for this signature
        trace.flush()
        if not any(isinstance(a, DeviceArray) for a in real):
            raise TypeError(f"{self.py_func.__name__}: a prange loop needs at least one device array")
        result = self._call_parfor(tuple(real))
        if result is not None or not replayable:
            trace.value_dependent = True  # a scalar goes back to the host code: no replayable plan
        else:
            trace.steps.append(("parfor", self, tuple(specs)))
        return result

    def trace_dry(self, *args):
        """Records the plan and generates the kernels without a device (used
        by host-side tests of the code generator)."""
        return lazy.trace_call(self.py_func, args, None, dry=True,
                               fastmath=bool(self.options.get("fastmath", False)))


def jit(signature_or_function=None, locals={}, cache=False, pipeline_class=None,
        boundscheck=False, **options):
    """Same call forms as mlir_jit (decorators.py:25-66)."""
    if callable(signature_or_function) and not isinstance(signature_or_function, (str, tuple, list)):
        return Dispatcher(signature_or_function, options)

    def wrapper(func):
        return Dispatcher(func, options)

    return wrapper


def njit(*args, **kws):
    """Equivalent to jit(nopython=True) (mlir_njit, decorators.py:69-81)."""
    kws.pop("forceobj", None)
    kws["nopython"] = True
    return jit(*args, **kws)


def njit_replace_parfors(*args, **kws):
    """Only the parallel loops are offloaded; the code around them stays with
    the host (mlir_njit_replace_parfors, decorators.py:84-104, where Numba
    keeps control and numba_mlir/mlir/passes.py:332-416 hands each parfor to the
    MLIR pipeline).  Every outermost `prange` loop of the function becomes its
    own kernel and the rest of the body runs on the host around them, whatever
    the number of loops; functions without loops behave as under `njit`."""
    kws["split_parfors"] = True
    return njit(*args, **kws)


class Vectorized:
    """Result of `vectorize`: a scalar Python function usable as an
    elementwise operation on device arrays (mlir_vectorize,
    numba_mlir/mlir/vectorize.py:45-70)."""

    def __init__(self, py_func, options):
        functools.update_wrapper(self, py_func)
        self.py_func = py_func
        self.options = options
        self._funcs = {}

    def _device_func(self, dtypes):
        fn = self._funcs.get(dtypes)
        if fn is None:
            from . import codegen_ir

            fn = codegen_ir.compile_device_function(self.py_func, dtypes)
            self._funcs[dtypes] = fn
        return fn

    def __call__(self, *args):
        trace = lazy.current_trace()
        if trace is None:
            args = tuple(_wrap_arg(a) for a in args)
            if not any(isinstance(a, DeviceArray) for a in args):
                raise TypeError("vectorize: no device array among the arguments (no CPU fallback)")
            return Dispatcher(lambda *xs: self(*xs), {})(*args)
        dtypes = []
        for a in args:
            if isinstance(a, lazy.LazyArray):
                dtypes.append(a.dtype)
            elif isinstance(a, DeviceArray):
                dtypes.append(a.dtype)
            else:
                dtypes.append(lazy.scalar_dtype(a))
        return lazy.call_device_func(trace, self._device_func(tuple(dtypes)), args)


def vectorize(*args, **kwargs):
    if len(args) == 1 and callable(args[0]) and not kwargs:
        return Vectorized(args[0], {})

    def wrapper(func):
        return Vectorized(func, kwargs)

    return wrapper
