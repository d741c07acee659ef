"""Array-expression front-end: NumPy expressions on device arrays -> fused kernels.

What the reference does with MLIR -- turn every NumPy call into a
`linalg.generic`, fuse the chain into one loop nest
(numba_mlir/mlir_compiler/lib/pipelines/PlierToLinalg.cpp:4439-4587; the
Black-Scholes test asserts one `scf.parallel`,
numba_mlir/mlir/tests/test_numpy.py:2796-2866) and outline it as one GPU
kernel -- is done here by recording the expression graph while the Python
function runs on symbolic arrays and emitting ONE CUDA kernel per group of
same-shaped results.  The kernel is an instance of the hand-written vectorised
loop `nmb::eltwise_tile` (csrc/kernels/nmb_device.cuh) around a generated
per-element body, compiled by NVRTC inside gpuxModuleLoad and launched through
gpuxLaunchKernel.

Typing follows Numba, like the reference (which reuses Numba's type inference):
ufunc loops are chosen by `numba.np.numpy_support.ufunc_find_matching_loop`,
Python floats are float64 and Python ints int64.

A traced call is recorded as a Plan (allocations + launches with argument
slots) and cached per argument signature, the analogue of the per-function
context in which the reference caches queue/module/kernel handles
(numba_mlir/mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940).
"""

import itertools
import re
import struct
import threading
import weakref

import numpy as np

from .device_array import DeviceArray, empty

# ----------------------------------------------------------------- dtypes ---
_CTYPE = {
    "float32": "float", "float64": "double", "int8": "int8_t", "int16": "int16_t",
    "int32": "int32_t", "int64": "int64_t", "uint8": "uint8_t", "uint16": "uint16_t",
    "uint32": "uint32_t", "uint64": "uint64_t", "bool": "bool",
}


def ctype(dtype):
    try:
        return _CTYPE[np.dtype(dtype).name]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported on the device") from None


def literal(value, dtype):
    """Exact C literal of a NumPy scalar."""
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        bits = struct.unpack("<I", struct.pack("<f", float(value)))[0]
        return f"__uint_as_float(0x{bits:08x}u)"
    if dtype == np.float64:
        bits = struct.unpack("<q", struct.pack("<d", float(value)))[0]
        return f"__longlong_as_double({bits}ll)" if bits >= 0 else f"__longlong_as_double((long long)0x{bits & (2**64 - 1):016x}ull)"
    if dtype == np.bool_:
        return "true" if value else "false"
    if dtype.kind == "u":
        return f"({ctype(dtype)}){int(value)}ull"
    return f"({ctype(dtype)}){int(value)}ll"


def scalar_dtype(value):
    """Numba's typing of Python scalars: float -> float64, int -> int64."""
    if isinstance(value, (bool, np.bool_)):
        return np.dtype(np.bool_)
    if isinstance(value, np.generic):
        return value.dtype
    if isinstance(value, int):
        return np.dtype(np.int64)
    if isinstance(value, float):
        return np.dtype(np.float64)
    raise TypeError(f"unsupported scalar {type(value)}")


_loop_cache = {}


def find_loop(ufunc, in_dtypes):
    """(loop input dtypes, output dtype) chosen the way Numba chooses."""
    key = (ufunc, tuple(in_dtypes))
    hit = _loop_cache.get(key)
    if hit is None:
        from numba.np import numpy_support as ns

        loop = ns.ufunc_find_matching_loop(ufunc, tuple(ns.from_dtype(d) for d in in_dtypes))
        if loop is None:
            raise TypeError(f"no {ufunc.__name__} loop for {in_dtypes}")
        hit = ([ns.as_dtype(t) for t in loop.inputs], ns.as_dtype(loop.outputs[0]))
        _loop_cache[key] = hit
    return hit


# ------------------------------------------------------------------- ops ----
def _flt(f32, f64):
    return lambda dt, *a: (f32 if dt == np.float32 else f64).format(*a)


def _int_or_float(int_expr, f32, f64):
    def emit(dt, *a):
        if dt.kind in "iub":
            return int_expr.format(*a)
        return (f32 if dt == np.float32 else f64).format(*a)

    return emit


# name -> (numpy ufunc, emitter(loop_dtype, *operand exprs))
UFUNCS = {
    "add": (np.add, lambda dt, a, b: f"({a} + {b})"),
    "subtract": (np.subtract, lambda dt, a, b: f"({a} - {b})"),
    "multiply": (np.multiply, lambda dt, a, b: f"({a} * {b})"),
    "true_divide": (np.true_divide, lambda dt, a, b: f"nmb::f_div({a}, {b})"),
    "negative": (np.negative, lambda dt, a: f"(-{a})"),
    "positive": (np.positive, lambda dt, a: f"({a})"),
    "absolute": (np.absolute, _int_or_float("nmb::i_abs({0})", "fabsf({0})", "fabs({0})")),
    "sqrt": (np.sqrt, lambda dt, a: f"nmb::f_sqrt({a})"),
    "log": (np.log, lambda dt, a: f"nmb::f_log({a})"),
    "exp": (np.exp, lambda dt, a: f"nmb::f_exp({a})"),
    "sin": (np.sin, _flt("sinf({0})", "sin({0})")),
    "cos": (np.cos, _flt("cosf({0})", "cos({0})")),
    "tan": (np.tan, _flt("tanf({0})", "tan({0})")),
    "tanh": (np.tanh, _flt("tanhf({0})", "tanh({0})")),
    "arctan2": (np.arctan2, _flt("atan2f({0}, {1})", "atan2({0}, {1})")),
    "arccos": (np.arccos, _flt("acosf({0})", "acos({0})")),
    "floor": (np.floor, _flt("floorf({0})", "floor({0})")),
    "ceil": (np.ceil, _flt("ceilf({0})", "ceil({0})")),
    "square": (np.square, lambda dt, a: f"({a} * {a})"),
    "power": (np.power, _int_or_float("nmb::i_pow({0}, {1})", "powf({0}, {1})", "pow({0}, {1})")),
    "maximum": (np.maximum, lambda dt, a, b: f"nmb::np_max({a}, {b})"),
    "minimum": (np.minimum, lambda dt, a, b: f"nmb::np_min({a}, {b})"),
    "less": (np.less, lambda dt, a, b: f"({a} < {b})"),
    "less_equal": (np.less_equal, lambda dt, a, b: f"({a} <= {b})"),
    "greater": (np.greater, lambda dt, a, b: f"({a} > {b})"),
    "greater_equal": (np.greater_equal, lambda dt, a, b: f"({a} >= {b})"),
    "equal": (np.equal, lambda dt, a, b: f"({a} == {b})"),
    "not_equal": (np.not_equal, lambda dt, a, b: f"({a} != {b})"),
    "logical_and": (np.logical_and, lambda dt, a, b: f"(({a} != 0) && ({b} != 0))"),
    "logical_or": (np.logical_or, lambda dt, a, b: f"(({a} != 0) || ({b} != 0))"),
    "logical_not": (np.logical_not, lambda dt, a: f"(!({a} != 0))"),
    "logical_xor": (np.logical_xor, lambda dt, a, b: f"(({a} != 0) != ({b} != 0))"),
    "floor_divide": (np.floor_divide, lambda dt, a, b: f"nmb::py_floordiv({a}, {b})"),
    "remainder": (np.remainder, lambda dt, a, b: f"nmb::py_mod({a}, {b})"),
    "bitwise_and": (np.bitwise_and, lambda dt, a, b: f"({a} & {b})"),
    "bitwise_or": (np.bitwise_or, lambda dt, a, b: f"({a} | {b})"),
    "bitwise_xor": (np.bitwise_xor, lambda dt, a, b: f"({a} ^ {b})"),
    "invert": (np.invert, lambda dt, a: f"(!{a})" if dt == np.bool_ else f"(~{a})"),
    "left_shift": (np.left_shift, lambda dt, a, b: f"nmb::i_shl({a}, {b})"),
    "right_shift": (np.right_shift, lambda dt, a, b: f"nmb::i_shr({a}, {b})"),
    "isnan": (np.isnan, lambda dt, a: f"({a} != {a})"),
    "isinf": (np.isinf, _flt("isinf({0})", "isinf({0})")),
    "isfinite": (np.isfinite, _flt("isfinite({0})", "isfinite({0})")),
    "sign": (np.sign, _int_or_float("nmb::i_sign({0})", "nmb::f_sign({0})", "nmb::f_sign({0})")),
    "reciprocal": (np.reciprocal, _int_or_float("(1 / {0})", "nmb::f_div(1.0f, {0})", "nmb::f_div(1.0, {0})")),
    "arcsin": (np.arcsin, _flt("asinf({0})", "asin({0})")),
    "arctan": (np.arctan, _flt("atanf({0})", "atan({0})")),
    "sinh": (np.sinh, _flt("sinhf({0})", "sinh({0})")),
    "cosh": (np.cosh, _flt("coshf({0})", "cosh({0})")),
    "expm1": (np.expm1, _flt("expm1f({0})", "expm1({0})")),
    "log1p": (np.log1p, _flt("log1pf({0})", "log1p({0})")),
    "log2": (np.log2, _flt("log2f({0})", "log2({0})")),
    "log10": (np.log10, _flt("log10f({0})", "log10({0})")),
    "rint": (np.rint, _flt("rintf({0})", "rint({0})")),
    "trunc": (np.trunc, _flt("truncf({0})", "trunc({0})")),
    "fmod": (np.fmod, _int_or_float("({1} == 0 ? 0 : {0} % {1})", "fmodf({0}, {1})", "fmod({0}, {1})")),
    "hypot": (np.hypot, _flt("hypotf({0}, {1})", "hypot({0}, {1})")),
    "exp2": (np.exp2, _flt("exp2f({0})", "exp2({0})")),
    "cbrt": (np.cbrt, _flt("cbrtf({0})", "cbrt({0})")),
    "degrees": (np.degrees, _flt("({0} * 57.29577951308232f)", "({0} * 57.29577951308232)")),
    "radians": (np.radians, _flt("({0} * 0.017453292519943295f)", "({0} * 0.017453292519943295)")),
}
_UFUNC_BY_OBJ = {u: name for name, (u, _e) in UFUNCS.items()}
_UFUNC_BY_OBJ[np.divide] = "true_divide"
_UFUNC_BY_OBJ[np.abs] = "absolute"
_UFUNC_BY_OBJ[np.mod] = "remainder"
_UFUNC_BY_OBJ[np.rad2deg] = "degrees"
_UFUNC_BY_OBJ[np.deg2rad] = "radians"
_UFUNC_BY_OBJ[np.bitwise_not] = "invert"

# 1/sqrt(x) under fastmath (never produced by NumPy dispatch)
UFUNCS["rsqrt"] = (None, _flt("nmb::f_rsqrt({0})", "(1.0 / sqrt({0}))"))

REDUCTIONS = {np.sum: "sum", np.prod: "prod", np.min: "min", np.max: "max", np.amin: "min",
              np.amax: "max", np.argmin: "argmin", np.argmax: "argmax"}


# ------------------------------------------------------------------ nodes ---
class Node:
    """Expression-graph node.  kind: 'leaf' (device array), 'arg' (scalar
    argument, a kernel parameter), 'const' (literal), 'op' (ufunc), 'cast',
    'where', 'call' (user scalar device function): these make up fused
    elementwise kernels.  'reduce' (op = the reduction, value = the axis),
    'dot' (matrix product) and 'reshape' (C-order reshape of a value that is
    not an array yet) are turned into arrays when a flush reaches them
    (Trace.lower), or, where a whole pattern is recognised, into one launch.
    `borrowed` marks a leaf that stands for an array of the caller into which
    the node's value was written directly."""

    __slots__ = ("kind", "dtype", "shape", "inputs", "op", "value", "slot", "sig", "reads", "borrowed")

    def __init__(self, kind, dtype, shape, inputs=(), op=None, value=None, slot=None):
        self.kind = kind
        self.dtype = np.dtype(dtype)
        self.shape = tuple(shape)
        self.inputs = tuple(inputs)
        self.op = op
        self.value = value
        self.slot = slot
        self.sig = None
        self.reads = None
        self.borrowed = False

    def become_leaf(self, slot, borrowed=False):
        """The node's value now lives in the array of `slot`."""
        self.kind = "leaf"
        self.slot = slot
        self.inputs = ()
        self.op = None
        self.value = None
        self.reads = None
        self.sig = None
        self.borrowed = borrowed


def node_reads(node):
    """Slots of the device arrays an expression reads."""
    r = node.reads
    if r is None:
        if node.kind == "leaf":
            r = frozenset((node.slot,))
        elif node.inputs:
            r = frozenset().union(*[node_reads(i) for i in node.inputs])
        else:
            r = frozenset()
        node.reads = r
    return r


def _extent(arr):
    """Byte range [lo, hi) that a strided view can touch."""
    return arr.extent


def broadcast_shapes(*shapes):
    return np.broadcast_shapes(*shapes)


class DeviceFunc:
    """Scalar function compiled to a CUDA __device__ function and usable as an
    elementwise operation (what @vectorize of a scalar body gives the
    reference, numba_mlir/mlir/vectorize.py:45-70)."""

    def __init__(self, name, source, arg_dtypes, ret_dtype, pair=None):
        self.name = name
        self.source = source
        self.arg_dtypes = tuple(np.dtype(d) for d in arg_dtypes)
        self.ret_dtype = np.dtype(ret_dtype)
        # name of the nmb_device.cuh routine that computes the function for two
        # float32 values at once, when the body is nothing but that function
        self.pair = pair


# ---------------------------------------------------------------- tracing ---
class Trace:
    """State of one traced call: slot table, pending stores, recorded steps."""

    def __init__(self, queue, args=None, dry=False, fastmath=False):
        self.queue = queue
        self.dry = dry  # record and generate code only (no device)
        self.fastmath = fastmath  # relaxed division/sqrt and a*b+c contraction
        self.slots = []          # slot -> ("arg", index, views) | ("tmp", shape, dtype, views)
        self.arrays = []         # slot -> DeviceArray (this call's binding)
        self.pending = []        # [(target LazyArray leaf, value Node)]
        self.steps = []
        self.value_dependent = False
        self.args = args
        self.live = []           # weak references to the unevaluated expressions
        self._extents = {}

    # aliasing --------------------------------------------------------------------
    # Expressions are evaluated late (at the next flush), stores are queued: the
    # order of reads and writes the program wrote is kept by three rules.  (1) An
    # expression that reads memory a queued store will write is built only after
    # that store has been emitted.  (2) Before a store is queued, every unevaluated
    # expression still reachable from the program that reads the store's memory is
    # given a temporary of its own, evaluated no later than the store.  (3) Within
    # one fused kernel an output may share memory with an input only element for
    # element (each thread reads its elements before it writes them); anything
    # else is split over consecutive kernels, through a temporary where a store's
    # own value reads other elements of its target (NumPy copies on overlap).
    def overlap(self, s1, s2):
        """0: the two arrays share no memory; 1: they are the same elements in
        the same order; 2: they overlap in some other way."""
        if s1 == s2:
            return 1
        a, b = self.arrays[s1], self.arrays[s2]
        ea, eb = self._extents.get(s1), self._extents.get(s2)
        if ea is None:
            ea = self._extents[s1] = _extent(a)
        if eb is None:
            eb = self._extents[s2] = _extent(b)
        if ea[0] >= eb[1] or eb[0] >= ea[1]:
            return 0
        if a.ptr == b.ptr and a.shape == b.shape and a.strides == b.strides and a.dtype == b.dtype:
            return 1
        return 2

    def pending_touches(self, slot, reads_too=False):
        """A queued store writes (or, with `reads_too`, its value reads) memory of `slot`."""
        for s, node in self.pending:
            if self.overlap(s, slot):
                return True
            if reads_too and any(self.overlap(r, slot) for r in node_reads(node)):
                return True
        return False

    def detach_readers(self, slot, value=None):
        """Rule (2): expressions that read the memory of `slot` and can still be
        used later get their values stored into temporaries, queued before
        whatever writes `slot` next.  `value` is the expression being stored
        into `slot` itself."""
        if not self.live:
            return
        alive = []
        for ref in self.live:
            lz = ref()
            if lz is None or (lz.node.kind == "leaf" and not lz.node.borrowed):
                continue
            alive.append(ref)
            if lz is value:
                continue
            if any(self.overlap(r, slot) for r in node_reads(lz.node)):
                tmp = self.add_tmp_slot(lz.node.shape, lz.node.dtype)
                self.pending.append((tmp, lz.node))
                lz.node = Node("leaf", lz.node.dtype, lz.node.shape, slot=tmp)
        self.live = alive

    def before_direct_write(self, slot):
        """A step that writes `slot` as soon as it is recorded (a reduction or a
        contraction into an existing array) comes after everything queued that
        reads or writes that memory."""
        self.detach_readers(slot)
        if self.pending_touches(slot, reads_too=True):
            self.flush()

    # slots ---------------------------------------------------------------------
    # slot -> ("arg", index) | ("tmp", shape, dtype) | ("view", base slot, op)
    #         | ("captured",)
    def add_arg_slot(self, index, array):
        self.slots.append(("arg", index) if index is not None else ("captured",))
        self.arrays.append(array)
        return len(self.slots) - 1

    def add_tmp_slot(self, shape, dtype):
        if self.dry:
            arr = fake_array(shape, dtype)
        else:
            arr = empty(shape, dtype, queue=self.queue)
        self.slots.append(("tmp", tuple(shape), np.dtype(dtype)))
        self.arrays.append(arr)
        self.steps.append(("alloc", len(self.slots) - 1))
        return len(self.slots) - 1

    def add_view_slot(self, base_slot, view_op, array):
        self.slots.append(("view", base_slot, view_op))
        self.arrays.append(array)
        return len(self.slots) - 1

    def leaf(self, slot):
        arr = self.arrays[slot]
        return LazyArray(self, Node("leaf", arr.dtype, arr.shape, slot=slot))

    def has_pending(self, slot):
        return any(self.overlap(s, slot) for s, _ in self.pending)

    # stores ----------------------------------------------------------------------
    def store(self, target_slot, node, value=None):
        self.detach_readers(target_slot, value)
        self.pending.append((target_slot, node))

    def flush(self):
        """Emits the pending stores in order: one fused kernel per output shape
        for every run of stores that rule (3) allows in one kernel.  Reductions
        and matrix products inside the stored values are run first (each into
        a temporary, or straight into the store's target when it is the whole
        value and the target's layout allows)."""
        queue, self.pending = self.pending, []
        batch, reads, writes = [], set(), set()

        def emit():
            groups = {}
            for slot, node in batch:
                groups.setdefault(self.arrays[slot].shape, []).append((slot, node))
            for shape, outs in groups.items():
                _emit_eltwise(self, shape, outs)
            batch.clear()
            reads.clear()
            writes.clear()

        i = 0
        while i < len(queue):
            slot, node = queue[i]
            i += 1
            if self._store_direct(slot, node, emit):
                continue
            self.lower(node)
            nreads = node_reads(node)
            if any(self.overlap(r, slot) == 2 for r in nreads):
                # the value reads other elements of the target than it writes
                tmp = self.add_tmp_slot(node.shape, node.dtype)
                queue.insert(i, (slot, Node("leaf", node.dtype, node.shape, slot=tmp)))
                slot = tmp
            if batch and (any(self.overlap(r, slot) == 2 for r in reads)
                          or any(self.overlap(w, slot) == 2 for w in writes)
                          or any(self.overlap(r, w) for r in nreads for w in writes)):
                emit()
            batch.append((slot, node))
            reads |= nreads
            writes.add(slot)
        emit()

    # lowering --------------------------------------------------------------------
    # Steps emitted here run at once, ahead of the elementwise stores still
    # batched by the flush in progress.  That is their program order: by rule (1)
    # no value reads memory that an earlier queued store writes, and the steps
    # themselves write only fresh temporaries (a direct store into the target
    # first emits the batch).
    def lower(self, node):
        """Turns every reduction, product and reshape inside `node` into a leaf."""
        kind = node.kind
        if kind in ("leaf", "arg", "const"):
            return
        if kind == "reduce":
            self._lower_reduce(node, None)
        elif kind == "dot":
            self._lower_dot(node, None)
        elif kind == "reshape":
            src = self.force(node.inputs[0])
            arr = self.arrays[src].reshape(node.shape)
            node.become_leaf(self.add_view_slot(src, ("reshape", node.shape), arr))
        else:
            spec = _match_rowcol(self, node)
            if spec is not None:
                self._lower_rowcol(node, spec, None)
                return
            for inp in node.inputs:
                self.lower(inp)

    def force(self, node):
        """Slot of an array that holds the value of `node`."""
        self.lower(node)
        if node.kind == "leaf":
            return node.slot
        if node.kind in ("arg", "const"):
            raise TypeError("a scalar was used where an array is needed")
        tmp = self.add_tmp_slot(node.shape, node.dtype)
        _emit_eltwise(self, node.shape, [(tmp, node)])
        node.become_leaf(tmp)
        return tmp

    def _lower_reduce(self, node, dst):
        from . import reduce_ops

        op, axis = node.op, node.value
        borrowed = dst is not None
        self.lower(node.inputs[0])
        mode = fused_reduce_mode(node)
        if mode is not None:
            # the operand is an elementwise chain: reduced while it is computed
            out = dst if dst is not None else self.add_tmp_slot(node.shape, node.dtype)
            if _emit_reduce_fused(self, node, mode, out):
                node.become_leaf(out, borrowed)
                return
            dst = out
        src = self.force(node.inputs[0])
        if dst is None:
            dst = self.add_tmp_slot(node.shape, node.dtype)
        self.steps.append(("reduce", op, axis, src, dst))
        if not self.dry:
            reduce_ops.reduce(self.arrays[src], op, axis, out=self.arrays[dst])
        node.become_leaf(dst, borrowed)

    def _lower_dot(self, node, dst):
        from . import contraction

        sa, sb = self.force(node.inputs[0]), self.force(node.inputs[1])
        dts = {self.arrays[s].dtype for s in (sa, sb)}
        if len(dts) != 1 or dts.pop() not in (np.float32, np.float64):
            raise TypeError("np.dot on device arrays takes two float32 or two float64 operands")
        borrowed = dst is not None
        if dst is None:
            dst = self.add_tmp_slot(node.shape, node.dtype)
        self.steps.append(("dot", sa, sb, dst))
        if not self.dry:
            contraction.gemm(self.arrays[sa], self.arrays[sb], self.arrays[dst], blocking=False)
        node.become_leaf(dst, borrowed)

    def _lower_rowcol(self, node, spec, dst):
        """One contraction launch for func(alpha * a @ b + row + col)."""
        from . import contraction

        alpha, dot_node, row, col, func = spec
        sa, sb = self.force(dot_node.inputs[0]), self.force(dot_node.inputs[1])

        def term(t, operand, transposed):
            if t is None:
                return None
            if _is_row_norms(self, t, operand, transposed):
                return "norms"
            s = self.force(t)
            if not self.arrays[s].is_c_contiguous:
                tmp = self.add_tmp_slot(self.arrays[s].shape, np.float32)
                _emit_eltwise(self, self.arrays[s].shape, [(tmp, Node("leaf", np.float32, self.arrays[s].shape, slot=s))])
                s = tmp
            return s

        rspec, cspec = term(row, sa, False), term(col, sb, True)
        borrowed = dst is not None
        if dst is None:
            dst = self.add_tmp_slot(node.shape, node.dtype)
        step = ("contract", sa, sb, float(alpha), rspec, cspec, func, dst)
        self.steps.append(step)
        if not self.dry:
            run_contract(step, self.arrays.__getitem__)
        node.become_leaf(dst, borrowed)

    def _store_direct(self, slot, node, emit):
        """A store whose whole value is a reduction, a product or a product with
        its epilogue writes the target itself when the layouts allow."""
        kind = node.kind
        spec = None
        if kind not in ("reduce", "dot"):
            red = _match_post_reduce(node)
            if red is not None:
                return self._store_post_reduce(slot, node, red, emit)
            spec = _match_rowcol(self, node)
            if spec is None:
                return False
        dst = self.arrays[slot]
        if dst.shape != node.shape or dst.dtype != node.dtype or dst.size == 0:
            return False
        if kind == "reduce":
            if not dst.is_c_contiguous:
                return False
        elif dst.ndim != 2 or (dst.strides[1] != dst.dtype.itemsize and dst.shape[1] > 1) or dst.strides[0] < 0:
            return False
        if any(self.overlap(r, slot) for r in node_reads(node)):
            return False
        emit()
        if kind == "reduce":
            self._lower_reduce(node, slot)
        elif kind == "dot":
            self._lower_dot(node, slot)
        else:
            self._lower_rowcol(node, spec, slot)
        return True

    def _store_post_reduce(self, slot, node, red, emit):
        """`target = g(reduce(f(inputs)))` with g elementwise over the reduced
        value alone: one generated reducer applies g on the way out."""
        dst = self.arrays[slot]
        if (dst.shape != node.shape or dst.dtype != node.dtype or dst.size == 0 or not dst.is_c_contiguous
                or any(self.overlap(r, slot) for r in node_reads(node))):
            return False
        self.lower(red.inputs[0])
        mode = fused_reduce_mode(red, leaf_ok=True)
        if mode is None:
            return False
        emit()
        if not _emit_reduce_fused(self, red, mode, slot, post=node):
            return False
        node.become_leaf(slot, borrowed=True)
        return True

    def materialize(self, lazy):
        """Device array (slot) holding the value of `lazy`."""
        node = lazy.node
        if node.kind == "leaf":
            if self.has_pending(node.slot):
                self.flush()
            return node.slot
        slot = self.add_tmp_slot(node.shape, node.dtype)
        self.store(slot, node)
        self.flush()
        if node.kind != "leaf":
            node.become_leaf(slot)  # later uses read the array instead of recomputing
        return node.slot


_tls = threading.local()


def current_trace():
    return getattr(_tls, "trace", None)


class _TraceScope:
    def __init__(self, trace):
        self.trace = trace

    def __enter__(self):
        self.prev = current_trace()
        _tls.trace = self.trace
        return self.trace

    def __exit__(self, *exc):
        _tls.trace = self.prev


def _as_node(trace, x):
    if isinstance(x, LazyArray):
        if x.node.kind == "leaf" and trace.pending and trace.has_pending(x.node.slot):
            trace.flush()  # the array is read after a recorded store to its memory
        return x.node
    if isinstance(x, DeviceArray):
        slot = trace.add_arg_slot(None, x)
        trace.value_dependent = True  # a captured array: not replayable
        return Node("leaf", x.dtype, x.shape, slot=slot)
    if isinstance(x, (bool, int, float, np.generic)):
        dt = scalar_dtype(x)
        return Node("const", dt, (), value=dt.type(x))
    if isinstance(x, np.ndarray) and x.dtype.name in _CTYPE:
        # a host array built inside the function (np.zeros, np.arange, ...):
        # uploaded for this call; like a captured device array it is not replayable
        from .device_array import from_host

        arr = fake_array(x.shape, x.dtype) if trace.dry else from_host(np.ascontiguousarray(x), queue=trace.queue)
        slot = trace.add_arg_slot(None, arr)
        trace.value_dependent = True
        return Node("leaf", arr.dtype, arr.shape, slot=slot)
    raise TypeError(f"cannot use {type(x)} in a device expression")


class LazyArray:
    """Symbolic array (or 0-d scalar) inside a traced function."""

    __array_priority__ = 1000

    def __init__(self, trace, node, concrete=None):
        self.trace = trace
        self.node = node
        self.concrete = concrete  # value of scalar arguments, for control flow
        if node.kind not in ("leaf", "arg", "const") and node_reads(node):
            trace.live.append(weakref.ref(self))  # an unevaluated expression over device memory

    # metadata ------------------------------------------------------------------
    @property
    def shape(self):
        return self.node.shape

    @property
    def dtype(self):
        return self.node.dtype

    @property
    def ndim(self):
        return len(self.node.shape)

    @property
    def size(self):
        return int(np.prod(self.node.shape, dtype=np.int64))

    @property
    def itemsize(self):
        return self.node.dtype.itemsize

    @property
    def nbytes(self):
        return self.size * self.node.dtype.itemsize

    @property
    def strides(self):
        """Byte strides (array.strides, numba_mlir/mlir/numpy/funcs.py): those
        of the device array for an argument or a view, C order for a value that
        is still an expression, which is how it is written out."""
        if self.node.kind == "leaf":
            return tuple(self.trace.arrays[self.node.slot].strides)
        out, step = [], self.node.dtype.itemsize
        for d in reversed(self.node.shape):
            out.append(step)
            step *= max(d, 1)
        return tuple(reversed(out))

    def __len__(self):
        return self.node.shape[0]

    # numpy protocols -------------------------------------------------------------
    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        out = kwargs.pop("out", None)
        if method != "__call__" or kwargs:
            return NotImplemented
        name = _UFUNC_BY_OBJ.get(ufunc)
        if name is None:
            raise TypeError(f"numpy.{ufunc.__name__} is not supported on device arrays")
        res = apply_ufunc(self.trace, name, inputs)
        if out is None:
            return res
        # np.add(a, b, c) / out=c: the value is stored into c, converted to its
        # type (numba_mlir/mlir/tests/test_numpy.py: test_binary_inplace)
        (target,) = out if isinstance(out, tuple) else (out,)
        if not isinstance(target, LazyArray):
            raise TypeError("out= must be a device array")
        target[...] = res
        return target

    def __array_function__(self, func, types, args, kwargs):
        if func in REDUCTIONS:
            return reduce_lazy(self.trace, REDUCTIONS[func], *args, **kwargs)
        if func is np.where and len(args) == 3:
            return where(self.trace, *args)
        if func is np.mean:
            return mean_lazy(self.trace, *args, **kwargs)
        if func in (np.var, np.std):
            v = var_lazy(self.trace, *args, **kwargs)
            return apply_ufunc(self.trace, "sqrt", (v,)) if func is np.std else v
        if func in (np.any, np.all, np.count_nonzero):
            return truth_reduce(self.trace, func, *args, **kwargs)
        if func is np.transpose and len(args) == 1 and not kwargs:
            return args[0].T
        if func is np.ravel and len(args) == 1:
            return args[0].ravel()
        if func is np.reshape:
            return args[0].reshape(*args[1:], **kwargs)
        if func is np.copy and len(args) == 1:
            return args[0].copy()
        if func in (np.ones_like, np.full_like):
            like = args[0]
            dt = np.dtype(kwargs.get("dtype") or like.dtype)
            out = self.trace.leaf(self.trace.add_tmp_slot(like.shape, dt))
            out[...] = dt.type(1) if func is np.ones_like else dt.type(args[1])
            return out
        if func is np.concatenate:
            return concatenate_lazy(self.trace, *args, **kwargs)
        if func is np.clip:
            return clip_lazy(self.trace, *args, **kwargs)
        if func is np.dot:
            return dot(self.trace, *args, **kwargs)
        if func in (np.empty_like, np.zeros_like):
            like = args[0]
            slot = self.trace.add_tmp_slot(like.shape, kwargs.get("dtype") or like.dtype)
            out = self.trace.leaf(slot)
            if func is np.zeros_like:
                out[...] = like.dtype.type(0)
            return out
        if func is np.shape:
            return self.shape
        if func is np.transpose and len(args) == 2 and not kwargs and args[1] is not None:
            a = args[0]
            axes = tuple(int(x) % a.ndim for x in args[1])
            if sorted(axes) != list(range(a.ndim)):
                raise ValueError("axes don't match array")
            return a._view(("transpose", axes), lambda x: _permuted(x, axes))
        if func is np.swapaxes and len(args) == 3 and not kwargs:
            a = args[0]
            axes = list(range(a.ndim))
            i, j = int(args[1]) % a.ndim, int(args[2]) % a.ndim
            axes[i], axes[j] = axes[j], axes[i]
            return a._view(("transpose", tuple(axes)), lambda x: _permuted(x, axes))
        if func is np.expand_dims and len(args) == 2 and not kwargs:
            a = args[0]
            new = args[1] if isinstance(args[1], (tuple, list)) else (args[1],)
            nd = a.ndim + len(new)
            new = {int(x) % nd for x in new}
            return a[tuple(None if d in new else slice(None) for d in range(nd))]
        if func is np.squeeze and len(args) == 1 and set(kwargs) <= {"axis"}:
            a = args[0]
            axis = kwargs.get("axis")
            drop = {d for d in range(a.ndim) if a.shape[d] == 1} if axis is None else \
                {int(x) % a.ndim for x in (axis if isinstance(axis, (tuple, list)) else (axis,))}
            if any(a.shape[d] != 1 for d in drop):
                raise ValueError("cannot select an axis to squeeze out which has size not equal to one")
            if not drop:
                return a
            return a._view(("getitem", tuple(0 if d in drop else slice(None) for d in range(a.ndim))),
                           lambda x: x[tuple(0 if d in drop else slice(None) for d in range(a.ndim))])
        if func is np.broadcast_to and len(args) == 2 and not kwargs:
            a = args[0]
            shape = tuple(int(d) for d in (args[1] if isinstance(args[1], (tuple, list)) else (args[1],)))
            if tuple(broadcast_shapes(a.shape, shape)) != shape:
                raise ValueError(f"cannot broadcast {a.shape} to {shape}")
            return a._view(("broadcast", shape), lambda x: _broadcast(x, shape))
        if func is np.atleast_2d and len(args) == 1 and not kwargs:
            a = args[0]
            if a.ndim >= 2:
                return a
            return a.reshape((1, a.shape[0]) if a.ndim else (1, 1))
        if func in _STACKS:
            return stack_lazy(self.trace, _STACKS[func], *args, **kwargs)
        if func is np.flip:
            return flip_lazy(self.trace, *args, **kwargs)
        if func is np.outer and len(args) == 2 and not kwargs:
            return outer_lazy(self.trace, *args)
        if func in (np.tril, np.triu):
            return triangle_lazy(self.trace, func is np.tril, *args, **kwargs)
        if func is np.cov:
            return cov_lazy(self.trace, *args, **kwargs)
        raise TypeError(f"numpy.{func.__name__} is not supported on device arrays")

    # operators -------------------------------------------------------------------
    def _bin(self, name, other, swap=False):
        return apply_ufunc(self.trace, name, (other, self) if swap else (self, other))

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("subtract", o)
    def __rsub__(self, o): return self._bin("subtract", o, True)
    def __mul__(self, o): return self._bin("multiply", o)
    def __rmul__(self, o): return self._bin("multiply", o, True)
    def __truediv__(self, o): return self._bin("true_divide", o)
    def __rtruediv__(self, o): return self._bin("true_divide", o, True)
    def __pow__(self, o): return self._bin("power", o)
    def __rpow__(self, o): return self._bin("power", o, True)
    def __floordiv__(self, o): return self._bin("floor_divide", o)
    def __rfloordiv__(self, o): return self._bin("floor_divide", o, True)
    def __mod__(self, o): return self._bin("remainder", o)
    def __rmod__(self, o): return self._bin("remainder", o, True)
    def __and__(self, o): return self._bin("bitwise_and", o)
    def __rand__(self, o): return self._bin("bitwise_and", o, True)
    def __or__(self, o): return self._bin("bitwise_or", o)
    def __ror__(self, o): return self._bin("bitwise_or", o, True)
    def __xor__(self, o): return self._bin("bitwise_xor", o)
    def __rxor__(self, o): return self._bin("bitwise_xor", o, True)
    def __lshift__(self, o): return self._bin("left_shift", o)
    def __rlshift__(self, o): return self._bin("left_shift", o, True)
    def __rshift__(self, o): return self._bin("right_shift", o)
    def __rrshift__(self, o): return self._bin("right_shift", o, True)
    def __invert__(self): return apply_ufunc(self.trace, "invert", (self,))

    # in-place operators write through to the array they name
    def _inplace(self, name, other):
        res = apply_ufunc(self.trace, name, (self, other))
        if self.node.kind != "leaf":
            return res  # a temporary: rebinding the name is all there is to do
        self[...] = res
        return self

    def __iadd__(self, o): return self._inplace("add", o)
    def __isub__(self, o): return self._inplace("subtract", o)
    def __imul__(self, o): return self._inplace("multiply", o)
    def __itruediv__(self, o): return self._inplace("true_divide", o)
    def __ifloordiv__(self, o): return self._inplace("floor_divide", o)
    def __imod__(self, o): return self._inplace("remainder", o)
    def __ipow__(self, o): return self._inplace("power", o)
    def __iand__(self, o): return self._inplace("bitwise_and", o)
    def __ior__(self, o): return self._inplace("bitwise_or", o)
    def __ixor__(self, o): return self._inplace("bitwise_xor", o)
    def __ilshift__(self, o): return self._inplace("left_shift", o)
    def __irshift__(self, o): return self._inplace("right_shift", o)
    def __neg__(self): return apply_ufunc(self.trace, "negative", (self,))
    def __pos__(self): return self
    def __abs__(self): return apply_ufunc(self.trace, "absolute", (self,))
    def __lt__(self, o): return self._bin("less", o)
    def __le__(self, o): return self._bin("less_equal", o)
    def __gt__(self, o): return self._bin("greater", o)
    def __ge__(self, o): return self._bin("greater_equal", o)
    def __eq__(self, o): return self._bin("equal", o)
    def __ne__(self, o): return self._bin("not_equal", o)
    __hash__ = None

    # concrete escapes (scalars only) ---------------------------------------------
    def _escape(self):
        if self.concrete is None:
            raise TypeError("the value of a device expression is not available while tracing; "
                            "only scalar arguments can drive Python control flow")
        self.trace.value_dependent = True
        return self.concrete

    def __bool__(self): return bool(self._escape())
    def __float__(self): return float(self._escape())
    def __int__(self): return int(self._escape())
    def __index__(self): return int(self._escape())

    # reductions / methods ----------------------------------------------------------
    def sum(self, axis=None, dtype=None, keepdims=False):
        return reduce_lazy(self.trace, "sum", self, axis=axis, dtype=dtype, keepdims=keepdims)

    def prod(self, axis=None, dtype=None, keepdims=False):
        return reduce_lazy(self.trace, "prod", self, axis=axis, dtype=dtype, keepdims=keepdims)

    def min(self, axis=None, keepdims=False):
        return reduce_lazy(self.trace, "min", self, axis=axis, keepdims=keepdims)

    def max(self, axis=None, keepdims=False):
        return reduce_lazy(self.trace, "max", self, axis=axis, keepdims=keepdims)

    def mean(self, axis=None, dtype=None, keepdims=False):
        return mean_lazy(self.trace, self, axis=axis, dtype=dtype, keepdims=keepdims)

    def clip(self, a_min=None, a_max=None):
        return clip_lazy(self.trace, self, a_min, a_max)

    def var(self, axis=None): return var_lazy(self.trace, self, axis=axis)
    def std(self, axis=None): return apply_ufunc(self.trace, "sqrt", (var_lazy(self.trace, self, axis=axis),))
    def any(self, axis=None): return truth_reduce(self.trace, np.any, self, axis=axis)
    def all(self, axis=None): return truth_reduce(self.trace, np.all, self, axis=axis)

    def copy(self):
        out = self.trace.leaf(self.trace.add_tmp_slot(self.shape, self.dtype))
        out[...] = self
        return out

    def ravel(self):
        return self.reshape(-1)

    def flatten(self):
        return self.copy().reshape(-1)
    def argmin(self, axis=None): return reduce_lazy(self.trace, "argmin", self, axis=axis)
    def argmax(self, axis=None): return reduce_lazy(self.trace, "argmax", self, axis=axis)
    def dot(self, other): return dot(self.trace, self, other)
    def __matmul__(self, other): return dot(self.trace, self, other)
    def __rmatmul__(self, other): return dot(self.trace, other, self)

    def astype(self, dtype):
        dtype = np.dtype(dtype)
        if dtype == self.dtype:
            return self
        return LazyArray(self.trace, Node("cast", dtype, self.shape, (self.node,)))

    # views -------------------------------------------------------------------------
    def _view(self, view_op, fn):
        slot = self.trace.materialize(self)
        arr = fn(self.trace.arrays[slot])
        return self.trace.leaf(self.trace.add_view_slot(slot, view_op, arr))

    @property
    def T(self):
        return self._view(("T",), lambda a: a.T)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if self.node.kind != "leaf":
            # a value that is not an array yet: reshaped when it becomes one
            shape = [int(d) for d in shape]
            if shape.count(-1) > 1:
                raise ValueError("can only specify one unknown dimension")
            if -1 in shape:
                known = int(np.prod([d for d in shape if d != -1], dtype=np.int64))
                shape[shape.index(-1)] = self.size // max(known, 1)
            if int(np.prod(shape, dtype=np.int64)) != self.size:
                raise ValueError(f"cannot reshape array of size {self.size} into {tuple(shape)}")
            if tuple(shape) == self.shape:
                return self
            return LazyArray(self.trace, Node("reshape", self.dtype, shape, (self.node,)))
        return self._view(("reshape", shape), lambda a: a.reshape(shape))

    def __getitem__(self, idx):
        if idx is Ellipsis or (isinstance(idx, slice) and idx == slice(None)):
            return self
        if self.node.kind != "leaf" and isinstance(idx, tuple) and all(
                i is None or (isinstance(i, slice) and i == slice(None)) for i in idx) \
                and sum(1 for i in idx if i is not None) <= self.ndim:
            # only new axes (x[:, None]): a reshape
            dims = iter(self.shape)
            shape = [1 if i is None else next(dims) for i in idx] + list(dims)
            return self.reshape(shape)
        if isinstance(idx, LazyArray) and (idx.ndim > 0 or idx.concrete is None):
            return gather_lazy(self.trace, self, idx)  # an index array, or a position computed on the device
        return self._view(("getitem", idx), lambda a: a[idx])

    def __setitem__(self, idx, value):
        whole = idx is Ellipsis or (isinstance(idx, slice) and idx == slice(None))
        if isinstance(idx, LazyArray) and (idx.ndim > 0 or idx.concrete is None):
            raise TypeError("assignment through an index array or a mask is not supported on device arrays")
        target = self if whole else self[idx]
        if target.node.kind != "leaf":
            raise TypeError("cannot assign into an expression")
        vnode = _as_node(self.trace, value)
        broadcast_shapes(vnode.shape, target.shape)  # raises on mismatch
        if np.broadcast_shapes(vnode.shape, target.shape) != target.shape:
            raise ValueError(f"could not broadcast {vnode.shape} into {target.shape}")
        if vnode.dtype != target.dtype:
            vnode = Node("cast", target.dtype, vnode.shape, (vnode,))
        self.trace.store(target.node.slot, vnode, value if isinstance(value, LazyArray) else None)


def _is_one(node):
    while node.kind == "cast":
        node = node.inputs[0]
    return node.kind == "const" and node.value == 1


def apply_ufunc(trace, name, inputs):
    nodes = [_as_node(trace, x) for x in inputs]
    ufunc, _emit = UFUNCS[name]
    loop_in, out_dt = find_loop(ufunc, [n.dtype for n in nodes])
    cast = [n if n.dtype == d else Node("cast", d, n.shape, (n,)) for n, d in zip(nodes, loop_in)]
    shape = broadcast_shapes(*[n.shape for n in nodes])
    node = Node("op", out_dt, shape, cast, op=name)
    if trace.fastmath and name == "true_divide" and _is_one(cast[0]) and cast[1].kind == "op" \
            and cast[1].op == "sqrt" and out_dt == np.float32 and cast[1].shape == shape:
        node = Node("op", out_dt, shape, cast[1].inputs, op="rsqrt")  # 1/sqrt(x): one instruction
    concrete = None
    if shape == () and all(isinstance(x, LazyArray) and x.concrete is not None or
                           not isinstance(x, (LazyArray, DeviceArray)) for x in inputs):
        vals = [x.concrete if isinstance(x, LazyArray) else x for x in inputs]
        with np.errstate(all="ignore"):
            concrete = out_dt.type(ufunc(*[d.type(v) for v, d in zip(vals, loop_in)]))
    return LazyArray(trace, node, concrete)


def where(trace, cond, x, y):
    c, a, b = (_as_node(trace, v) for v in (cond, x, y))
    out_dt = np.result_type(a.dtype, b.dtype)
    a = a if a.dtype == out_dt else Node("cast", out_dt, a.shape, (a,))
    b = b if b.dtype == out_dt else Node("cast", out_dt, b.shape, (b,))
    shape = broadcast_shapes(c.shape, a.shape, b.shape)
    return LazyArray(trace, Node("where", out_dt, shape, (c, a, b)))


def call_device_func(trace, func, inputs):
    nodes = [_as_node(trace, x) for x in inputs]
    cast = [n if n.dtype == d else Node("cast", d, n.shape, (n,)) for n, d in zip(nodes, func.arg_dtypes)]
    shape = broadcast_shapes(*[n.shape for n in nodes])
    return LazyArray(trace, Node("call", func.ret_dtype, shape, cast, op=func))


_REDUCE_KERNEL_DTYPES = ("float32", "float64", "int32", "int64")


def reduce_lazy(trace, op, a, axis=None, dtype=None, keepdims=False, out=None):
    if out is not None:
        raise TypeError("out= is not supported in device reductions")
    from . import reduce_ops

    if not isinstance(a, LazyArray):
        a = LazyArray(trace, _as_node(trace, a))
    if isinstance(axis, LazyArray):
        axis = int(axis)
    if isinstance(keepdims, LazyArray):
        keepdims = bool(keepdims)
    final = None
    if dtype is not None and np.dtype(dtype) != a.dtype:
        a = a.astype(dtype)  # NumPy casts the elements first, then reduces in `dtype`
    if a.dtype.name not in _REDUCE_KERNEL_DTYPES:
        # narrow integers and bool: reduce the values in a 32-bit type (sums and
        # products wrap the same way modulo 2^16 or 2^8), cast the result back
        if a.dtype.kind not in "iub":
            raise TypeError(f"reductions of {a.dtype} are not supported on the device")
        if op in ("sum", "prod"):
            final = a.dtype if dtype is not None else None  # NumPy's default widens to the platform int
            a = a.astype(np.int32 if a.dtype.itemsize < 4 else np.int64)
        else:
            final = a.dtype if not op.startswith("arg") else None
            a = a.astype(np.int32 if a.dtype.itemsize < 4 else np.int64)
    res = _reduce_node(trace, op, a, axis, reduce_ops)
    if final is not None and res.dtype != final:
        res = res.astype(final)
    if keepdims:
        nd = len(a.shape)
        kept = (1,) * nd if axis is None else tuple(1 if d == axis % nd else s for d, s in enumerate(a.shape))
        res = res.reshape(kept)
    return res


def mean_lazy(trace, a, axis=None, dtype=None, keepdims=False, out=None):
    """NumPy's mean: the sum in `dtype` (float64 for integer input, the input
    type for floats) divided by the element count; an integer `dtype` keeps
    the truncated quotient."""
    if out is not None:
        raise TypeError("out= is not supported in device reductions")
    if not isinstance(a, LazyArray):
        a = LazyArray(trace, _as_node(trace, a))
    if isinstance(axis, LazyArray):
        axis = int(axis)
    if dtype is None:
        dtype = np.float64 if a.dtype.kind in "iub" else a.dtype
    dtype = np.dtype(dtype)
    count = a.size if axis is None else a.shape[axis % len(a.shape)]
    total = reduce_lazy(trace, "sum", a, axis=axis, dtype=dtype, keepdims=keepdims)
    if dtype.kind in "iub":
        return (total / np.float64(count)).astype(dtype)
    return total / dtype.type(count)


def var_lazy(trace, a, axis=None, dtype=None, keepdims=False, ddof=0, out=None):
    """np.var as NumPy computes it: mean(|x - mean(x)|^2)."""
    if out is not None or ddof != 0:
        raise TypeError("out= and ddof are not supported on device arrays")
    if not isinstance(a, LazyArray):
        a = LazyArray(trace, _as_node(trace, a))
    m = mean_lazy(trace, a, axis=axis, dtype=dtype, keepdims=True)
    d = a - m
    return mean_lazy(trace, d * d, axis=axis, dtype=dtype, keepdims=keepdims)


def truth_reduce(trace, func, a, axis=None, keepdims=False, out=None):
    """np.any / np.all / np.count_nonzero through the min / max / sum kernels."""
    if out is not None:
        raise TypeError("out= is not supported on device arrays")
    if not isinstance(a, LazyArray):
        a = LazyArray(trace, _as_node(trace, a))
    nz = a if a.dtype == np.bool_ else (a != a.dtype.type(0))
    if func is np.count_nonzero:
        return reduce_lazy(trace, "sum", nz.astype(np.int64), axis=axis, keepdims=keepdims)
    return reduce_lazy(trace, "max" if func is np.any else "min", nz, axis=axis, keepdims=keepdims)


def concatenate_lazy(trace, arrays, axis=0, out=None, dtype=None):
    if out is not None:
        raise TypeError("out= is not supported on device arrays")
    parts = [x if isinstance(x, LazyArray) else LazyArray(trace, _as_node(trace, x)) for x in arrays]
    nd = len(parts[0].shape)
    axis %= nd
    dt = np.dtype(dtype) if dtype is not None else np.result_type(*[p.dtype for p in parts])
    shape = list(parts[0].shape)
    shape[axis] = sum(p.shape[axis] for p in parts)
    res = trace.leaf(trace.add_tmp_slot(tuple(shape), dt))
    pos = 0
    for p in parts:
        idx = tuple(slice(pos, pos + p.shape[axis]) if d == axis else slice(None) for d in range(nd))
        res[idx] = p
        pos += p.shape[axis]
    return res


def _lazy(trace, x):
    return x if isinstance(x, LazyArray) else LazyArray(trace, _as_node(trace, x))


# hstack / vstack / dstack (numba_mlir/mlir/numpy/funcs.py: numpy.hstack, vstack,
# dstack): the operands get the rank NumPy gives them, then it is a concatenate
_STACKS = {np.vstack: "v", np.hstack: "h", np.dstack: "d"}


def stack_lazy(trace, kind, tup, dtype=None, casting=None):
    parts = [_lazy(trace, x) for x in tup]
    if not parts:
        raise ValueError("need at least one array to concatenate")

    def at_least(x, nd):
        if x.ndim >= nd:
            return x
        if x.ndim == 0:
            return x.reshape((1,) * nd)
        if nd == 2:
            return x.reshape(1, x.shape[0])                      # (N,) -> (1, N)
        return x.reshape(1, x.shape[0], 1) if x.ndim == 1 else x.reshape(x.shape + (1,))

    if kind == "v":
        return concatenate_lazy(trace, [at_least(x, 2) for x in parts], axis=0, dtype=dtype)
    if kind == "d":
        return concatenate_lazy(trace, [at_least(x, 3) for x in parts], axis=2, dtype=dtype)
    parts = [at_least(x, 1) for x in parts]
    return concatenate_lazy(trace, parts, axis=0 if parts[0].ndim == 1 else 1, dtype=dtype)


_GATHER_SOURCE = """//NMB200:CUDA-SOURCE
#include "nmb_device.cuh"
extern "C" __global__ void __launch_bounds__(256) nmb_gather(
    const {T}* __restrict__ src, const {I}* __restrict__ idx, {T}* __restrict__ out,
    int64_t n, int64_t extent, int64_t row_stride, int64_t inner) {{
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += step) {{
    const int64_t i = e / inner, j = e - i * inner;
    int64_t k = (int64_t)idx[i];
    k = k < 0 ? k + extent : k;
    k = k < 0 ? 0 : (k >= extent ? extent - 1 : k);  // stays inside the array whatever the index holds
    out[e] = src[k * row_stride + j];
  }}
}}
"""


def gather_lazy(trace, a, idx):
    """a[idx] with an integer index array (numba_mlir/mlir/tests/test_numpy.py:
    test_getitem_offset): element i of the result is a[idx[i]] (a row of `a`
    when it has more dimensions); negative indices count from the end.  An
    index outside the array, for which NumPy raises, reads the nearest valid
    element: a kernel cannot raise, and it must not read outside the array."""
    if idx.dtype.kind == "b":
        return select_lazy(trace, a, idx)
    if idx.dtype.kind not in "iu":
        raise TypeError("an index array must hold integers or booleans")
    if a.ndim == 0:
        raise IndexError("too many indices for a 0-dimensional array")
    if a.shape[0] == 0:
        raise IndexError("index array into an empty array")
    a_slot = trace.materialize(a)
    if a.ndim > 1 and not trace.arrays[a_slot].is_c_contiguous:
        a_slot = trace.materialize(a.copy())
    i_slot = trace.materialize(idx)
    if not trace.arrays[i_slot].is_c_contiguous:
        i_slot = trace.materialize(idx.copy())
    src, ind = trace.arrays[a_slot], trace.arrays[i_slot]
    inner = int(np.prod(src.shape[1:], dtype=np.int64))
    row_stride = src.strides[0] // src.dtype.itemsize if src.ndim == 1 else inner
    out_slot = trace.add_tmp_slot(tuple(ind.shape) + tuple(src.shape[1:]), src.dtype)
    n = int(np.prod(ind.shape, dtype=np.int64)) * inner
    if n:
        key = ("gather", src.dtype.name, ind.dtype.name)
        blob = _kernel_cache.get(key)
        if blob is None:
            blob = _kernel_cache[key] = _GATHER_SOURCE.format(T=ctype(src.dtype), I=ctype(ind.dtype)).encode()
        grid = min((n + 255) // 256, 148 * 8)
        step = ("launch", blob, "nmb_gather", (grid,), (256,),
                (("slot", a_slot), ("slot", i_slot), ("slot", out_slot), ("i64", n), ("i64", src.shape[0]),
                 ("i64", row_stride), ("i64", inner)))
        trace.steps.append(step)
        if not trace.dry:
            run_launch(trace.queue, step, trace.arrays, trace.args)
    return trace.leaf(out_slot)


_SELECT_SOURCE = """//NMB200:CUDA-SOURCE
#include "nmb_device.cuh"
// Order-preserving selection out[k] = src[i] for the k-th set mask[i]: counts
// per block of 2048 elements, one block turns the counts into offsets (and the
// total), then every block writes its elements from its offset on.
__device__ __forceinline__ int tile_count(const unsigned char* __restrict__ mask, int64_t n, int64_t base) {{
  int c = 0;
#pragma unroll
  for (int l = 0; l < 8; ++l) c += (base + l < n) && mask[base + l] != 0;
  return c;
}}
// exclusive prefix of `v` over the 256 threads of the block; `total` = the block's sum
__device__ __forceinline__ int block_prefix(int v, int& total) {{
  __shared__ int warp_sums[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {{
    const int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }}
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {{
    before += w < warp ? warp_sums[w] : 0;
    all += warp_sums[w];
  }}
  __syncthreads();
  total = all;
  return before + inc - v;
}}
extern "C" __global__ void __launch_bounds__(256) nmb_select_count(
    const unsigned char* __restrict__ mask, int64_t n, int64_t* __restrict__ offsets) {{
  int total;
  block_prefix(tile_count(mask, n, ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8), total);
  if (threadIdx.x == 0) offsets[blockIdx.x] = total;
}}
// offsets[b] <- sum of offsets[0..b); offsets[blocks] <- the total
extern "C" __global__ void __launch_bounds__(256) nmb_select_offsets(int64_t* __restrict__ offsets, int64_t blocks) {{
  __shared__ int64_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t start = 0; start < blocks; start += 256) {{
    const int64_t b = start + threadIdx.x;
    const int v = b < blocks ? (int)offsets[b] : 0;  // a block holds at most 2048
    int total;
    const int before = block_prefix(v, total);
    if (b < blocks) offsets[b] = carry + before;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }}
  if (threadIdx.x == 0) offsets[blocks] = carry;
}}
extern "C" __global__ void __launch_bounds__(256) nmb_select_write(
    const {T}* __restrict__ src, const unsigned char* __restrict__ mask, {T}* __restrict__ out, int64_t n,
    const int64_t* __restrict__ offsets) {{
  const int64_t base = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 8;
  int total;
  int64_t k = offsets[blockIdx.x] + block_prefix(tile_count(mask, n, base), total);
#pragma unroll
  for (int l = 0; l < 8; ++l)
    if (base + l < n && mask[base + l] != 0) out[k++] = src[base + l];
}}
"""


def select_lazy(trace, a, mask):
    """a[mask] with a boolean array of a's shape (numba_mlir/mlir/tests/
    test_numpy.py: test_getitem_mask): the selected elements in C order.  The
    size of the result is read back from the device, so the call is traced
    afresh every time instead of being replayed from a recorded plan."""
    if tuple(mask.shape) != tuple(a.shape):
        raise IndexError(f"boolean index of shape {tuple(mask.shape)} does not match the array's {tuple(a.shape)}")
    if trace.dry:
        raise TypeError("the size of a[mask] is not available while tracing without a device")
    slots = []
    for x in (a, mask):
        slot = trace.materialize(x)
        if not trace.arrays[slot].is_c_contiguous:
            slot = trace.materialize(x.copy())
        slots.append(slot)
    a_slot, m_slot = slots
    n = a.size
    trace.value_dependent = True
    if n == 0:
        return trace.leaf(trace.add_tmp_slot((0,), a.dtype))
    key = ("select", a.dtype.name)
    blob = _kernel_cache.get(key)
    if blob is None:
        blob = _kernel_cache[key] = _SELECT_SOURCE.format(T=ctype(a.dtype)).encode()
    blocks = (n + 2047) // 2048
    off_slot = trace.add_tmp_slot((blocks + 1,), np.int64)

    def launch(name, grid, params):
        step = ("launch", blob, name, (grid,), (256,), params)
        trace.steps.append(step)
        run_launch(trace.queue, step, trace.arrays, trace.args)

    launch("nmb_select_count", blocks, (("slot", m_slot), ("i64", n), ("slot", off_slot)))
    launch("nmb_select_offsets", 1, (("slot", off_slot), ("i64", blocks)))
    count = int(trace.arrays[off_slot][blocks:].copy_to_host()[0])
    out_slot = trace.add_tmp_slot((count,), a.dtype)
    if count:
        launch("nmb_select_write", blocks, (("slot", a_slot), ("slot", m_slot), ("slot", out_slot), ("i64", n),
                                            ("slot", off_slot)))
    return trace.leaf(out_slot)


def flip_lazy(trace, m, axis=None):
    """np.flip: a view with negative strides (numba_mlir/mlir/numpy/funcs.py: numpy.flip)."""
    m = _lazy(trace, m)
    axes = range(m.ndim) if axis is None else ([axis] if isinstance(axis, (int, np.integer)) else list(axis))
    axes = {int(a) % m.ndim for a in axes}
    return m[tuple(slice(None, None, -1) if d in axes else slice(None) for d in range(m.ndim))]


def outer_lazy(trace, a, b):
    a, b = _lazy(trace, a).ravel(), _lazy(trace, b).ravel()
    return apply_ufunc(trace, "multiply", (a.reshape(a.shape[0], 1), b.reshape(1, b.shape[0])))


def triangle_lazy(trace, lower, m, k=0):
    """np.tril / np.triu over the last two axes: a select against the element's
    own row and column numbers."""
    m = _lazy(trace, m)
    if m.ndim < 2:
        raise ValueError("tril and triu need an array of at least two dimensions")
    rows, cols = m.shape[-2], m.shape[-1]
    diff = _index_array(trace, (1, cols), 1) - _index_array(trace, (rows, 1), 0)   # column - row
    keep = apply_ufunc(trace, "less_equal" if lower else "greater_equal", (diff, np.int64(k)))
    return where(trace, keep, m, m.dtype.type(0))


def cov_lazy(trace, m, y=None, rowvar=True, bias=False, ddof=None, fweights=None, aweights=None, dtype=None):
    """np.cov of one set of observations (numba_mlir/mlir/numpy/funcs.py:
    numpy.cov), with NumPy's steps: the data in float64 (or `dtype`), minus
    the mean of every variable, times its own transpose (the float64 product),
    times 1 / (N - ddof)."""
    if y is not None or fweights is not None or aweights is not None:
        raise TypeError("np.cov on device arrays takes one array and no weights")
    m = _lazy(trace, m)
    if m.ndim > 2:
        raise ValueError("m has more than 2 dimensions")
    dt = np.dtype(dtype) if dtype is not None else np.result_type(m.dtype, np.float64)
    x = m if m.dtype == dt else m.astype(dt)
    if x.ndim < 2:
        x = x.reshape(1, x.size)
    elif not rowvar and x.shape[0] != 1:
        x = x.T
    if ddof is None:
        ddof = 0 if bias else 1
    fact = max(x.shape[1] - ddof, 0)
    centred = x - mean_lazy(trace, x, axis=1, keepdims=True)
    c = dot(trace, centred, centred.T) * np.true_divide(1, fact).astype(dt)
    return reduce_lazy(trace, "sum", c) if c.shape == (1, 1) else c


def clip_lazy(trace, a, a_min=None, a_max=None, out=None):
    """np.clip: bounds are converted to the array's type, as Numba types it;
    with `out` the result is stored there (test_numpy.py: test_ternary_inplace)."""
    if not isinstance(a, LazyArray):
        a = LazyArray(trace, _as_node(trace, a))

    def bound(b):
        return a.dtype.type(b) if isinstance(b, (bool, int, float, np.generic)) else b

    res = a
    if a_min is not None:
        res = apply_ufunc(trace, "maximum", (res, bound(a_min)))
    if a_max is not None:
        res = apply_ufunc(trace, "minimum", (res, bound(a_max)))
    if out is not None:
        if not isinstance(out, LazyArray):
            raise TypeError("out= must be a device array")
        out[...] = res
        return out
    return res


def _reduce_node(trace, op, a, axis, reduce_ops):
    """The reduction as a graph node; it runs when a flush reaches it."""
    src = _as_node(trace, a)
    shape = src.shape
    if axis is None:
        if int(np.prod(shape, dtype=np.int64)) == 0:
            raise ValueError("zero-size array to reduction operation")
        oshape = ()
    else:
        axis = int(axis)
        if not -len(shape) <= axis < len(shape):
            raise ValueError("axis out of range")
        axis %= len(shape)
        if shape[axis] == 0:
            raise ValueError("zero-size reduction axis")
        oshape = shape[:axis] + shape[axis + 1:]
    return LazyArray(trace, Node("reduce", reduce_ops.out_dtype(op, src.dtype), oshape, (src,), op=op, value=axis))


def dot(trace, a, b, out=None):
    """np.dot as a graph node: the product runs when a flush reaches it, alone
    (the tensor-core gemm) or together with the elementwise chain around it."""
    a = a if isinstance(a, LazyArray) else LazyArray(trace, _as_node(trace, a))
    b = b if isinstance(b, LazyArray) else LazyArray(trace, _as_node(trace, b))
    if out is None and (len(a.shape) == 1 or len(b.shape) == 1):
        # vector operands: the matrix product of the reshaped operands
        if len(a.shape) == 1 and len(b.shape) == 1:
            return reduce_lazy(trace, "sum", a * b)
        if len(a.shape) == 1:
            return dot(trace, a.reshape(1, a.shape[0]), b).reshape(b.shape[1])
        return dot(trace, a, b.reshape(b.shape[0], 1)).reshape(a.shape[0])
    if len(a.shape) != 2 or len(b.shape) != 2 or a.shape[1] != b.shape[0]:
        raise ValueError("dot needs 2-D operands with matching inner dimension")
    node = Node("dot", np.result_type(a.dtype, b.dtype), (a.shape[0], b.shape[1]),
                (_as_node(trace, a), _as_node(trace, b)))
    res = LazyArray(trace, node)
    if out is not None:
        out[...] = res
        return out
    return res


# ---- the elementwise chain around a product, as the contraction's epilogue ----
def _const_value(node):
    while node.kind == "cast":
        node = node.inputs[0]
    return node.value if node.kind == "const" else None


def _scaled_dot(node):
    """(c, dot node) when `node` is c * dot (either order), -dot or dot."""
    if node.kind == "dot":
        return 1.0, node
    if node.kind == "op" and node.op == "negative" and node.inputs[0].kind == "dot":
        return -1.0, node.inputs[0]
    if node.kind == "op" and node.op == "multiply":
        x, y = node.inputs
        for c, d in ((x, y), (y, x)):
            v = _const_value(c)
            if v is not None and d.kind == "dot" and c.dtype == np.float32:
                return float(v), d
    return None, None


def _match_rowcol(trace, node):
    """Recognises func(alpha * dot(a, b) + row + col) with func the identity or
    sqrt(maximum(., 0)), `row` of shape (M, 1) and `col` of shape (1, N) or
    (N,), all float32.  Returns (alpha, dot node, row, col, func) or None."""
    if node.kind != "op" or len(node.shape) != 2 or node.dtype != np.float32:
        return None
    m, n = node.shape
    if m <= 1 or n <= 1:
        return None
    func, body = 0, node
    if node.op == "sqrt":
        inner = node.inputs[0]
        if inner.kind != "op" or inner.op != "maximum":
            return None
        x, y = inner.inputs
        if _const_value(y) == 0:
            body = x
        elif _const_value(x) == 0:
            body = y
        else:
            return None
        func = 1
    terms = []

    def collect(t, sign):
        if t.kind == "op" and t.op == "add":
            collect(t.inputs[0], sign)
            collect(t.inputs[1], sign)
        elif t.kind == "op" and t.op == "subtract":
            collect(t.inputs[0], sign)
            collect(t.inputs[1], -sign)
        else:
            terms.append((sign, t))

    collect(body, 1.0)
    if len(terms) > 3:
        return None
    alpha = product = row = col = None
    for sign, t in terms:
        c, d = _scaled_dot(t)
        if d is not None:
            if product is not None or d.shape != (m, n) or d.dtype != np.float32:
                return None
            alpha, product = sign * c, d
        elif sign != 1.0 or t.dtype != np.float32 or t.kind in ("arg", "const"):
            return None
        elif t.shape == (m, 1) and row is None:
            row = t
        elif t.shape in ((1, n), (n,)) and col is None:
            col = t
        else:
            return None
    if product is None or (func == 0 and row is None and col is None and alpha == 1.0):
        return None
    if any(i.dtype != np.float32 for i in product.inputs):
        return None
    return alpha, product, row, col, func


def _match_post_reduce(node):
    """The reduction node when `node` is an elementwise chain over ONE
    reduction's value and scalars only (np.sqrt(np.sum(...)), sum / count, ...)
    with the reduction's shape; None otherwise."""
    if node.kind not in ("op", "cast", "where", "call"):
        return None
    found = []

    def walk(n):
        if n.kind == "reduce":
            if not found:
                found.append(n)
            return n is found[0]
        if n.kind in ("const", "arg"):
            return n.shape == ()
        if n.kind in ("op", "cast", "where", "call"):
            return all(walk(i) for i in n.inputs)
        return False  # arrays, products, reshapes

    if not walk(node) or not found or found[0].shape != node.shape:
        return None
    return found[0]


def _is_row_norms(trace, term, operand_slot, transposed):
    """`term` is sum(x * x, axis=1) (possibly reshaped) of the matrix x whose
    rows the contraction's operand holds: x is the array of `operand_slot`, or
    its transpose when the operand is the second factor of the product."""
    while term.kind == "reshape":
        term = term.inputs[0]
    if term.kind != "reduce" or term.op != "sum" or term.value != 1:
        return False
    sq = term.inputs[0]
    if sq.kind != "op" or len(sq.shape) != 2:
        return False
    if sq.op == "square":
        x, y = sq.inputs[0], sq.inputs[0]
    elif sq.op == "multiply":
        x, y = sq.inputs
    else:
        return False
    if x.kind != "leaf" or y.kind != "leaf" or trace.overlap(x.slot, y.slot) != 1:
        return False
    arr, op_arr = trace.arrays[x.slot], trace.arrays[operand_slot]
    if transposed:
        op_arr = op_arr.T
    return (arr.ptr == op_arr.ptr and arr.shape == op_arr.shape and arr.strides == op_arr.strides
            and arr.dtype == np.float32)


def run_contract(step, get):
    from . import contraction

    _tag, sa, sb, alpha, row, col, func, dst = step

    def term(t):
        return t if t is None or isinstance(t, str) else get(t)

    contraction.contract_rowcol(get(sa), get(sb).T, get(dst), alpha, term(row), term(col), func)


# ---------------------------------------------------------------- codegen ---
def _leaf_access(leaf_arr, out_shape):
    """How a leaf is addressed from the flat C-order output index i.

    Returns (kind, params): 'full' (same shape, contiguous: index i), 'splat'
    (one element), 'row' (contiguous trailing block, leading dims broadcast:
    i % size), 'col' (contiguous leading block, trailing dims broadcast:
    i / inner), 'strided' (general: per-dimension element strides)."""
    shape = (1,) * (len(out_shape) - leaf_arr.ndim) + leaf_arr.shape
    it = leaf_arr.dtype.itemsize
    strides = (0,) * (len(out_shape) - leaf_arr.ndim) + tuple(s // it for s in leaf_arr.strides)
    strides = tuple(0 if d == 1 else s for d, s in zip(shape, strides))
    n = int(np.prod(shape, dtype=np.int64))
    if n == 1:
        return "splat", ()
    contiguous = leaf_arr.is_c_contiguous
    if contiguous and shape == tuple(out_shape):
        return "full", ()
    if contiguous:
        lead = 0
        while lead < len(shape) and shape[lead] == 1:
            lead += 1
        if shape[lead:] == tuple(out_shape[lead:]):
            return "row", (n,)
        tail = len(shape)
        while tail > 0 and shape[tail - 1] == 1:
            tail -= 1
        if shape[:tail] == tuple(out_shape[:tail]):
            return "col", (int(np.prod(out_shape[tail:], dtype=np.int64)),)
    return "strided", tuple(strides)


# float32 operations that exist as one instruction on two values (add/sub/mul.rn.f32x2)
# (helper in nmb_device.cuh, number of operands it takes per element); `log` is
# this library's own polynomial, evaluated for two elements with packed FMAs
# Operations that may read a packed product: none of them adds to its operand
# before rounding (multiplies; the IEEE division and square root, which use their
# operands as multiplicands and as the addend of a residual; log, which starts
# with integer operations; exp, which starts with a multiply; comparisons).
_PRODUCT_READERS = frozenset(["multiply", "square", "true_divide", "sqrt", "log", "exp", "less", "less_equal",
                              "greater", "greater_equal", "equal", "not_equal", "isnan"])
_PACKED_OPS = {"add": ("add2", 2), "subtract": ("sub2", 2), "multiply": ("mul2", 2), "square": ("mul2", 2),
               "log": ("log_pair", 1)}


def _second_lane(text):
    """The chain text of element l rewritten for element l + 1."""
    return re.sub(r"\bt(\d+)\b", r"t\1_b", text).replace(".v[l]", ".v[l + 1]").replace("(r.base + l)", "(r.base + l + 1)")


def _paired_lines(em, lines, out_assign, fuse_ok=False):
    """The chain for two adjacent elements at once: every line twice, except the
    float32 additions, subtractions and multiplications, which become one
    packed instruction for both elements (IEEE results, half the issue slots)."""
    out = []
    for i, line in enumerate(lines):
        hit = em.packable.get(i)
        if hit is not None and hit[0] == "mul2" and f"t{i}" in em.scalar_only and not fuse_ok:
            hit = None
        if hit is None:
            out.append(line)
            out.append(_second_lane(line))
        else:
            fn, operands = hit
            both = ", ".join(f"{x}, {_second_lane(x)}" for x in operands)
            out.append(f"float t{i}, t{i}_b; nmb::{fn}({both}, t{i}, t{i}_b);")
    for line in out_assign:
        out.append(line)
        out.append(_second_lane(line))
    return out


class _Emitter:
    def __init__(self, trace, out_shape):
        self.trace = trace
        self.out_shape = tuple(out_shape)
        self.lines = []
        self.names = {}          # id(node) -> C expression
        self.leaves = []         # [(slot, kind, params, dtype)]
        self.leaf_index = {}
        self.scalar_args = []    # [(arg index, dtype)]
        self.scalar_index = {}
        self.funcs = {}
        self.sig = []
        self.packable = {}       # line index -> (packed helper, operand expressions)
        self.scalar_only = set() # names of values read by something that may add to them
        self.uses_index = False  # some value is the element's own coordinate (needs the flat position)

    def leaf(self, node):
        key = node.slot
        if key not in self.leaf_index:
            arr = self.trace.arrays[node.slot]
            kind, params = _leaf_access(arr, self.out_shape)
            self.leaf_index[key] = len(self.leaves)
            self.leaves.append((node.slot, kind, params, arr.dtype))
        return self.leaf_index[key]

    def emit(self, node):
        key = id(node)
        if key in self.names:
            return self.names[key]
        if node.kind == "leaf":
            expr = f"r.in{self.leaf(node)}.v[l]"
            self.sig.append(("leaf", self.leaf_index[node.slot]))
        elif node.kind == "const":
            expr = literal(node.value, node.dtype)
            self.sig.append(("const", expr))
        elif node.kind == "arg":
            if node.value not in self.scalar_index:
                self.scalar_index[node.value] = len(self.scalar_args)
                self.scalar_args.append((node.value, node.dtype))
            expr = f"s{self.scalar_index[node.value]}"
            self.sig.append(("arg", self.scalar_index[node.value], node.dtype.name))
        elif node.kind == "index":
            # the element's own coordinate along one axis, from its flat position
            axis = node.value + len(self.out_shape) - len(node.shape)
            extent = self.out_shape[axis]
            stride = int(np.prod(self.out_shape[axis + 1:], dtype=np.int64))
            expr = "(r.base + l)"
            if stride != 1:
                expr = f"({expr} / {stride}ll)"
            if axis != 0:
                expr = f"({expr} % {extent}ll)"
            self.uses_index = True
            self.sig.append(("index", axis, stride, extent))
        else:
            ins = [self.emit(i) for i in node.inputs]
            # A packed multiply must not feed an addition: the assembler merges
            # mul.f32x2 with a dependent add/sub.f32x2 into one fused multiply-add
            # even when both carry .rn, which would change the rounding.  So a
            # product stays a scalar multiply (whose .rn is honoured) unless every
            # reader is known not to add to it.
            pair_call = node.kind == "call" and node.op.pair and node.dtype == np.float32
            if not (node.kind == "op" and node.op in _PRODUCT_READERS) and not pair_call:
                for e in ins:
                    self.scalar_only.add(e)
            if node.kind == "cast":
                rhs = f"static_cast<{ctype(node.dtype)}>({ins[0]})"
                if node.inputs[0].dtype.kind == "f" and node.dtype.kind == "b":
                    rhs = f"({ins[0]} != 0)"
            elif node.kind == "where":
                rhs = f"(({ins[0]}) ? {ins[1]} : {ins[2]})"
            elif node.kind == "call":
                self.funcs[node.op.name] = node.op.source
                rhs = f"{node.op.name}({', '.join(ins)})"
                if pair_call:
                    self.packable[len(self.lines)] = (node.op.pair, ins)
            else:
                loop_dt = node.inputs[0].dtype
                rhs = UFUNCS[node.op][1](loop_dt, *ins)
                if (node.op in _PACKED_OPS and node.dtype == np.float32
                        and all(i.dtype == np.float32 for i in node.inputs)):
                    # two elements' worth of this operation fit f32x2 instructions
                    fn, arity = _PACKED_OPS[node.op]
                    self.packable[len(self.lines)] = (fn, (ins * 2)[:arity])
            expr = f"t{len(self.lines)}"
            self.lines.append(f"const {ctype(node.dtype)} {expr} = {rhs};")
            self.sig.append((node.kind, node.op if node.kind == "op" else
                             getattr(node.op, "name", None), node.dtype.name, tuple(ins)))
        self.names[key] = expr
        return expr


_kernel_cache = {}


def _emit_eltwise(trace, out_shape, outs):
    """One fused kernel storing every (slot, node) of `outs` (same shape)."""
    n = int(np.prod(out_shape, dtype=np.int64))
    if n == 0:
        return
    em = _Emitter(trace, out_shape)
    results = [(slot, em.emit(node), trace.arrays[slot]) for slot, node in outs]

    def out_strides(arr):
        """Element strides of a non-contiguous assignment target (a sliced or
        transposed view), None for a contiguous one."""
        if arr.is_c_contiguous:
            return None
        return tuple(st // arr.dtype.itemsize for st in arr.strides)

    ostrides = [out_strides(arr) for _s, _e, arr in results]
    # vector width: 4 elements per step when every access allows it
    vec_ok = True
    for slot, kind, params, dt in em.leaves:
        arr = trace.arrays[slot]
        unit = 4 * dt.itemsize if dt.itemsize <= 4 else 16
        if kind in ("full", "row") and arr.ptr % unit:
            vec_ok = False
        if kind in ("row", "col") and params[0] % 4:
            vec_ok = False
        if kind == "strided":
            pass
    for (slot, _expr, arr), st in zip(results, ostrides):
        unit = 4 * arr.dtype.itemsize if arr.dtype.itemsize <= 4 else 16
        if st is None and arr.ptr % unit:
            vec_ok = False
    vec = 4 if vec_ok else 1
    n_streams = sum(1 for _s, k, _p, _d in em.leaves if k == "full") + len(results)
    unroll = 4 if n_streams <= 3 else 2

    # inputs that are also written by this kernel (element for element, rule (3)
    # of Trace): their pointers are not `__restrict__` and their loads do not
    # take the read-only path
    shared_in = frozenset(i for i, (slot, _k, _p, _d) in enumerate(em.leaves)
                          if any(trace.overlap(slot, o) for o, _e, _a in results))
    shared_out = frozenset(j for j, (o, _e, _a) in enumerate(results)
                           if any(trace.overlap(slot, o) for slot, _k, _p, _d in em.leaves))
    shaped = any(k == "strided" for _s, k, _p, _d in em.leaves) or any(st is not None for st in ostrides)
    sig = (tuple(out_shape) if shaped else len(out_shape), shared_in, shared_out,
           tuple((k, p if k == "strided" else (), d.name) for _s, k, p, d in em.leaves),
           tuple(em.sig), tuple((e, a.dtype.name, st) for (_s, e, a), st in zip(results, ostrides)), vec, unroll,
           trace.fastmath)
    hit = _kernel_cache.get(sig)
    if hit is None:
        hit = _generate(em, results, out_shape, vec, unroll, ostrides, trace.fastmath, shared_in, shared_out)
        _kernel_cache[sig] = hit
    blob, kname = hit

    params = []
    for slot, kind, p, dt in em.leaves:
        params.append(("slot", slot))
        if kind in ("row", "col"):
            params.append(("i64", p[0]))
    for index, dt in em.scalar_args:
        params.append(("scalar", index, dt))
    for slot, _expr, _arr in results:
        params.append(("slot", slot))
    params.append(("i64", n))
    tile = 256 * vec * unroll
    step = ("launch", blob, kname, ((n + tile - 1) // tile,), (256,), tuple(params))
    trace.steps.append(step)
    if not trace.dry:
        run_launch(trace.queue, step, trace.arrays, trace.args)


class _ValueHolder:
    """Stands where an output array does for a chain whose value is not stored."""

    def __init__(self, dtype):
        self.dtype = np.dtype(dtype)


_FUSED_REDUCE_OPS = ("sum", "prod", "min", "max")
_FUSED_ARG_OPS = ("argmin", "argmax")  # along the last axis only


def reduce_resident(em, mode="all"):
    """Blocks per multiprocessor a generated reducer is compiled for: eight (at
    most 32 registers) for a row reduction of a short chain, six (40) for other
    short chains, four (64) for a long one."""
    if len(em.lines) <= 4 and mode == "rows":
        return 8
    return 6 if len(em.lines) <= 8 else 4


def fused_reduce_mode(node, leaf_ok=False):
    """How reduce(f(inputs)) can run in one pass over the inputs: 'rows' (the
    last axis), 'cols' (the first axis), 'all', or None (run the chain into a
    temporary first).  A plain array as operand goes to the library kernels
    unless `leaf_ok` (a post-chain is to be fused into the generated kernel)."""
    src = node.inputs[0]
    if node.op not in _FUSED_REDUCE_OPS + _FUSED_ARG_OPS or src.kind in ("arg", "const") or not node_reads(src):
        return None
    if src.kind == "leaf" and not leaf_ok:
        return None
    if src.dtype.name not in _REDUCE_KERNEL_DTYPES:
        return None
    nd, axis = len(src.shape), node.value
    if node.op in _FUSED_ARG_OPS:
        # the position of the extreme value of every row, one warp per row
        return "rows" if nd >= 2 and axis == nd - 1 and src.shape[-1] % 4 == 0 else None
    if axis is None or nd == 1:
        return "all"
    if axis == nd - 1:
        return "rows"
    if axis == 0:
        return "cols"
    return None


def _emit_reduce_fused(trace, node, mode, dst, post=None):
    """One kernel for reduce(chain): the chain's inputs are read once.  `post`
    is an elementwise chain over the reduced value alone (its root node): it is
    applied to every result on its way out, so sqrt(sum(...)) or a mean's
    division need no launch of their own."""
    src = node.inputs[0]
    shape = src.shape
    n = int(np.prod(shape, dtype=np.int64))
    em = _Emitter(trace, shape)
    expr = em.emit(src)
    results = [(None, expr, _ValueHolder(src.dtype))]
    n_chain = len(em.lines)
    post_expr, out_dt = "racc", node.dtype
    if post is not None:
        em.names[id(node)] = "racc"
        em.sig.append(("racc", node.dtype.name))
        post_expr, out_dt = em.emit(post), post.dtype
    if mode == "rows":
        rows, cols = n // shape[-1], shape[-1]
    elif mode == "cols":
        rows, cols = shape[0], n // shape[0]
    else:
        rows, cols = 1, n
    vec_ok = mode == "all" or cols % 4 == 0
    for slot, kind, params, dt in em.leaves:
        arr = trace.arrays[slot]
        unit = 4 * dt.itemsize if dt.itemsize <= 4 else 16
        if kind in ("full", "row") and arr.ptr % unit:
            vec_ok = False
        if kind in ("row", "col") and params[0] % 4:
            vec_ok = False
    vec = 4 if vec_ok else 1
    n_streams = sum(1 for _s, k, _p, _d in em.leaves if k == "full")
    unroll = 4 if n_streams <= 2 else 2
    sms = (148 if trace.dry else trace.queue.sm_count) * reduce_resident(em, mode)  # residency slots
    block_row = mode == "rows" and cols >= 8192 and rows < sms and node.op not in _FUSED_ARG_OPS
    acc_dt = node.dtype
    # column reductions: one group of 256 * vec columns per block (four groups,
    # whole 16 KB rows per block, measured slower: 66 us against 61 us)
    col_vecs = 1
    shaped = any(k == "strided" for _s, k, _p, _d in em.leaves)
    sig = ("reduce", mode, node.op, acc_dt.name, block_row, col_vecs, tuple(shape) if shaped else len(shape),
           tuple((k, p if k == "strided" else (), d.name) for _s, k, p, d in em.leaves),
           tuple(em.sig), (expr, src.dtype.name), (n_chain, post_expr, np.dtype(out_dt).name), vec, unroll,
           trace.fastmath)
    hit = _kernel_cache.get(sig)
    if hit is None:
        hit = _generate(em, results, shape, vec, unroll, [None], trace.fastmath,
                        reduce=(mode, node.op, acc_dt, block_row, col_vecs, n_chain, post_expr, out_dt))
        _kernel_cache[sig] = hit
    blob, kname = hit

    params = []
    for slot, kind, p, dt in em.leaves:
        params.append(("slot", slot))
        if kind in ("row", "col"):
            params.append(("i64", p[0]))
    for index, dt in em.scalar_args:
        params.append(("scalar", index, dt))
    params.append(("slot", dst))
    if mode == "rows":
        units = rows if block_row else (rows + 7) // 8
        grid = (max(1, min(units, sms)),)
        params += [("i64", rows), ("i64", cols)]
    elif mode == "cols":
        gx = (cols + 256 * vec * col_vecs - 1) // (256 * vec * col_vecs)
        gy = max(1, min((sms + gx - 1) // gx, (rows + 31) // 32, 65535))
        groups = (gy + 15) // 16  # the device merges row blocks in groups of 16 (kColFanIn)
        if gx * (groups + 1) * 4 > 65536 - 4:
            return False  # more column tiles than ticket counters
        grid = (gx, gy)
        params += [("scratch", (gy + groups) * cols * acc_dt.itemsize), ("i64", rows), ("i64", cols)]
    else:
        tile = 256 * vec * unroll
        grid = (max(1, min((n + tile - 1) // tile, sms)),)
        params += [("scratch", grid[0] * acc_dt.itemsize), ("i64", n)]
    step = ("launch", blob, kname, grid, (256,), tuple(params))
    trace.steps.append(step)
    if not trace.dry:
        run_launch(trace.queue, step, trace.arrays, trace.args)
    return True


def _generate(em, results, out_shape, vec, unroll, ostrides, fastmath=False, shared_in=frozenset(),
              shared_out=frozenset(), reduce=None):
    """CUDA C for one fused chain; returns (tagged source blob, kernel name).
    With `reduce` = (mode, op, accumulator dtype, block_row, column groups per
    thread, number of chain lines before the post-chain, post expression, output
    dtype) the single result is not stored but reduced on the way
    (nmb::reduce_*_fused); the lines after the chain's own and the post
    expression turn the reduced value `racc` into what is stored."""
    members, ctor, kparams = [], [], []
    in_fields, loads = [], []
    nd = len(out_shape)
    for i, (slot, kind, p, dt) in enumerate(em.leaves):
        ct = ctype(dt)
        restrict = "" if i in shared_in else " __restrict__"
        ldg = "*" if i in shared_in else "__ldg"
        members.append(f"const {ct}*{restrict} in{i};")
        kparams.append(f"const {ct}*{restrict} in{i}")
        ctor.append(f"in{i}")
        in_fields.append(f"nmb::Vec<{ct}, V> in{i};")
        if kind == "full":
            loads.append(f"r.in{i} = nmb::load_stream<{ct}, V>(in{i} + i);")
        elif kind == "splat":
            loads.append(f"{{ const {ct} x = {ldg}(in{i}); for (int l = 0; l < V; ++l) r.in{i}.v[l] = x; }}")
        elif kind == "row":
            members.append(f"int64_t m{i};")
            kparams.append(f"int64_t m{i}")
            ctor.append(f"m{i}")
            # i % m without a 64-bit division when m is a power of two or the index fits 32 bits
            loads.append(f"r.in{i} = nmb::load_reuse<{ct}, V>(in{i} + nmb::wrap_index(i, m{i}));")
        elif kind == "col":
            members.append(f"int64_t m{i};")
            kparams.append(f"int64_t m{i}")
            ctor.append(f"m{i}")
            loads.append(f"{{ const {ct} x = __ldg(in{i} + (i / m{i})); for (int l = 0; l < V; ++l) r.in{i}.v[l] = x; }}")
        else:  # strided: decompose the flat index over the output shape
            body = [f"for (int l = 0; l < V; ++l) {{ int64_t rem = i + l, off = 0, q;"]
            for d in range(nd - 1, -1, -1):
                if p[d] != 0:
                    body.append(f"q = rem % {out_shape[d]}ll; off += q * ({p[d]}ll); rem /= {out_shape[d]}ll;")
                else:
                    body.append(f"rem /= {out_shape[d]}ll;")
            body.append(f"r.in{i}.v[l] = {ldg}(in{i} + off); }}")
            loads.append(" ".join(body))
    if em.uses_index:
        in_fields.append("int64_t base;")  # flat position of the step's first element
        loads.append("r.base = i;")
    for j, (index, dt) in enumerate(em.scalar_args):
        members.append(f"{ctype(dt)} s{j};")
        kparams.append(f"{ctype(dt)} s{j}")
        ctor.append(f"s{j}")
    out_fields, stores, out_assign = [], [], []
    for j, (slot, expr, arr) in enumerate(results):
        ct = ctype(arr.dtype)
        out_fields.append(f"nmb::Vec<{ct}, V> out{j};")
        out_assign.append(f"o.out{j}.v[l] = {expr};")
        if reduce is not None:
            continue
        restrict = "" if j in shared_out else " __restrict__"
        members.append(f"{ct}*{restrict} out{j};")
        kparams.append(f"{ct}*{restrict} out{j}")
        ctor.append(f"out{j}")
        if ostrides[j] is None:
            stores.append(f"nmb::store_stream<{ct}, V>(out{j} + i, o.out{j});")
        else:  # a strided view: decompose the flat index over the output shape
            body = ["for (int l = 0; l < V; ++l) { int64_t rem = i + l, off = 0;"]
            for d in range(nd - 1, -1, -1):
                body.append(f"off += (rem % {out_shape[d]}ll) * ({ostrides[j][d]}ll); rem /= {out_shape[d]}ll;")
            body.append(f"out{j}[off] = o.out{j}.v[l]; }}")
            stores.append(" ".join(body))
    nl = "\n      "
    funcs = "\n".join(em.funcs.values())
    chain_lines, post_method = em.lines, ""
    if reduce is not None:
        n_chain, post_expr, out_dt = reduce[5], reduce[6], reduce[7]
        chain_lines = em.lines[:n_chain]
        post_method = (f"  __device__ __forceinline__ {ctype(out_dt)} post({ctype(reduce[2])} racc) const {{\n    "
                       + "\n    ".join(em.lines[n_chain:]) + f"\n    return {post_expr};\n  }}\n")
    if reduce is None:
        kparams.append("int64_t n")
        kernel = f"""extern "C" __global__ void __launch_bounds__(256) nmb_fused({', '.join(kparams)}) {{
  Chain chain{{{', '.join(ctor)}}};
  nmb::eltwise_tile<256, {vec}, {unroll}>(chain, n);
}}"""
        kname = "nmb_fused"
    else:
        mode, op, acc_dt, block_row, col_vecs = reduce[:5]
        act, oct = ctype(acc_dt), ctype(reduce[7])
        opc, ident = {"sum": ("nmb::OpAdd", f"{act}(0)"), "prod": ("nmb::OpMul", f"{act}(1)"),
                      "min": ("nmb::OpMin", f"nmb::neutral_min<{act}>()"),
                      "max": ("nmb::OpMax", f"nmb::neutral_max<{act}>()"),
                      "argmin": (None, None), "argmax": (None, None)}[op]
        kname = "nmb_fused_reduce"
        if op in _FUSED_ARG_OPS:
            tail = "int64_t* __restrict__ out, int64_t rows, int64_t cols"
            call = (f"nmb::reduce_rows_arg_fused<256, {vec}, {unroll}, {'true' if op == 'argmin' else 'false'}>"
                    "(chain, rows, cols, out);")
        elif mode == "rows":
            tail = f"{oct}* __restrict__ out, int64_t rows, int64_t cols"
            call = (f"__shared__ {act} scratch[32];\n  nmb::reduce_rows_fused<256, {vec}, {unroll}, "
                    f"{'true' if block_row else 'false'}>(chain, rows, cols, out, {opc}(), {ident}, scratch);")
        elif mode == "cols":
            tail = (f"{oct}* __restrict__ out, {act}* partials, uint32_t* counters, int64_t rows, "
                    "int64_t cols")
            call = (f"nmb::reduce_cols_fused<256, {vec}, {col_vecs}, {unroll}>(chain, rows, cols, "
                    f"out, partials, counters, {opc}(), {ident});")
        else:
            tail = f"{oct}* __restrict__ out, {act}* partials, uint32_t* counters, int64_t n"
            call = (f"__shared__ {act} scratch[32];\n  nmb::reduce_all_fused<256, {vec}, {unroll}>(chain, n, "
                    f"out, partials, counters, {opc}(), {ident}, scratch);")
        # compiled for `resident` blocks per multiprocessor: the host launches one
        # block per residency slot, rows and tiles go round robin
        kernel = f"""extern "C" __global__ void __launch_bounds__(256, {reduce_resident(em, mode)}) nmb_fused_reduce({', '.join(kparams + [tail])}) {{
  Chain chain{{{', '.join(ctor)}}};
  {call}
}}"""
    scalar_loop = f"""#pragma unroll
    for (int l = 0; l < V; ++l) {{
      {nl.join(list(chain_lines) + out_assign)}
    }}"""
    # under fastmath a*b+c may contract, so every product is packed too and the
    # assembler's merging of packed multiply and add is welcome
    n_packed = sum(1 for i, hit in em.packable.items()
                   if i < len(chain_lines) and (fastmath or not (hit[0] == "mul2" and f"t{i}" in em.scalar_only)))
    if n_packed:
        compute_body = f"""    if constexpr (V % 2 == 0) {{
#pragma unroll
    for (int l = 0; l < V; l += 2) {{
      {nl.join(_paired_lines(em, chain_lines, out_assign, fuse_ok=fastmath))}
    }}
    }} else {{
{scalar_loop}
    }}"""
    else:
        compute_body = scalar_loop
    # fastmath: a*b+c may contract and division/sqrt take the approximate
    # instructions (<= 2 ulp), as the reference's fast SPIR-V mode allows
    head = "//NMB200:OPTIONS\n#define NMB_FASTMATH 1" if fastmath else "//NMB200:OPTIONS --fmad=false"
    src = f"""//NMB200:CUDA-SOURCE
{head}
#include "nmb_device.cuh"
{funcs}
struct Chain {{
  {(nl[:-4]).join(members)}
  template <int V> struct In {{ {' '.join(in_fields) or 'int unused;'} }};
  template <int V> struct Out {{ {' '.join(out_fields)} }};
  template <int V> __device__ __forceinline__ void load(int64_t i, In<V>& r) const {{
    {(nl[:-2]).join(loads)}
  }}
  template <int V> __device__ __forceinline__ void compute(const In<V>& r, Out<V>& o) const {{
{compute_body}
  }}
{post_method}
  template <int V> __device__ __forceinline__ void store(int64_t i, const Out<V>& o) const {{
    {(nl[:-2]).join(stores)}
  }}
}};
{kernel}
"""
    return src.encode(), kname


# ------------------------------------------------------------- execution ----
def run_launch(queue, step, arrays, args):
    _tag, blob, kname, grid, block, params = step
    kernel = queue.get_kernel(queue.load_module(blob), kname)
    packed = []
    for p in params:
        if p[0] == "slot":
            packed.append(("ptr", arrays[p[1]].ptr))
        elif p[0] == "i64":
            packed.append(np.int64(p[1]))
        elif p[0] == "scratch":
            # partials of `p[1]` bytes, then the ticket counters, in the queue's scratch
            counters, data = queue.scratch(p[1])
            packed.append(("ptr", data))
            packed.append(("ptr", counters))
        else:
            packed.append(p[2].type(args[p[1]]))
    queue.launch(kernel, grid, block, packed)


def assign(target, value):
    """Eager `target[...] = value` outside a traced function."""
    trace = Trace(target.queue)
    with _TraceScope(trace):
        slot = trace.add_arg_slot(None, target)
        trace.leaf(slot)[...] = value if not isinstance(value, DeviceArray) else trace.leaf(
            trace.add_arg_slot(None, value))
        trace.flush()


# ------------------------------------------------------------------ plans ---
class Plan:
    """Recorded launches of one traced call, replayable on new arguments of
    the same signature."""

    def __init__(self, trace, result_spec):
        self.slots = trace.slots
        self.steps = trace.steps
        self.result_spec = result_spec
        self.queue = trace.queue
        self._native = {}  # queue -> launches as the native launch path takes them
        self.native_ok = self._native_form() is not None

    def _native_form(self):
        """The plan as (kernel source, kernel name, grid, block, codes, sources)
        per launch when it consists only of launches over the call's own
        arguments (no temporaries, reductions or products) and returns nothing
        or arguments: such a plan is replayed by the native launch path.  None
        otherwise."""
        from .runtime import param_code

        launches = []
        for step in self.steps:
            if step[0] != "launch":
                return None
            _tag, blob, kname, grid, block, params = step
            codes, sources = [], []
            for p in params:
                if p[0] == "slot":
                    s = self.slots[p[1]]
                    if s[0] != "arg":
                        return None
                    codes.append(b"p")
                    sources.append(s[1])
                elif p[0] == "i64":
                    codes.append(b"k")
                    sources.append(int(p[1]))
                elif p[0] == "scalar":
                    codes.append(param_code(p[2]))
                    sources.append(p[1])
                else:
                    return None
            launches.append((blob, kname, tuple(grid), tuple(block), b"".join(codes), tuple(sources)))
        for i in _result_slots(self.result_spec):
            if self.slots[i][0] != "arg":
                return None
        return launches

    def replay_native(self, args, queue):
        """`replay` for a plan in native form: one call into the native launch
        path, which reads the pointers and scalars out of `args` itself."""
        from . import runtime as _rt

        spec = self._native.get(queue)
        if spec is None:
            spec = self._native[queue] = tuple(
                (queue.get_kernel(queue.load_module(blob), kname), grid, block, codes, sources)
                for blob, kname, grid, block, codes, sources in self._native_form())
        try:
            _rt.fastcall().replay(queue.handle, spec, args)
        except RuntimeError:
            _rt.check()
            raise
        spec_r = self.result_spec
        if spec_r is None:
            return None
        return _build_result(spec_r, _ArgSlots(self.slots, args))

    def replay(self, args, queue=None):
        """Runs the recorded steps on `args`; allocations and launches go to
        `queue` (the queue of the call's arguments), the recording queue by
        default."""
        from . import contraction, reduce_ops

        slots = self.slots
        arrays = [None] * len(slots)

        def get(i):
            arr = arrays[i]
            if arr is None:
                s = slots[i]
                if s[0] == "arg":
                    arr = args[s[1]]
                elif s[0] == "view":
                    base, op = get(s[1]), s[2]
                    arr = _apply_view(base, op)
                else:
                    raise RuntimeError("plan slot used before its allocation")
                arrays[i] = arr
            return arr

        q = queue if queue is not None else self.queue
        for step in self.steps:
            tag = step[0]
            if tag == "alloc":
                s = slots[step[1]]
                arrays[step[1]] = empty(s[1], s[2], queue=q)
            elif tag == "launch":
                for p in step[5]:
                    if p[0] == "slot":
                        get(p[1])
                run_launch(q, step, arrays, args)
            elif tag == "reduce":
                reduce_ops.reduce(get(step[3]), step[1], step[2], out=get(step[4]))
            elif tag == "dot":
                contraction.gemm(get(step[1]), get(step[2]), get(step[3]), blocking=False)
            elif tag == "contract":
                run_contract(step, get)
            elif tag == "parfor":
                # a `prange` loop cut out of the function: its own compiled kernel
                real = [get(s[1]) if s[0] == "slot" else args[s[1]] if s[0] == "arg" else s[1] for s in step[2]]
                step[1]._call_parfor(tuple(real))
        for i in _result_slots(self.result_spec):
            get(i)
        return _build_result(self.result_spec, arrays)


class _ArgSlots:
    """Indexable like a plan's array list, for plans whose slots are arguments."""

    def __init__(self, slots, args):
        self.slots, self.args = slots, args

    def __getitem__(self, i):
        return self.args[self.slots[i][1]]


def _result_slots(spec):
    if spec is None:
        return []
    if spec[0] == "slot":
        return [spec[1]]
    if spec[0] == "tuple":
        return [i for s in spec[1] for i in _result_slots(s)]
    return []


def _build_result(spec, arrays):
    if spec is None:
        return None
    if spec[0] == "slot":
        return arrays[spec[1]]
    if spec[0] == "tuple":
        return tuple(_build_result(s, arrays) for s in spec[1])
    return spec[1]  # ("value", x)


def signature_of(args):
    """Cache key of a recorded plan: per-argument layout plus, when array
    arguments share memory, how they overlap (the order of the recorded
    kernels depends on it)."""
    sig = []
    extents = []
    for i, a in enumerate(args):
        if isinstance(a, DeviceArray):
            sig.append(a.trace_sig)
            extents.append(a.extent + (i,))
        elif isinstance(a, (bool, int, float, np.generic)):
            sig.append(("scalar", scalar_dtype(a).name))
        else:
            return None
    if len(extents) > 1:
        extents.sort()
        for k in range(len(extents) - 1):
            j = k + 1
            while j < len(extents) and extents[j][0] < extents[k][1]:
                sig.append(("alias", extents[k][2], extents[j][2], extents[j][0] - extents[k][0]))
                j += 1
    return tuple(sig)


_fake_addresses = itertools.count(0x7F0000000000, 1 << 36)


def _permuted(arr, axes):
    return DeviceArray(arr._buf, [arr.shape[i] for i in axes], arr.dtype, [arr.strides[i] for i in axes],
                       arr._offset)


def _broadcast(arr, shape):
    """View of `arr` with the extent `shape`: new and stretched axes get stride 0."""
    lead = len(shape) - arr.ndim
    strides = [0] * lead + [0 if d == 1 and shape[lead + i] != 1 else st
                            for i, (d, st) in enumerate(zip(arr.shape, arr.strides))]
    return DeviceArray(arr._buf, shape, arr.dtype, strides, arr._offset)


def _apply_view(base, op):
    """The view `op` (recorded by LazyArray._view) of a new base array."""
    if op[0] == "T":
        return base.T
    if op[0] == "reshape":
        return base.reshape(op[1])
    if op[0] == "transpose":
        return _permuted(base, op[1])
    if op[0] == "broadcast":
        return _broadcast(base, op[1])
    return base[op[1]]


def fake_array(shape, dtype, ptr=None):
    """Array descriptor without memory, for code generation without a device;
    every one gets an address range of its own."""
    from .device_array import _Foreign

    dtype = np.dtype(dtype)
    n = int(np.prod(shape, dtype=np.int64))
    if ptr is None:
        ptr = next(_fake_addresses)
    return DeviceArray(_Foreign(None, ptr, n * dtype.itemsize, None), shape, dtype)


# ---- arrays created inside a traced function ------------------------------
# np.empty / zeros / ones / full called with a shape have no array argument, so
# NumPy's protocols never show them to the trace; the function therefore runs
# with its module-level `numpy` name (and any of those functions imported by
# name) bound to stand-ins that hand out device temporaries while a trace is
# active (the reference types numpy.empty, zeros, ones in
# numba_mlir/mlir/numpy/funcs.py and allocates them on the device) and are
# NumPy itself otherwise.
def _shape_of(shape):
    if isinstance(shape, (int, np.integer, LazyArray)):
        shape = (shape,)
    return tuple(int(d) for d in shape)


def _device_empty(shape, dtype=float, order="C", **kwargs):
    trace = current_trace()
    if trace is None or kwargs or order != "C" or np.dtype(dtype).name not in _CTYPE:
        return np.empty(shape, dtype, order, **kwargs)
    return trace.leaf(trace.add_tmp_slot(_shape_of(shape), np.dtype(dtype)))


def _device_filled(np_func, value):
    def create(shape, *args, **kwargs):
        trace = current_trace()
        if value is None:  # np.full(shape, fill_value, dtype=None)
            fill = args[0] if args else kwargs.pop("fill_value")
            rest = args[1:]
            dtype = rest[0] if rest else kwargs.pop("dtype", None)
            if dtype is None:
                dtype = scalar_dtype(fill) if isinstance(fill, (bool, int, float, np.generic)) else None
        else:
            fill = value
            dtype = args[0] if args else kwargs.pop("dtype", float)
            rest = args[1:]
        if trace is None or kwargs or rest[1:] or dtype is None or np.dtype(dtype).name not in _CTYPE \
                or not isinstance(fill, (bool, int, float, np.generic, LazyArray)):
            return np_func(shape, *args, **kwargs)
        out = trace.leaf(trace.add_tmp_slot(_shape_of(shape), np.dtype(dtype)))
        out[...] = fill if isinstance(fill, LazyArray) else np.dtype(dtype).type(fill)
        return out

    create.__name__ = np_func.__name__
    return create


def _index_array(trace, shape, axis):
    """int64 array whose elements are their own coordinate along `axis`."""
    return LazyArray(trace, Node("index", np.int64, shape, value=axis))


def _device_arange(*args, dtype=None, **kwargs):
    """np.arange with host scalars: start + step * (the element's position)."""
    trace = current_trace()
    vals = [a.concrete if isinstance(a, LazyArray) and a.concrete is not None else a for a in args]
    if trace is None or kwargs or not vals or not all(isinstance(v, (int, float, np.integer, np.floating))
                                                      for v in vals):
        return np.arange(*args, dtype=dtype, **kwargs)
    start, stop, step = (0, vals[0], 1) if len(vals) == 1 else (vals[0], vals[1], vals[2] if len(vals) > 2 else 1)
    out_dt = np.dtype(dtype) if dtype is not None else np.arange(0, 1, 1).dtype if all(
        isinstance(v, (int, np.integer)) for v in (start, stop, step)) else np.dtype(np.float64)
    if out_dt.name not in _CTYPE or step == 0:
        return np.arange(*args, dtype=dtype)
    n = max(0, int(np.ceil((stop - start) / step)))
    if any(isinstance(a, LazyArray) for a in args):
        trace.value_dependent = True  # the length came from an argument's value
    work = np.dtype(np.int64) if out_dt.kind in "iub" else np.dtype(np.float64)
    res = _index_array(trace, (n,), 0)
    if work.kind == "f":
        res = res.astype(work)
    if step != 1:
        res = res * work.type(step)
    if start != 0:
        res = res + work.type(start)
    return res if res.dtype == out_dt else res.astype(out_dt)


def _device_eye(N, M=None, k=0, dtype=float, order="C", **kwargs):
    trace = current_trace()
    if trace is None or kwargs or order != "C" or np.dtype(dtype).name not in _CTYPE \
            or not all(isinstance(v, (int, np.integer)) for v in (N, k) + (() if M is None else (M,))):
        return np.eye(N, M, k, dtype, order, **kwargs)
    M = N if M is None else M
    diff = _index_array(trace, (1, int(M)), 1) - _index_array(trace, (int(N), 1), 0)  # column - row
    dt = np.dtype(dtype)
    return where(trace, diff == np.int64(k), dt.type(1), dt.type(0))


def _device_layout(np_func, fortran):
    """np.asarray / ascontiguousarray / asfortranarray of a traced array: NumPy
    converts the argument before any protocol could see it, so they are
    routed here.  Column-major order is a transposed view of a C-ordered copy
    of the transpose."""
    def convert(a, dtype=None, **kwargs):
        trace = current_trace()
        if trace is None or not isinstance(a, LazyArray) or kwargs:
            return np_func(a, dtype, **kwargs)
        if dtype is not None and np.dtype(dtype) != a.dtype:
            a = a.astype(dtype)
        if np_func is np.asarray:
            return a
        if not fortran or a.ndim < 2:
            if a.node.kind != "leaf":
                return a
            arr = trace.arrays[a.node.slot]
            return a if arr.is_c_contiguous else a.copy()
        t = trace.leaf(trace.add_tmp_slot(a.shape[::-1], a.dtype))
        t[...] = (a if a.node.kind == "leaf" else trace.leaf(trace.materialize(a))).T
        return t.T

    convert.__name__ = np_func.__name__
    return convert


_CREATORS = {np.asarray: _device_layout(np.asarray, False),
             np.ascontiguousarray: _device_layout(np.ascontiguousarray, False),
             np.asfortranarray: _device_layout(np.asfortranarray, True),
             np.arange: _device_arange, np.eye: _device_eye, np.empty: _device_empty, np.zeros: _device_filled(np.zeros, 0), np.ones: _device_filled(np.ones, 1),
             np.full: _device_filled(np.full, None)}


class _NumpyStandIn:
    """`numpy` as the traced function sees it: everything is NumPy's except the
    array creators above."""

    def __getattr__(self, name):
        value = getattr(np, name)
        try:
            return _CREATORS.get(value, value)
        except TypeError:  # unhashable attribute
            return value


_numpy_stand_in = _NumpyStandIn()
_rebound = weakref.WeakKeyDictionary()


def with_device_creators(func):
    """`func` with the module-level names that are NumPy (or one of its array
    creators) rebound to the stand-ins; the function itself when it has none.
    The copy sees the module's other names as they are when it is first made
    (Numba likewise freezes globals when it compiles)."""
    import types

    if not isinstance(func, types.FunctionType):
        return func
    hit = _rebound.get(func)
    if hit is not None:
        return hit
    changes = {}
    for name in func.__code__.co_names:
        value = func.__globals__.get(name)
        if value is np:
            changes[name] = _numpy_stand_in
        else:
            try:
                if value in _CREATORS:
                    changes[name] = _CREATORS[value]
            except TypeError:
                pass
    if not changes:
        new = func
    else:
        scope = dict(func.__globals__)
        scope.update(changes)
        new = types.FunctionType(func.__code__, scope, func.__name__, func.__defaults__, func.__closure__)
        new.__kwdefaults__ = func.__kwdefaults__
    _rebound[func] = new
    return new


def trace_call(func, args, queue, dry=False, fastmath=False):
    """Runs `func` on symbolic arguments, executing the device work as it is
    recorded (unless `dry`).  Returns (result, plan or None)."""
    func = with_device_creators(func)
    trace = Trace(queue, args, dry=dry, fastmath=fastmath)
    with _TraceScope(trace):
        sym = []
        for i, a in enumerate(args):
            if isinstance(a, DeviceArray):
                slot = trace.add_arg_slot(i, a)
                sym.append(trace.leaf(slot))
            elif isinstance(a, (bool, int, float, np.generic)):
                dt = scalar_dtype(a)
                sym.append(LazyArray(trace, Node("arg", dt, (), value=i), concrete=dt.type(a)))
            else:
                sym.append(a)
        res = func(*sym)
        spec = _result_spec(trace, res)
        trace.flush()
    result = _build_result(spec, trace.arrays)
    plan = None if trace.value_dependent else Plan(trace, spec)
    if dry:
        return trace, plan
    return result, plan


def _result_spec(trace, res):
    if res is None:
        return None
    if isinstance(res, LazyArray):
        if res.shape == () and res.concrete is not None and res.node.kind != "leaf":
            trace.value_dependent = True  # scalar computed on the host
            return ("value", res.concrete)
        return ("slot", trace.materialize(res))
    if isinstance(res, tuple):
        return ("tuple", tuple(_result_spec(trace, r) for r in res))
    return ("value", res)
