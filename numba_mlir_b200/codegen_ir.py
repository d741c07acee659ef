"""Typed Numba IR -> CUDA C, for `@kernel` bodies and scalar device functions.

The reference types kernel bodies with Numba's own type inference and then
lowers the typed IR through MLIR to SPIR-V (numba_mlir/mlir/inner_compiler.py:21-59,
numba_mlir/mlir_compiler/lib/Lowering.cpp:311-1290).  Here the same typed IR
(bytecode -> Numba IR -> SSA -> nopython type inference, Numba's stock passes)
is translated to CUDA C: one labelled C block per IR block, every Numba
variable a C local of its inferred type, every operation cast to the types its
Numba signature names, so the arithmetic is the arithmetic Numba's CPU target
performs.  The source is compiled by NVRTC inside gpuxModuleLoad.
"""

import math
import operator
import re

import numpy as np

from . import lazy


class UnsupportedError(TypeError):
    pass


# ------------------------------------------------------------- typed IR -----
_capture_pipeline = None


def _get_pipeline():
    global _capture_pipeline
    if _capture_pipeline is not None:
        return _capture_pipeline
    from numba.core import ir
    from numba.core.compiler import CompilerBase, DefaultPassBuilder
    from numba.core.compiler_machinery import FunctionPass, register_pass
    from numba.core.typed_passes import NopythonTypeInference, PreLowerStripPhis
    from numba.core.untyped_passes import IRProcessing

    from . import kernel_impl

    @register_pass(mutates_CFG=False, analysis_only=False)
    class ResolveKernelApiAttrs(FunctionPass):
        """`atomic.add`, `local.array`, `group.reduce_add` ... written inline:
        getattr on the API namespace objects becomes the global function, so
        the plain `infer_global` typing applies (the reference leaves this form
        unsupported, mlir/tests/test_gpu.py:848-855)."""

        _name = "nmb_resolve_kernel_api_attrs"

        def __init__(self):
            FunctionPass.__init__(self)

        def run_pass(self, state):
            func_ir = state.func_ir
            defs = {}
            for blk in func_ir.blocks.values():
                for inst in blk.body:
                    if isinstance(inst, ir.Assign) and isinstance(inst.value, (ir.Global, ir.FreeVar)):
                        defs[inst.target.name] = inst.value.value
            changed = False
            for blk in func_ir.blocks.values():
                for inst in blk.body:
                    if (isinstance(inst, ir.Assign) and isinstance(inst.value, ir.Expr)
                            and inst.value.op == "getattr" and inst.value.value.name in defs):
                        owner = defs[inst.value.value.name]
                        fn = kernel_impl.API_ATTRS.get((owner, inst.value.attr))
                        if fn is not None:
                            inst.value = ir.Global(fn.__name__, fn, inst.loc)
                            changed = True
            # The namespace objects themselves have no Numba type; once their
            # attribute reads are gone their loads are dead.
            owners = {o for o, _a in kernel_impl.API_ATTRS}
            for blk in func_ir.blocks.values():
                for inst in blk.body:
                    if (isinstance(inst, ir.Assign) and isinstance(inst.value, (ir.Global, ir.FreeVar))
                            and inst.value.value in owners):
                        inst.value = ir.Const(None, inst.loc)
                        changed = True
            return changed

    @register_pass(mutates_CFG=False, analysis_only=True)
    class CaptureTypedIR(FunctionPass):
        _name = "nmb_capture_typed_ir"

        def __init__(self):
            FunctionPass.__init__(self)

        def run_pass(self, state):
            state.cr = TypedIR(state.func_ir, state.typemap, state.calltypes, state.return_type,
                               state.args)
            return False

    class CapturePipeline(CompilerBase):
        def define_pipelines(self):
            pm = DefaultPassBuilder.define_untyped_pipeline(self.state, "nmb_untyped")
            pm.add_pass_after(ResolveKernelApiAttrs, IRProcessing)
            pm.add_pass(NopythonTypeInference, "nopython frontend")
            pm.add_pass(PreLowerStripPhis, "remove phis nodes")
            pm.add_pass(CaptureTypedIR, "capture typed IR")
            pm.finalize()
            return [pm]

    _capture_pipeline = CapturePipeline
    return CapturePipeline


class TypedIR:
    def __init__(self, func_ir, typemap, calltypes, return_type, args):
        self.func_ir = func_ir
        self.typemap = typemap
        self.calltypes = calltypes
        self.return_type = return_type
        self.args = args


def typed_ir(py_func, argtypes):
    """Runs Numba's front-end and type inference on `py_func`."""
    from numba.core import compiler
    from numba.core.registry import cpu_target

    from . import kernel_impl  # noqa: F401  (registers the API typing)

    flags = compiler.Flags()
    flags.nrt = True
    return compiler.compile_extra(
        cpu_target.typing_context, cpu_target.target_context, py_func, tuple(argtypes), None,
        flags, {}, pipeline_class=_get_pipeline())


# ----------------------------------------------------------- C helpers ------
def _nb_types():
    from numba.core import types

    return types


def c_scalar_type(t):
    types = _nb_types()
    t = types.unliteral(t)
    if isinstance(t, types.Boolean):
        return "bool"
    if isinstance(t, types.Integer):
        return ("int" if t.signed else "uint") + str(t.bitwidth) + "_t"
    if isinstance(t, types.Float):
        return {32: "float", 64: "double"}[t.bitwidth]
    raise UnsupportedError(f"type {t} has no device representation")


def _is_scalar(t):
    types = _nb_types()
    t = types.unliteral(t)
    return isinstance(t, (types.Boolean, types.Integer, types.Float))


def _const_literal(value, t):
    types = _nb_types()
    t = types.unliteral(t)
    if isinstance(t, types.Boolean):
        return "true" if value else "false"
    if isinstance(t, types.Integer):
        v = int(value)
        if v == -(2**63):
            return "(int64_t)0x8000000000000000ull"
        suffix = "ll" if t.signed else "ull"
        return f"({c_scalar_type(t)}){v}{suffix}"
    if isinstance(t, types.Float):
        return lazy.literal(value, np.float32 if t.bitwidth == 32 else np.float64)
    raise UnsupportedError(f"constant of type {t}")


class _NameRef:
    """Stands in for an ir.Var where only the name is needed."""

    def __init__(self, name):
        self.name = name


class ArrayRep:
    """C variables describing one array value: data pointer, shape, element
    strides."""

    def __init__(self, name, nbtype, index_ctype="int64_t"):
        self.name = name
        self.dtype = nbtype.dtype
        self.ndim = nbtype.ndim
        self.ctype = c_scalar_type(nbtype.dtype)
        self.index_ctype = index_ctype
        self.ptr = f"{name}_p"
        self.shape = [f"{name}_s{d}" for d in range(self.ndim)]
        self.strides = [f"{name}_t{d}" for d in range(self.ndim)]

    def decls(self):
        out = [f"{self.ctype}* {self.ptr};"]
        if self.ndim:
            out.append(f"{self.index_ctype} " + ", ".join(self.shape + self.strides) + ";")
        return out


_MATH_FUNCS = {
    # name: (float32 form, float64 form)
    "sqrt": ("nmb::f_sqrt({0})", "nmb::f_sqrt({0})"), "exp": ("nmb::f_exp({0})", "nmb::f_exp({0})"),
    "log": ("nmb::f_log({0})", "nmb::f_log({0})"), "erf": ("nmb::f_erf({0})", "nmb::f_erf({0})"),
    "sin": ("sinf({0})", "sin({0})"), "cos": ("cosf({0})", "cos({0})"),
    "tan": ("tanf({0})", "tan({0})"), "tanh": ("tanhf({0})", "tanh({0})"),
    "floor": ("floorf({0})", "floor({0})"), "ceil": ("ceilf({0})", "ceil({0})"),
    "fabs": ("fabsf({0})", "fabs({0})"), "acos": ("acosf({0})", "acos({0})"),
    "asin": ("asinf({0})", "asin({0})"), "atan": ("atanf({0})", "atan({0})"),
    "atan2": ("atan2f({0}, {1})", "atan2({0}, {1})"), "pow": ("powf({0}, {1})", "pow({0}, {1})"),
    "log2": ("log2f({0})", "log2({0})"), "log10": ("log10f({0})", "log10({0})"),
    "erfc": ("erfcf({0})", "erfc({0})"), "expm1": ("expm1f({0})", "expm1({0})"),
    "log1p": ("log1pf({0})", "log1p({0})"), "sinh": ("sinhf({0})", "sinh({0})"),
    "cosh": ("coshf({0})", "cosh({0})"),
}
_NP_TO_MATH = {"arccos": "acos", "arcsin": "asin", "arctan": "atan", "arctan2": "atan2",
               "absolute": "fabs", "power": "pow"}

_BINOPS = {
    operator.add: "+", operator.sub: "-", operator.mul: "*", operator.iadd: "+", operator.isub: "-",
    operator.imul: "*", operator.lt: "<", operator.le: "<=", operator.gt: ">", operator.ge: ">=",
    operator.eq: "==", operator.ne: "!=", operator.and_: "&", operator.or_: "|", operator.xor: "^",
    operator.iand: "&", operator.ior: "|", operator.ixor: "^", operator.lshift: "<<",
    operator.rshift: ">>", operator.ilshift: "<<", operator.irshift: ">>",
}
_DIVS = {operator.truediv: "true", operator.itruediv: "true", operator.floordiv: "floor",
         operator.ifloordiv: "floor", operator.mod: "mod", operator.imod: "mod",
         operator.pow: "pow", operator.ipow: "pow"}


_NARROW_BINOPS = (operator.add, operator.sub, operator.mul, operator.iadd, operator.isub, operator.imul,
                  operator.floordiv, operator.ifloordiv, operator.mod, operator.imod, operator.and_,
                  operator.or_, operator.xor, operator.iand, operator.ior, operator.ixor, operator.lshift,
                  operator.rshift, operator.ilshift, operator.irshift)


def index_like_vars(tir):
    """Names of the integer variables (and tuples, ranges, iterators of them)
    whose every definition is an index computation: work-item ids and sizes,
    array shapes, loop counters of ranges over such values, integer constants
    below 2^31, and sums, products, quotients, shifts, min/max of those.  They
    can live in 32 bits when the caller promised 32-bit indexing.  Values read
    from arrays, scalar kernel arguments and results of other calls stay wide.
    Greatest fixed point: every candidate starts narrow and is dropped when one
    of its definitions depends on something wide."""
    from numba.core import ir, types

    from . import kernel_impl as K

    typemap = tir.typemap

    def candidate(name):
        t = types.unliteral(typemap.get(name))
        if isinstance(t, types.Integer) and t.bitwidth == 64:
            return True
        if isinstance(t, (types.UniTuple, types.Tuple, types.NamedUniTuple)):
            return len(t.types) > 0 and all(isinstance(types.unliteral(e), types.Integer) for e in t.types)
        if isinstance(t, (types.RangeType, types.RangeIteratorType)):
            return True
        if isinstance(t, types.Pair):
            return isinstance(types.unliteral(t.first_type), types.Integer)
        return False

    defs = {}
    consts = {}
    for blk in tir.func_ir.blocks.values():
        for inst in blk.body:
            if isinstance(inst, ir.Assign):
                defs.setdefault(inst.target.name, []).append(inst.value)
                if isinstance(inst.value, (ir.Global, ir.FreeVar, ir.Const)):
                    consts[inst.target.name] = inst.value.value
    narrow = {name for name in defs if candidate(name)}

    def small(v):
        if isinstance(v, (bool, np.bool_)):
            return True
        if isinstance(v, (int, np.integer)):
            return -2**31 < int(v) < 2**31
        if isinstance(v, tuple):
            return all(small(x) for x in v)
        return False

    def ok(var):
        """`var` (an operand) is narrow, or of a type that fits 32 bits anyway."""
        if var.name in narrow:
            return True
        t = types.unliteral(typemap.get(var.name))
        return isinstance(t, types.Boolean) or (isinstance(t, types.Integer) and t.bitwidth <= 32)

    def callee(expr):
        fv = expr.func.name
        if fv in consts:
            return consts[fv]
        t = typemap.get(fv)
        key = getattr(t, "typing_key", None)
        if key is None:
            key = getattr(t, "key", None)
            if isinstance(key, tuple):
                key = key[0]
        return key

    def def_ok(value):
        if isinstance(value, ir.Arg):
            return False
        if isinstance(value, (ir.Global, ir.FreeVar, ir.Const)):
            return small(value.value)
        if isinstance(value, ir.Var):
            return ok(value)
        if not isinstance(value, ir.Expr):
            return False
        op = value.op
        if op in ("binop", "inplace_binop"):
            return value.fn in _NARROW_BINOPS and ok(value.lhs) and ok(value.rhs)
        if op == "unary":
            return value.fn in (operator.neg, operator.pos, operator.invert) and ok(value.value)
        if op in ("cast", "exhaust_iter", "getiter", "iternext", "pair_first"):
            return ok(value.value)
        if op == "build_tuple":
            return all(ok(i) for i in value.items)
        if op in ("getitem", "static_getitem"):
            st = types.unliteral(typemap.get(value.value.name))
            return not isinstance(st, types.Array) and ok(value.value)
        if op == "getattr":
            st = types.unliteral(typemap.get(value.value.name))
            return isinstance(st, types.Array) and value.attr in ("shape", "size", "ndim", "strides")
        if op == "call":
            fn = callee(value)
            if fn is range or getattr(fn, "__name__", "") == "prange" or fn in (min, max, abs, int):
                return all(ok(a) for a in value.args)
            if fn in K.ID_FUNCS or fn is len:
                return True
            return False
        return False

    changed = True
    while changed:
        changed = False
        for name in list(narrow):
            if not all(def_ok(v) for v in defs[name]):
                narrow.discard(name)
                changed = True
    return frozenset(narrow)


class Translator:
    """Translates one typed function to a C statement list.

    mode 'kernel': parameters are the kernel's own, `return` leaves the kernel.
    mode 'device': a `__device__` function returning a scalar."""

    def __init__(self, tir, mode, func_name, index32=False, fastmath=False):
        from numba.core import ir, types

        # fastmath: a*b+c may contract, so packed products may feed packed sums
        self.fastmath = bool(fastmath)

        self.ir = ir
        self.types = types
        self.tir = tir
        self.mode = mode
        self.func_name = func_name
        # gpu_use_64bit_index=False (numba_mlir/mlir/target.py:176-203; the
        # reference then types `index` values as i32 in device code,
        # mlir/lib/Conversion/GpuToGpuRuntime.cpp:976-1030): work-item ids, loop
        # counters, shapes, strides and whatever is computed from them alone
        # are 32-bit C variables, and element offsets are 32-bit products.
        self.index32 = bool(index32)
        self.narrow = set(index_like_vars(tir)) if self.index32 else set()
        self.typemap = tir.typemap
        self.calltypes = tir.calltypes
        self.cnames = {}
        self.decls = []           # C declarations at function top
        self.declared = set()
        self.shared_decls = []
        self.local_arrays = []   # (index in shared_decls, name, C type, bytes) of local.array buffers
        self.consts = {}          # var name -> compile-time Python object
        self.tuples = {}          # var name -> list of element reps (C exprs / nested)
        self.arrays = {}          # var name -> ArrayRep
        self.written_params = set()
        self.alias = {}           # array var -> root (param) var
        self.uses_barrier = False
        self.uses_group_reduce = False
        self.counter = 0
        self.par_ranges = {}      # range variable -> (id expr, count expr): grid-strided loops
        self.block_prologue = {}  # block label -> C statements placed at its start
        self.block_epilogue = {}  # block label -> C statements placed before its terminator
        self.return_store = None  # parfor mode: C lvalue the scalar return value is written to

    # naming -------------------------------------------------------------------
    def cname(self, name):
        c = self.cnames.get(name)
        if c is None:
            base = re.sub(r"[^0-9a-zA-Z_]", "_", name).strip("_") or "v"
            c = f"v{len(self.cnames)}_{base}"[:60]
            self.cnames[name] = c
        return c

    def fresh(self, prefix):
        self.counter += 1
        return f"{prefix}{self.counter}"

    def vtype(self, name):
        return self.typemap[name]

    # value representation -------------------------------------------------------
    def declare(self, name):
        """Declares the C storage of Numba variable `name` once."""
        if name in self.declared:
            return
        self.declared.add(name)
        types = self.types
        t = types.unliteral(self.vtype(name))
        c = self.cname(name)
        narrow = name in self.narrow
        if _is_scalar(t):
            self.decls.append(f"{'int32_t' if narrow else c_scalar_type(t)} {c};")
        elif isinstance(t, types.Array):
            rep = ArrayRep(c, t, "int32_t" if self.index32 else "int64_t")
            self.arrays[name] = rep
            self.decls.extend(rep.decls())
        elif isinstance(t, (types.UniTuple, types.Tuple, types.NamedUniTuple)):
            elems = []
            for k, et in enumerate(t.types):
                if not _is_scalar(et):
                    raise UnsupportedError(f"tuple element type {et}")
                self.decls.append(f"{'int32_t' if narrow else c_scalar_type(et)} {c}_e{k};")
                elems.append(f"{c}_e{k}")
            self.tuples[name] = elems
        elif isinstance(t, (types.RangeType, types.RangeIteratorType)):
            self.decls.append(f"{'int32_t' if narrow else 'int64_t'} {c}_a, {c}_b, {c}_c;")
        elif isinstance(t, types.Pair):
            if not _is_scalar(t.first_type):
                raise UnsupportedError(f"iteration over {t.first_type}")
            self.decls.append(f"{'int32_t' if narrow else c_scalar_type(t.first_type)} {c}_v; bool {c}_ok;")
        # everything else (functions, modules, dtypes, None) lives at compile time

    def scalar(self, var, as_type=None):
        """C expression of a scalar Numba variable, optionally cast."""
        name = var.name
        t = self.types.unliteral(self.vtype(name))
        if name in self.consts and _is_scalar(t):
            expr = _const_literal(self.consts[name], t)
        else:
            if not _is_scalar(t):
                raise UnsupportedError(f"{name}: {t} used as a scalar")
            self.declare(name)
            expr = self.cname(name)
        if as_type is not None:
            at = self.types.unliteral(as_type)
            if at != t:
                return self.cast_expr(expr, t, at)
        return expr

    def cast_expr(self, expr, from_t, to_t):
        types = self.types
        to_t = types.unliteral(to_t)
        if isinstance(to_t, types.Boolean):
            return f"(({expr}) != 0)"
        return f"(({c_scalar_type(to_t)})({expr}))"

    def tuple_elems(self, var):
        name = var.name
        if name in self.tuples:
            return self.tuples[name]
        if name in self.consts and isinstance(self.consts[name], tuple):
            t = self.types.unliteral(self.vtype(name))
            return [_const_literal(v, et) for v, et in zip(self.consts[name], t.types)]
        raise UnsupportedError(f"{name} is not a tuple of scalars")

    def index_list(self, var):
        """Index variable -> list of int64 C expressions."""
        t = self.types.unliteral(self.vtype(var.name))
        if _is_scalar(t):
            return [self.scalar(var, self.types.int64)]
        return [f"((int64_t)({e}))" for e in self.tuple_elems(var)]

    def element_ref(self, arr_var, idx_exprs):
        rep = self.arrays[arr_var.name] if arr_var.name in self.arrays else None
        if rep is None:
            self.declare(arr_var.name)
            rep = self.arrays[arr_var.name]
        if len(idx_exprs) != rep.ndim:
            raise UnsupportedError("only full scalar indexing of arrays is supported in kernels")
        if self.index32:
            off = " + ".join(f"(int32_t)({i}) * {s}" for i, s in zip(idx_exprs, rep.strides)) or "0"
        else:
            off = " + ".join(f"({i}) * {s}" for i, s in zip(idx_exprs, rep.strides)) or "0"
        return f"{rep.ptr}[{off}]"

    def root_of(self, name):
        while name in self.alias:
            name = self.alias[name]
        return name

    # expressions ------------------------------------------------------------------
    def assign(self, target, value, out):
        ir, types = self.ir, self.types
        tname = target.name
        ttype = types.unliteral(self.vtype(tname))

        if isinstance(value, ir.Arg):
            self.bind_arg(tname, value.index, out)
            return
        if isinstance(value, (ir.Global, ir.FreeVar, ir.Const)):
            v = value.value
            if _is_scalar(ttype) and isinstance(v, (bool, int, float, np.generic)):
                self.declare(tname)
                out.append(f"{self.cname(tname)} = {_const_literal(v, ttype)};")
                self.consts[tname] = v
            else:
                self.consts[tname] = v
            return
        if isinstance(value, ir.Var):
            self.copy_var(tname, value.name, out)
            return
        if not isinstance(value, ir.Expr):
            raise UnsupportedError(f"IR node {type(value).__name__}")

        op = value.op
        if op in ("binop", "inplace_binop"):
            sig = self.calltypes[value]
            self.declare(tname)
            out.append(f"{self.cname(tname)} = "
                       f"{self.binop(value.fn, value.lhs, value.rhs, sig, tname in self.narrow)};")
        elif op == "unary":
            sig = self.calltypes[value]
            a = self.scalar(value.value, sig.args[0])
            self.declare(tname)
            if value.fn is operator.neg:
                e = f"(-{a})"
            elif value.fn is operator.pos:
                e = a
            elif value.fn is operator.not_:
                e = f"(!({a}))"
            elif value.fn is operator.invert:
                e = f"(~{a})"
            else:
                raise UnsupportedError(f"unary {value.fn}")
            out.append(f"{self.cname(tname)} = {self.cast_expr(e, sig.args[0], sig.return_type)};")
        elif op == "cast":
            src_t = types.unliteral(self.vtype(value.value.name))
            if isinstance(ttype, types.NoneType) or isinstance(src_t, types.NoneType):
                self.consts[tname] = None
            elif _is_scalar(ttype):
                self.declare(tname)
                out.append(f"{self.cname(tname)} = {self.scalar(value.value, ttype)};")
            else:
                self.copy_var(tname, value.value.name, out)
        elif op == "call":
            self.call(target, value, out)
        elif op in ("getitem", "static_getitem"):
            self.getitem(target, value, out)
        elif op == "getattr":
            self.getattr(target, value, out)
        elif op == "build_tuple":
            self.declare(tname)
            for dst, item, et in zip(self.tuples[tname], value.items, ttype.types):
                out.append(f"{dst} = {self.scalar(item, et)};")
        elif op == "exhaust_iter":
            self.copy_var(tname, value.value.name, out)
        elif op == "getiter":
            src_t = types.unliteral(self.vtype(value.value.name))
            if not isinstance(src_t, types.RangeType):
                raise UnsupportedError(f"iteration over {src_t}")
            self.declare(tname)
            s, d = self.cname(value.value.name), self.cname(tname)
            out.append(f"{d}_a = {s}_a; {d}_b = {s}_b; {d}_c = {s}_c;")
        elif op == "iternext":
            self.declare(tname)
            it, d = self.cname(value.value.name), self.cname(tname)
            out.append(f"{d}_ok = {it}_c > 0 ? ({it}_a < {it}_b) : ({it}_a > {it}_b); "
                       f"{d}_v = {it}_a; if ({d}_ok) {it}_a += {it}_c;")
        elif op == "pair_first":
            self.declare(tname)
            out.append(f"{self.cname(tname)} = {self.cast_expr(self.cname(value.value.name) + '_v', None, ttype)};")
        elif op == "pair_second":
            self.declare(tname)
            out.append(f"{self.cname(tname)} = {self.cname(value.value.name)}_ok;")
        else:
            raise UnsupportedError(f"expression '{op}' is not supported in device code")

    def copy_var(self, tname, sname, out):
        types = self.types
        ttype = types.unliteral(self.vtype(tname))
        if sname in self.consts and not _is_scalar(ttype):
            self.consts[tname] = self.consts[sname]
            if not isinstance(ttype, (types.UniTuple, types.Tuple)):
                return
        if _is_scalar(ttype):
            self.declare(tname)
            src = _NameRef(sname)
            out.append(f"{self.cname(tname)} = {self.scalar(src, ttype)};")
        elif isinstance(ttype, types.Array):
            self.declare(tname)
            self.declare(sname)
            d, s = self.arrays[tname], self.arrays[sname]
            self.alias[tname] = sname
            stm = [f"{d.ptr} = {s.ptr};"]
            stm += [f"{a} = {b};" for a, b in zip(d.shape + d.strides, s.shape + s.strides)]
            out.append(" ".join(stm))
        elif isinstance(ttype, (types.UniTuple, types.Tuple, types.NamedUniTuple)):
            self.declare(tname)
            src = self.tuple_elems(_NameRef(sname))
            for a, b, et in zip(self.tuples[tname], src, ttype.types):
                out.append(f"{a} = ({c_scalar_type(et)})({b});")
        elif isinstance(ttype, (types.RangeType, types.RangeIteratorType)):
            self.declare(tname)
            d, s = self.cname(tname), self.cname(sname)
            out.append(f"{d}_a = {s}_a; {d}_b = {s}_b; {d}_c = {s}_c;")
        elif isinstance(ttype, types.NoneType):
            self.consts[tname] = None
        elif sname in self.consts:
            self.consts[tname] = self.consts[sname]
        else:
            raise UnsupportedError(f"cannot copy a value of type {ttype}")

    def binop(self, fn, lhs, rhs, sig, narrow=False):
        """C expression of a binary operation; `narrow`: the result is a 32-bit
        index value (both operands are)."""
        types = self.types
        a = self.scalar(lhs, sig.args[0])
        b = self.scalar(rhs, sig.args[1])
        rt = types.unliteral(sig.return_type)
        at = types.unliteral(sig.args[0])
        if fn in _BINOPS:
            return self.cast_expr(f"({a} {_BINOPS[fn]} {b})", None, rt)
        kind = _DIVS.get(fn)
        if kind == "true":
            return f"nmb::f_div(({c_scalar_type(rt)})({a}), ({c_scalar_type(rt)})({b}))"
        if kind == "floor":
            if isinstance(at, types.Integer):
                ct = "int32_t" if narrow else c_scalar_type(at)
                return f"nmb::py_floordiv(({ct})({a}), ({ct})({b}))"
            return ("floorf" if rt.bitwidth == 32 else "floor") + f"(nmb::f_div({a}, {b}))"
        if kind == "mod":
            if isinstance(at, types.Integer):
                ct = "int32_t" if narrow else c_scalar_type(at)
                return f"nmb::py_mod(({ct})({a}), ({ct})({b}))"
            return f"nmb::py_mod({a}, {b})"
        if kind == "pow":
            if isinstance(rt, types.Integer):
                return f"nmb::i_pow(({c_scalar_type(rt)})({a}), ({c_scalar_type(rt)})({b}))"
            f = "powf" if rt.bitwidth == 32 else "pow"
            return f"{f}(({c_scalar_type(rt)})({a}), ({c_scalar_type(rt)})({b}))"
        raise UnsupportedError(f"binary operator {fn}")

    def getitem(self, target, value, out):
        types = self.types
        src = value.value
        st = types.unliteral(self.vtype(src.name))
        tname = target.name
        ttype = types.unliteral(self.vtype(tname))
        if isinstance(st, types.Array):
            if value.op == "static_getitem" and value.index_var is None:
                idx = value.index if isinstance(value.index, tuple) else (value.index,)
                idx_exprs = [f"{int(i)}ll" for i in idx]
            else:
                idx_exprs = self.index_list(value.index_var if value.op == "static_getitem" else value.index)
            self.declare(tname)
            if isinstance(ttype, types.Array):
                # fewer integer indices than dimensions: a view of the trailing dimensions
                # (numba_mlir/mlir/tests/test_gpu.py:429-452)
                self.declare(src.name)
                srep, trep = self.arrays[src.name], self.arrays[tname]
                k = len(idx_exprs)
                if k + trep.ndim != srep.ndim:
                    raise UnsupportedError("only integer indices (no slices) select sub-arrays in kernels")
                off = " + ".join(f"({i}) * {st_}" for i, st_ in zip(idx_exprs, srep.strides)) or "0"
                stm = [f"{trep.ptr} = {srep.ptr} + ({off});"]
                for d in range(trep.ndim):
                    stm.append(f"{trep.shape[d]} = {srep.shape[d + k]}; {trep.strides[d]} = {srep.strides[d + k]};")
                out.append(" ".join(stm))
                self.alias[tname] = src.name
                return
            out.append(f"{self.cname(tname)} = {self.cast_expr(self.element_ref(src, idx_exprs), None, ttype)};")
        elif isinstance(st, (types.UniTuple, types.Tuple, types.NamedUniTuple)):
            if value.op != "static_getitem" or not isinstance(value.index, int):
                raise UnsupportedError("tuples need constant indices in device code")
            elems = self.tuple_elems(src)
            self.declare(tname)
            out.append(f"{self.cname(tname)} = {self.cast_expr(elems[value.index], None, ttype)};")
        else:
            raise UnsupportedError(f"indexing of {st}")

    def getattr(self, target, value, out):
        types = self.types
        src = value.value
        st = types.unliteral(self.vtype(src.name))
        tname = target.name
        if isinstance(st, types.Array):
            self.declare(src.name)
            rep = self.arrays[src.name]
            if value.attr == "shape":
                self.declare(tname)
                for dst, s in zip(self.tuples[tname], rep.shape):
                    out.append(f"{dst} = {s};")
            elif value.attr == "size":
                self.declare(tname)
                out.append(f"{self.cname(tname)} = " + (" * ".join(rep.shape) or "1") + ";")
            elif value.attr == "ndim":
                self.consts[tname] = rep.ndim
                self.declare(tname)
                out.append(f"{self.cname(tname)} = {rep.ndim};")
            elif value.attr == "dtype":
                self.consts[tname] = st.dtype
            else:
                raise UnsupportedError(f"array attribute .{value.attr}")
        elif src.name in self.consts:
            self.consts[tname] = getattr(self.consts[src.name], value.attr)
        else:
            raise UnsupportedError(f"attribute .{value.attr} of {st}")

    # calls -------------------------------------------------------------------------
    def callee(self, func_var):
        if func_var.name in self.consts:
            return self.consts[func_var.name]
        t = self.vtype(func_var.name)
        key = getattr(t, "typing_key", None)
        if key is None:
            key = getattr(t, "key", None)
            if isinstance(key, tuple):
                key = key[0]
        return key

    def call(self, target, expr, out):
        from . import kernel_impl as K

        types = self.types
        fn = self.callee(expr.func)
        sig = self.calltypes[expr]
        tname = target.name
        rt = types.unliteral(sig.return_type)
        args = list(expr.args)
        if expr.kws:
            # keyword arguments are folded into the positional order of the typed signature
            pysig = getattr(sig, "pysig", None)
            if pysig is None:
                raise UnsupportedError(f"keyword arguments in a call to {fn!r}")
            kw = dict(expr.kws)
            args += [kw[n] for n in list(pysig.parameters)[len(args):] if n in kw]
        c = None

        def sargs():
            return [self.scalar(a, t) for a, t in zip(args, sig.args)]

        if fn is range or (hasattr(fn, "__name__") and fn.__name__ == "prange"):
            self.declare(tname)
            d = self.cname(tname)
            vals = [self.scalar(a, types.int64) for a in args]
            if len(vals) == 1:
                vals = ["0", vals[0], "1"]
            elif len(vals) == 2:
                vals = vals + ["1"]
            if tname in self.par_ranges:
                # a parallel loop: this thread takes iterations id, id + count, ...
                tid, cnt = self.par_ranges[tname]
                out.append(f"{d}_c = {vals[2]}; {d}_a = {vals[0]} + {tid} * {d}_c; {d}_b = {vals[1]}; "
                           f"{d}_c *= {cnt};")
            else:
                out.append(f"{d}_a = {vals[0]}; {d}_b = {vals[1]}; {d}_c = {vals[2]};")
            return
        if fn in K.ID_FUNCS:
            c = f"nmb::k_{fn.__name__}({self.scalar(args[0], types.int64)}, nmb_gs)"
        elif fn in (K.atomic_add, K.atomic_sub):
            arr, idx, val = args
            self.declare(arr.name)
            self.written_params.add(self.root_of(arr.name))
            rep = self.arrays[arr.name]
            ref = self.element_ref(arr, self.index_list(idx))
            v = self.scalar(val, rep.dtype)
            if fn is K.atomic_sub:
                v = f"(-({v}))"
            c = f"nmb::atomic_add(&{ref}, ({rep.ctype})({v}))"
        elif fn is K.barrier:
            self.uses_barrier = True
            out.append("__syncthreads();")
            self.consts[tname] = None
            return
        elif fn is K.mem_fence:
            flags = self.consts.get(args[0].name, K.GLOBAL_MEM_FENCE) if args else K.GLOBAL_MEM_FENCE
            out.append("__threadfence_block();" if flags == K.LOCAL_MEM_FENCE else "__threadfence();")
            self.consts[tname] = None
            return
        elif fn in (K.local_array, K.private_array):
            self.make_array(target, fn is K.local_array, args, out)
            return
        elif fn in K.GROUP_REDUCE:
            self.uses_barrier = True
            ct = c_scalar_type(rt)
            scratch = self.fresh("nmb_red")
            self.shared_decls.append(f"__shared__ {ct} {scratch}[32];")
            opname, neutral = K.GROUP_REDUCE[fn]
            self.uses_group_reduce = True
            c = (f"nmb::group_reduce(({ct})({self.scalar(args[0], rt)}), nmb::{opname}(), "
                 f"nmb::neutral_{neutral}<{ct}>(), {scratch}, nmb_gr_vals, nmb_active, nmb_group_full)")
        elif fn in (math.sqrt, math.exp, math.log, math.erf, math.sin, math.cos, math.tan, math.tanh,
                    math.floor, math.ceil, math.fabs, math.acos, math.asin, math.atan, math.atan2,
                    math.pow, math.log2, math.log10, math.erfc, math.expm1, math.log1p, math.sinh,
                    math.cosh) or isinstance(fn, np.ufunc):
            name = fn.__name__
            name = _NP_TO_MATH.get(name, name)
            if name in ("floor", "ceil") and isinstance(rt, types.Integer):
                a = self.scalar(args[0], types.float64)
                c = f"(({c_scalar_type(rt)}){name}({a}))"
            elif name in _MATH_FUNCS and isinstance(rt, types.Float):
                forms = _MATH_FUNCS[name]
                ops = [self.scalar(a, rt) for a in args]
                c = forms[0 if rt.bitwidth == 32 else 1].format(*ops)
            elif isinstance(fn, np.ufunc) and name in lazy.UFUNCS:
                loop_t = sig.args[0]
                ops = [self.scalar(a, loop_t) for a in args]
                c = lazy.UFUNCS[name][1](np.dtype(str(types.unliteral(loop_t))), *ops)
            else:
                raise UnsupportedError(f"{name} is not supported in device code")
        elif fn is abs:
            a = self.scalar(args[0], rt)
            c = f"nmb::i_abs({a})" if isinstance(rt, types.Integer) else (
                f"fabsf({a})" if rt.bitwidth == 32 else f"fabs({a})")
        elif fn in (min, max):
            ops = [self.scalar(a, rt) for a in args]
            cmp = "<" if fn is min else ">"
            c = ops[0]
            for o in ops[1:]:
                # Python's min/max: keep the earlier operand on ties
                c = f"(({o}) {cmp} ({c}) ? ({o}) : ({c}))"
        elif fn in (int, float, bool) or isinstance(self.vtype(expr.func.name), types.NumberClass) \
                or (isinstance(fn, type) and issubclass(fn, np.generic)):
            src_t = types.unliteral(self.vtype(args[0].name))
            c = self.cast_expr(self.scalar(args[0]), src_t, rt)
        elif fn is len:
            self.declare(args[0].name)
            c = self.arrays[args[0].name].shape[0]
        else:
            raise UnsupportedError(f"call to {fn!r} is not supported in device code")

        if isinstance(rt, types.NoneType):
            out.append(f"{c};")
            self.consts[tname] = None
        else:
            self.declare(tname)
            out.append(f"{self.cname(tname)} = {self.cast_expr(c, None, rt)};")

    def make_array(self, target, shared, args, out):
        """local.array / private.array with a static shape (one buffer per call
        site: numba_mlir/mlir/kernel_impl.py:366-437)."""
        types = self.types
        tname = target.name
        ttype = types.unliteral(self.vtype(tname))
        shape = self.static_value(args[0])
        if isinstance(shape, (int, np.integer)):
            shape = (int(shape),)
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape)) if shape else 1
        self.declare(tname)
        rep = self.arrays[tname]
        buf = self.fresh("nmb_local" if shared else "nmb_private")
        if shared:
            self.local_arrays.append((len(self.shared_decls), buf, rep.ctype,
                                      max(n, 1) * np.dtype(str(ttype.dtype)).itemsize))
            self.shared_decls.append(f"__shared__ __align__(16) {rep.ctype} {buf}[{max(n, 1)}];")
        else:
            # zero-filled like the reference's simulator (kernel_sim_impl.py:166-168)
            self.decls.append(f"{rep.ctype} {buf}[{max(n, 1)}] = {{}};")
        stm = [f"{rep.ptr} = {buf};"]
        acc = 1
        strides = []
        for s in reversed(shape):
            strides.append(acc)
            acc *= s
        strides.reverse()
        for d, (s, st) in enumerate(zip(shape, strides)):
            stm.append(f"{rep.shape[d]} = {s}; {rep.strides[d]} = {st};")
        out.append(" ".join(stm))

    def static_value(self, var):
        from numba.core import ir_utils

        if var.name in self.consts:
            return self.consts[var.name]
        t = self.vtype(var.name)
        if hasattr(t, "literal_value"):
            return t.literal_value
        try:
            return ir_utils.find_const(self.tir.func_ir, var)
        except Exception:
            pass
        if isinstance(t, (self.types.Tuple, self.types.UniTuple)) and all(
                hasattr(e, "literal_value") for e in t.types):
            return tuple(e.literal_value for e in t.types)
        defn = ir_utils.guard(ir_utils.get_definition, self.tir.func_ir, var)
        if isinstance(defn, self.ir.Expr) and defn.op == "build_tuple":
            return tuple(self.static_value(i) for i in defn.items)
        if isinstance(defn, self.ir.Expr) and defn.op == "binop" and defn.fn in (
                operator.add, operator.sub, operator.mul, operator.floordiv):
            # arithmetic on constants, e.g. a shape written as 4 * GROUP_SIZE
            return defn.fn(self.static_value(defn.lhs), self.static_value(defn.rhs))
        raise UnsupportedError(f"{var.name} must be a compile-time constant")

    # arguments ------------------------------------------------------------------------
    def bind_arg(self, tname, index, out):
        types = self.types
        t = types.unliteral(self.vtype(tname))
        p = self.param_names[index]
        self.declare(tname)
        if _is_scalar(t):
            out.append(f"{self.cname(tname)} = {p};")
        elif isinstance(t, types.Array):
            rep = self.arrays[tname]
            self.alias[tname] = f"<param{index}>"
            stm = [f"{rep.ptr} = ({rep.ctype}*){p}_p;"]
            for d in range(rep.ndim):
                stm.append(f"{rep.shape[d]} = {p}_s{d};")
            if t.layout == "C":
                for d in range(rep.ndim - 1, -1, -1):
                    stm.append(f"{rep.strides[d]} = " + ("1;" if d == rep.ndim - 1 else
                                                         f"{rep.strides[d + 1]} * {p}_s{d + 1};"))
            else:
                for d in range(rep.ndim):
                    stm.append(f"{rep.strides[d]} = {p}_t{d};")
            out.append(" ".join(stm))
        else:
            raise UnsupportedError(f"argument of type {t}")

    def parallel_update(self, store, blocks):
        """(sign, operand) when `store` writes `x[idx] (+|-)= operand` back to the
        element it was read from, else None."""
        import operator as op

        ir = self.ir
        if getattr(self, "_defs", None) is None:
            self._defs = _single_defs(blocks, ir)
        d = self._defs.get(store.value.name)
        if d is None or len(d) != 1 or not isinstance(d[0], ir.Expr) or d[0].op != "inplace_binop":
            return None
        e = d[0]
        if e.fn not in (op.iadd, op.isub):
            return None
        ld = _resolve(self._defs, ir, e.lhs.name)
        if not (isinstance(ld, ir.Expr) and ld.op in ("getitem", "static_getitem")):
            return None
        if ld.value.name != store.target.name:
            return None
        st_idx = store.index_var if isinstance(store, ir.StaticSetItem) else store.index
        ld_idx = ld.index_var if ld.op == "static_getitem" else ld.index
        if st_idx is None or ld_idx is None or st_idx.name != ld_idx.name:
            return None
        return (1 if e.fn is op.iadd else -1), e.rhs

    # packed inner loops ---------------------------------------------------------------
    # sm_100 adds, subtracts and multiplies two float32 values in one instruction
    # (nmb::add2 / sub2 / mul2).  A loop `for q in range(C)` with a small even
    # constant C whose iterations are independent of one another is emitted as
    # straight-line code, two iterations at a time, with the float32 +, -, * of
    # the two iterations packed; everything else is emitted once per iteration.
    # Iterations are known to be independent when the body is one block of
    # assignments and element stores, every array it stores to is a private
    # array indexed directly by the loop variable in one fixed position (so
    # iteration q touches only elements with that index equal to q, in loads
    # and stores alike), and no scalar computed in one iteration is read in
    # the next.  The rounding of every operation is what the loop's was.
    _PACK_FNS = {operator.add: "add2", operator.iadd: "add2", operator.sub: "sub2", operator.isub: "sub2",
                 operator.mul: "mul2", operator.imul: "mul2"}
    _PACK_MAX_TRIP = 16

    def _array_origin(self, defs, name):
        """('private' | 'local' | 'arg', defining variable) of an array variable, or None."""
        from . import kernel_impl as K

        ir = self.ir
        for _ in range(64):
            d = defs.get(name)
            if d is None or len(d) != 1:
                return None
            d = d[0]
            if isinstance(d, ir.Var):
                name = d.name
                continue
            if isinstance(d, ir.Arg):
                return ("arg", name)
            if isinstance(d, ir.Expr) and d.op == "call":
                fn = self.callee(d.func)
                if fn is K.private_array:
                    return ("private", name)
                if fn is K.local_array:
                    return ("local", name)
            return None
        return None

    def _pure_call(self, expr):
        types = self.types
        try:
            fn = self.callee(expr.func)
        except Exception:
            return False
        if fn in (int, float, bool, abs, min, max) or isinstance(fn, np.ufunc):
            return True
        if isinstance(self.vtype(expr.func.name), types.NumberClass):
            return True
        if isinstance(fn, type) and issubclass(fn, np.generic):
            return True
        return getattr(fn, "__module__", None) == "math"

    def packable_loops(self):
        """{header label: (body label, exit label, trip count, induction variable
        name)} of the loops that are emitted two iterations at a time."""
        from numba.core.analysis import compute_cfg_from_blocks

        ir, types = self.ir, self.types
        blocks = self.tir.func_ir.blocks
        defs = _single_defs(blocks, ir)
        found = {}
        try:
            loops = compute_cfg_from_blocks(blocks).loops()
        except Exception:
            return found
        for loop in loops.values():
            if len(loop.body) != 2 or len(loop.entries) != 1 or len(loop.exits) != 1:
                continue
            head = loop.header
            (body_label,) = [b for b in loop.body if b != head]
            if head in self.block_prologue or head in self.block_epilogue or \
                    body_label in self.block_prologue or body_label in self.block_epilogue:
                continue
            hb, bb = blocks[head].body, blocks[body_label].body
            # header: iternext / pair_first / pair_second / phi copy / branch
            if len(hb) != 5 or not isinstance(hb[4], ir.Branch) or hb[4].truebr != body_label:
                continue
            ops = [getattr(i.value, "op", None) if isinstance(i, ir.Assign) else None for i in hb[:3]]
            if ops != ["iternext", "pair_first", "pair_second"] or not isinstance(hb[3], ir.Assign) \
                    or not isinstance(hb[3].value, ir.Var) or hb[3].value.name != hb[1].target.name \
                    or hb[4].cond.name != hb[2].target.name:
                continue
            phi = hb[3].target.name
            if not isinstance(bb[-1], ir.Jump) or bb[-1].target != head:
                continue
            # trip count: range(C) or range(0, C) with a constant C
            it = _resolve(defs, ir, hb[0].value.value.name)
            if not (isinstance(it, ir.Expr) and it.op == "getiter"):
                continue
            rng = _resolve(defs, ir, it.value.name)
            if not (isinstance(rng, ir.Expr) and rng.op == "call" and self.callee(rng.func) is range
                    and 1 <= len(rng.args) <= 2 and not rng.kws):
                continue
            if it.value.name in self.par_ranges:
                continue
            try:
                bounds = [self.static_value(a) for a in rng.args]
            except UnsupportedError:
                continue
            if not all(isinstance(b, (int, np.integer)) for b in bounds) or (len(bounds) == 2 and bounds[0] != 0):
                continue
            trip = int(bounds[-1])
            if trip < 2 or trip % 2 or trip > self._PACK_MAX_TRIP:
                continue
            if self._independent_iterations(bb[:-1], defs, phi, blocks, body_label, head):
                found[head] = (body_label, hb[4].falsebr, trip, phi)
        return found

    def _independent_iterations(self, stmts, defs, phi, blocks, body_label, head):
        ir, types = self.ir, self.types
        f32 = types.float32
        defined = set()
        loop_var = {phi}            # names that hold the loop variable itself
        index_pos = {}              # tuple variable -> positions holding the loop variable
        stored, loaded = [], []     # (array variable, index variable)
        packed = 0
        body_targets = {i.target.name for i in stmts if isinstance(i, ir.Assign)}
        for inst in stmts:
            if isinstance(inst, ir.Del):
                continue
            if isinstance(inst, (ir.SetItem, ir.StaticSetItem)):
                idx = inst.index_var if isinstance(inst, ir.StaticSetItem) else inst.index
                if idx is None:
                    return False
                used = [inst.target, idx, inst.value]
                stored.append((inst.target.name, idx.name))
            elif isinstance(inst, ir.Assign):
                v = inst.value
                used = []
                if isinstance(v, ir.Var):
                    used = [v]
                    if v.name in loop_var:
                        loop_var.add(inst.target.name)
                elif isinstance(v, (ir.Const, ir.Global, ir.FreeVar)):
                    pass
                elif isinstance(v, ir.Expr):
                    used = v.list_vars()
                    if v.op in ("binop", "inplace_binop"):
                        sig = self.calltypes[v]
                        if v.fn in self._PACK_FNS and all(types.unliteral(t) == f32 for t in sig.args) \
                                and types.unliteral(sig.return_type) == f32:
                            packed += 1
                    elif v.op in ("getitem", "static_getitem"):
                        idx = v.index_var if v.op == "static_getitem" else v.index
                        vt = types.unliteral(self.vtype(v.value.name))
                        if isinstance(vt, types.Array):
                            if idx is None or not _is_scalar(types.unliteral(self.vtype(inst.target.name))):
                                return False
                            loaded.append((v.value.name, idx.name))
                    elif v.op == "build_tuple":
                        index_pos[inst.target.name] = [k for k, item in enumerate(v.items) if item.name in loop_var]
                    elif v.op == "call":
                        if not self._pure_call(v):
                            return False
                    elif v.op not in ("unary", "cast", "getattr"):
                        return False
                else:
                    return False
                # a value of this iteration only: defined before it is read, once
                if inst.target.name in defined:
                    return False
            else:
                return False
            if any(u.name in body_targets and u.name not in defined for u in used):
                return False  # read before it is assigned: carried from the previous iteration
            if isinstance(inst, ir.Assign):
                defined.add(inst.target.name)
        if not packed:
            return False

        def position(index_name):
            """Position of the loop variable in an index, or None."""
            if index_name in loop_var:
                return 0
            pos = index_pos.get(index_name)
            return pos[0] if pos and len(pos) == 1 else None

        roots = {}
        for arr, idx in stored:
            origin = self._array_origin(defs, arr)
            if origin is None or origin[0] != "private":
                return False
            pos = position(idx)
            if pos is None or roots.setdefault(origin[1], pos) != pos:
                return False
        for arr, idx in loaded:
            origin = self._array_origin(defs, arr)
            if origin is None:
                return False
            if origin[1] in roots and position(idx) != roots[origin[1]]:
                return False
        # values leaving the loop must be scalars (they are copied out of the last iteration)
        for label, blk in blocks.items():
            if label in (body_label, head):
                continue
            for inst in blk.body:
                for u in inst.list_vars():
                    if u.name in defined and not _is_scalar(types.unliteral(self.vtype(u.name))):
                        if not any(isinstance(i, ir.Assign) and i.target.name == u.name for i in blk.body):
                            return False
        return True

    def _renamed(self, inst, ren):
        """Copy of a statement with the variables of `ren` renamed (types and call
        signatures registered for the copies)."""
        ir = self.ir

        def v(var):
            n = ren.get(var.name)
            return ir.Var(var.scope, n, var.loc) if n is not None else var

        def value(val):
            if isinstance(val, ir.Var):
                return v(val)
            if isinstance(val, ir.Expr):
                kws = {}
                for k, x in val._kws.items():
                    if isinstance(x, ir.Var):
                        kws[k] = v(x)
                    elif isinstance(x, (list, tuple)) and x and all(isinstance(e, ir.Var) for e in x):
                        kws[k] = type(x)(v(e) for e in x)
                    else:
                        kws[k] = x
                new = ir.Expr(val.op, val.loc, **kws)
                if val in self.calltypes:
                    self.calltypes[new] = self.calltypes[val]
                return new
            return val

        if isinstance(inst, ir.Assign):
            return ir.Assign(value(inst.value), v(inst.target), inst.loc)
        if isinstance(inst, ir.StaticSetItem):
            return ir.StaticSetItem(v(inst.target), inst.index,
                                    v(inst.index_var) if inst.index_var is not None else None,
                                    v(inst.value), inst.loc)
        return ir.SetItem(v(inst.target), v(inst.index), v(inst.value), inst.loc)

    def emit_packed_loop(self, head, info, out):
        ir, types = self.ir, self.types
        body_label, exit_label, trip, phi = info
        blocks = self.tir.func_ir.blocks
        stmts = [i for i in blocks[body_label].body[:-1] if not isinstance(i, ir.Del)]
        local = [i.target.name for i in stmts if isinstance(i, ir.Assign)]
        copies = []
        for c in range(trip):
            ren = {}
            for name in local + [phi]:
                new = f"{name}.u{head}.{c}"
                ren[name] = new
                self.typemap[new] = self.typemap[name]
                if name in self.narrow:
                    self.narrow.add(new)
            self.consts[ren[phi]] = c
            copies.append((ren, [self._renamed(i, ren) for i in stmts]))
        f32 = types.float32
        # A packed multiply must not feed an addition: the assembler merges
        # mul.f32x2 with a dependent add/sub.f32x2 into a fused multiply-add even
        # when both carry .rn.  A product is packed only when every reader is a
        # multiply of this loop body; otherwise it stays a scalar multiply, whose
        # .rn is honoured.
        is_mul = lambda e: isinstance(e, ir.Expr) and e.op in ("binop", "inplace_binop") and \
            self._PACK_FNS.get(e.fn) == "mul2"  # noqa: E731
        keep_scalar = set()
        for inst in ([] if self.fastmath else stmts):
            reader_is_mul = isinstance(inst, ir.Assign) and is_mul(inst.value)
            if not reader_is_mul:
                keep_scalar.update(u.name for u in inst.list_vars())
        for label, blk in blocks.items():
            if label != body_label and not self.fastmath:
                for inst in blk.body:
                    keep_scalar.update(u.name for u in inst.list_vars())
        for c0 in range(0, trip, 2):
            (ren0, s0), (ren1, s1) = copies[c0], copies[c0 + 1]
            for k, (a, b) in enumerate(zip(s0, s1)):
                v = a.value if isinstance(a, ir.Assign) else None
                if isinstance(v, ir.Expr) and v.op in ("binop", "inplace_binop") and v.fn in self._PACK_FNS \
                        and not (is_mul(v) and stmts[k].target.name in keep_scalar):
                    sig = self.calltypes[v]
                    if all(types.unliteral(t) == f32 for t in sig.args) and types.unliteral(sig.return_type) == f32:
                        self.declare(a.target.name)
                        self.declare(b.target.name)
                        w = b.value
                        out.append(f"nmb::{self._PACK_FNS[v.fn]}({self.scalar(v.lhs, f32)}, {self.scalar(w.lhs, f32)}, "
                                   f"{self.scalar(v.rhs, f32)}, {self.scalar(w.rhs, f32)}, "
                                   f"{self.cname(a.target.name)}, {self.cname(b.target.name)});")
                        continue
                for inst, ren in ((a, ren0), (b, ren1)):
                    self.statement(inst, out, blocks)
                    # the loop variable of this copy is a constant: later index
                    # expressions use the literal
                    if isinstance(inst, ir.Assign) and isinstance(inst.value, ir.Var) \
                            and inst.value.name in self.consts \
                            and _is_scalar(types.unliteral(self.vtype(inst.target.name))) \
                            and inst.value.name == ren[phi]:
                        self.consts[inst.target.name] = self.consts[inst.value.name]
        # values of the last iteration under the loop's own names, for code after the loop
        last = copies[-1][0]
        for name in local:
            if _is_scalar(types.unliteral(self.vtype(name))):
                self.declare(name)
                src = _NameRef(last[name])
                out.append(f"{self.cname(name)} = {self.scalar(src, self.vtype(name))};")
        out.append(f"goto L{exit_label};")

    # statements -------------------------------------------------------------------------
    def statement(self, inst, out, blocks):
        """C text of one IR statement, appended to `out`."""
        ir, types = self.ir, self.types
        if isinstance(inst, ir.Assign):
            if isinstance(inst.value, ir.Const) and inst.value.value is ir.UNDEFINED:
                return
            self.assign(inst.target, inst.value, out)
        elif isinstance(inst, (ir.SetItem, ir.StaticSetItem)):
            arr = inst.target
            self.declare(arr.name)
            self.written_params.add(self.root_of(arr.name))
            rep = self.arrays[arr.name]
            if isinstance(inst, ir.StaticSetItem) and inst.index_var is None:
                idx = inst.index if isinstance(inst.index, tuple) else (inst.index,)
                idx_exprs = [f"{int(i)}ll" for i in idx]
            else:
                idx_exprs = self.index_list(inst.index_var if isinstance(inst, ir.StaticSetItem)
                                            else inst.index)
            ref = self.element_ref(arr, idx_exprs)
            upd = self.parallel_update(inst, blocks) if self.mode == "parfor" else None
            if upd is not None:
                # `x[idx] += v` inside a parallel loop is an atomic update, as the
                # reference makes it (mlir/tests/test_numpy.py:1039-1057)
                sign, val = upd
                v = self.scalar(val, rep.dtype)
                out.append(f"nmb::atomic_add(&{ref}, ({rep.ctype})({'-' if sign < 0 else ''}({v})));")
            else:
                out.append(f"{ref} = {self.scalar(inst.value, rep.dtype)};")
        elif isinstance(inst, ir.Del):
            return
        elif isinstance(inst, ir.Jump):
            out.append(f"goto L{inst.target};")
        elif isinstance(inst, ir.Branch):
            out.append(f"if ({self.scalar(inst.cond, types.boolean)}) goto L{inst.truebr}; "
                       f"else goto L{inst.falsebr};")
        elif isinstance(inst, ir.Return):
            if self.mode == "parfor" and self.return_store is not None:
                out.append(f"{self.return_store} = {self.scalar(inst.value, self.tir.return_type)}; return;")
            elif self.mode in ("kernel", "parfor"):
                out.append("return;")
            else:
                out.append(f"return {self.scalar(inst.value, self.tir.return_type)};")
        elif isinstance(inst, (ir.Raise, ir.StaticRaise)):
            out.append("return;" if self.mode in ("kernel", "parfor") else "return 0;")
        else:
            raise UnsupportedError(f"statement {type(inst).__name__} in device code")

    def translate(self, param_names):
        ir, types = self.ir, self.types
        self.param_names = param_names
        blocks = self.tir.func_ir.blocks
        order = sorted(blocks)
        body = []
        packed = self.packable_loops() if self.mode in ("kernel", "parfor") else {}
        for label in order:
            out = [f"L{label}: ;"] + list(self.block_prologue.get(label, ()))
            if label in packed:
                self.emit_packed_loop(label, packed[label], out)
                body.append("\n    ".join(out))
                continue
            for inst in blocks[label].body:
                if isinstance(inst, (ir.Jump, ir.Branch, ir.Return)) and label in self.block_epilogue:
                    out.extend(self.block_epilogue[label])
                self.statement(inst, out, blocks)
            body.append("\n    ".join(out))
        return body


# -------------------------------------------------------------- drivers -----
def _argtype_of(a):
    from numba import typeof
    from numba.core import types

    from .device_array import DeviceArray

    if isinstance(a, DeviceArray):
        from numba.np.numpy_support import from_dtype

        layout = "C" if a.is_c_contiguous else "A"
        return types.Array(from_dtype(a.dtype), a.ndim, layout)
    if isinstance(a, bool):
        return types.boolean
    if isinstance(a, int):
        return types.int64
    if isinstance(a, float):
        return types.float64
    return typeof(a)


_device_func_counter = [0]


def compile_device_function(py_func, dtypes):
    """Scalar Python function -> lazy.DeviceFunc (a CUDA __device__ function)."""
    from numba.np.numpy_support import as_dtype, from_dtype

    argtypes = [from_dtype(np.dtype(d)) for d in dtypes]
    tir = typed_ir(py_func, argtypes)
    _device_func_counter[0] += 1
    name = f"nmb_dev_{re.sub(r'[^0-9a-zA-Z_]', '_', py_func.__name__)}_{_device_func_counter[0]}"
    tr = Translator(tir, "device", name)
    params = [f"a{i}" for i in range(len(argtypes))]
    body = tr.translate(params)
    if tr.shared_decls:
        raise UnsupportedError("local memory is not available in scalar device functions")
    rt = c_scalar_type(tir.return_type)
    sig = ", ".join(f"{c_scalar_type(t)} a{i}" for i, t in enumerate(argtypes))
    src = (f"__device__ __forceinline__ {rt} {name}({sig}) {{\n    " + "\n    ".join(tr.decls)
           + "\n    " + "\n    ".join(body) + "\n}\n")
    return lazy.DeviceFunc(name, src, dtypes, as_dtype(tir.return_type), pair=_pair_routine(tr, tir))


# float32 functions nmb_device.cuh also has for two values at once (f32x2 instructions)
_PAIR_ROUTINES = {math.erf: "erf_pair", math.log: "log_pair"}


def _pair_routine(tr, tir):
    """Name of the two-values-at-once routine when the scalar function is
    nothing but `return f(x)` in float32 for an f of _PAIR_ROUTINES."""
    ir, types = tr.ir, tr.types
    if len(tir.args) != 1 or types.unliteral(tir.args[0]) != types.float32 or \
            types.unliteral(tir.return_type) != types.float32:
        return None
    blocks = tir.func_ir.blocks
    if len(blocks) != 1:
        return None
    defs = _single_defs(blocks, ir)
    calls = [i.value for blk in blocks.values() for i in blk.body
             if isinstance(i, ir.Assign) and isinstance(i.value, ir.Expr) and i.value.op == "call"]
    if len(calls) != 1 or len(calls[0].args) != 1 or calls[0].kws:
        return None
    routine = _PAIR_ROUTINES.get(tr.callee(calls[0].func))
    if routine is None or not isinstance(_resolve(defs, ir, calls[0].args[0].name), ir.Arg):
        return None
    (ret,) = [i for blk in blocks.values() for i in blk.body if isinstance(i, ir.Return)]
    value = _resolve(defs, ir, ret.value.name)
    while isinstance(value, ir.Expr) and value.op == "cast":
        value = _resolve(defs, ir, value.value.name)
    return routine if value is calls[0] else None


class CompiledKernel:
    def __init__(self, source, name, param_layout, uses_barrier):
        self.source = source
        self.name = name
        self.param_layout = param_layout  # per Python argument: ("array", ndim, layout) | ("scalar", dtype)
        self.uses_barrier = uses_barrier
        self._handles = {}      # queue -> kernel handle (the queue owns and frees it)
        self._block_sizes = {}  # (queue, global size) -> suggested local size
        self._kinds = {}
        # bytes of work-group-local memory requested at launch (local arrays too
        # large for static shared memory); the kernel then takes one more
        # parameter, the offset the runtime placed them at
        self.local_bytes = 0

    def kinds(self, trailing_int64=0):
        """Launch parameter kinds: the arguments, then `trailing_int64` sizes,
        then the local-memory request if there is one."""
        k = self._kinds.get(trailing_int64)
        if k is None:
            from .kernel_impl import param_kinds

            k = param_kinds(self.param_layout, trailing_int64)
            if self.local_bytes:
                k = k + (("local", self.local_bytes),)
            self._kinds[trailing_int64] = k
        return k

    def layout_code(self):
        """The argument layout as the native launch path reads it: per array
        'A', its rank, 'C' (shape follows the pointer) or 'S' (shape and
        element strides follow); per scalar its type letter."""
        code = getattr(self, "_layout_code", None)
        if code is None:
            from .runtime import param_code

            parts = []
            for lay in self.param_layout:
                if lay[0] == "array":
                    parts.append(b"A" + bytes([lay[1]]) + (b"C" if lay[2] == "C" else b"S"))
                else:
                    parts.append(param_code(lay[1]))
            code = self._layout_code = b"".join(parts)
        return code

    def handle_on(self, queue):
        """Kernel handle on `queue`, loading the module on first use."""
        h = self._handles.get(queue)
        if h is None:
            h = queue.get_kernel(queue.load_module(self.source.encode()), self.name)
            self._handles[queue] = h
        return h

    def block_size_on(self, queue, kernel, global_size):
        key = (queue, global_size)
        b = self._block_sizes.get(key)
        if b is None:
            b = self._block_sizes[key] = queue.suggest_block_size(kernel, global_size)
        return b


# Static shared memory of one kernel (CUDA's limit).  Local arrays stay static
# while everything fits: their addresses are then immediates, which measured
# 15 % faster on the k-means program than the same arrays at a run-time offset.
_STATIC_SHARED_LIMIT = 48 * 1024


def compile_kernel(py_func, args, ndim, fastmath=False, index32=False, max_threads=None):
    """@kernel body + concrete arguments -> CompiledKernel (tagged CUDA source).

    The grid mapping is the reference's: get_global_id(d) is
    blockIdx.d*blockDim.d + threadIdx.d (LowerToGpu.cpp:1113-1137), the grid is
    ceil(global/local) groups and work-items past the global size are masked
    off (mlir/lib/Conversion/GpuToGpuRuntime.cpp:1460-1546)."""
    argtypes = [_argtype_of(a) for a in args]
    tir = typed_ir(py_func, argtypes)
    from numba.core import types

    tr = Translator(tir, "kernel", "nmb_kernel", index32=index32, fastmath=fastmath)
    pnames = [f"p{i}" for i in range(len(argtypes))]
    body = tr.translate(pnames)
    written = {int(r[6:-1]) for r in tr.written_params if r.startswith("<param")}
    kparams, layout = [], []
    for i, t in enumerate(argtypes):
        t = types.unliteral(t)
        if isinstance(t, types.Array):
            ct = c_scalar_type(t.dtype)
            qual = f"{ct}* __restrict__" if i in written else f"const {ct}* __restrict__"
            kparams.append(f"{qual} p{i}_p")
            kparams += [f"int64_t p{i}_s{d}" for d in range(t.ndim)]
            if t.layout != "C":
                kparams += [f"int64_t p{i}_t{d}" for d in range(t.ndim)]
            layout.append(("array", t.ndim, t.layout))
        else:
            kparams.append(f"{c_scalar_type(t)} p{i}")
            layout.append(("scalar", np.dtype(str(t))))
    kparams += ["int64_t nmb_g0", "int64_t nmb_g1", "int64_t nmb_g2"]
    # Local arrays are static shared memory while they fit beside the kernel's
    # other static buffers (48 KB per group in all); otherwise all are carved out
    # of the dynamic shared memory the launch asks for through a local-memory
    # parameter ({NULL, size, ptr}, GpuRuntimeToLlvm.cpp:514-528), up to the
    # device's limit per group.
    local_bytes = 0
    other_static = (9216 if tr.uses_group_reduce else 0) + 1024  # group-reduction buffers, small scratch
    if sum(nb for _i, _b, _c, nb in tr.local_arrays) + other_static > _STATIC_SHARED_LIMIT:
        for idx, buf, ct, nb in tr.local_arrays:
            tr.shared_decls[idx] = (f"{ct}* const {buf} = reinterpret_cast<{ct}*>"
                                    f"(nmb_dyn_local + nmb_local_off + {local_bytes}ull);")
            local_bytes += (nb + 15) // 16 * 16
        tr.shared_decls.insert(0, "extern __shared__ __align__(16) unsigned char nmb_dyn_local[];")
        kparams.append("unsigned long long nmb_local_off")
    opts = "\n#define NMB_FASTMATH 1" if fastmath else " --fmad=false"
    group_prologue = ""
    if tr.uses_group_reduce:
        # group reductions need to know which work-items of the group exist
        group_prologue = """__shared__ unsigned char nmb_active[1024];
    __shared__ __align__(16) unsigned char nmb_gr_vals[8192];
    {
        const int nmb_tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
        nmb_active[nmb_tid] = nmb_item_active;
    }
    const bool nmb_group_full = (blockDim.x * blockDim.y * blockDim.z) % 32 == 0 &&
        (int64_t)(blockIdx.x + 1) * blockDim.x <= nmb_g0 && (int64_t)(blockIdx.y + 1) * blockDim.y <= nmb_g1 &&
        (int64_t)(blockIdx.z + 1) * blockDim.z <= nmb_g2;
    __syncthreads();"""
    src = f"""//NMB200:CUDA-SOURCE
//NMB200:OPTIONS{opts}
#include "nmb_device.cuh"
extern "C" __global__ void nmb_kernel({', '.join(kparams)}) {{
    const int64_t nmb_gs[3] = {{nmb_g0, nmb_g1, nmb_g2}};
    // work-items past the global size are masked off
    const bool nmb_item_active = nmb::k_get_global_id(0, nmb_gs) < nmb_g0 &&
        nmb::k_get_global_id(1, nmb_gs) < nmb_g1 && nmb::k_get_global_id(2, nmb_gs) < nmb_g2;
    {group_prologue}
    if (!nmb_item_active) return;
    {' '.join(tr.shared_decls)}
    {chr(10).join('    ' + d for d in tr.decls)}
    {(chr(10) + '    ').join(body)}
}}
"""
    ck = CompiledKernel(src, "nmb_kernel", layout, tr.uses_barrier)
    ck.local_bytes = local_bytes
    return ck


# ------------------------------------------------------- prange loop nests ---
class CompiledParfor(CompiledKernel):
    """A function whose outermost `prange` loop is the grid.

    `extents(args)` gives the trip counts of the parallel loops the host could
    work out from the arguments (None where it could not); the loops are
    grid-strided, so any launch shape is correct and the extents only size it."""

    def __init__(self, source, name, param_layout, inner_parallel, extent_fns, epilogue=None,
                 return_dtype=None):
        CompiledKernel.__init__(self, source, name, param_layout, False)
        self.inner_parallel = inner_parallel
        self.extent_fns = extent_fns
        # epilogue: None, or the bytes of per-block partials the kernel needs (it then
        # takes three more pointers: partials, ticket counter, return cell)
        self.epilogue = epilogue
        self.return_dtype = return_dtype

    def extents(self, args):
        out = []
        for fn in self.extent_fns:
            try:
                out.append(None if fn is None else max(0, int(fn(args))))
            except Exception:
                out.append(None)
        return out


def uses_prange(py_func):
    code = getattr(py_func, "__code__", None)
    return code is not None and "prange" in code.co_names


def _single_defs(blocks, ir):
    defs = {}
    for blk in blocks.values():
        for inst in blk.body:
            if isinstance(inst, ir.Assign):
                defs.setdefault(inst.target.name, []).append(inst.value)
    return defs


def _resolve(defs, ir, name):
    """Follows single-assignment copies to the defining expression."""
    seen = 0
    while seen < 64:
        d = defs.get(name)
        if d is None or len(d) != 1:
            return None
        if isinstance(d[0], ir.Var):
            name = d[0].name
            seen += 1
            continue
        return d[0]
    return None


def _extent_fn(tr, defs, call_expr):
    """Host-side trip count of `prange(...)` as a function of the call's
    Python arguments, for the common forms (argument scalars, shapes, len,
    constants and + - * // of those); None when it cannot be told."""
    import operator as op

    ir, types = tr.ir, tr.types

    def sym(var, depth=0):
        if depth > 16:
            return None
        name = var.name
        if name in tr.consts and isinstance(tr.consts[name], (int, np.integer)):
            v = int(tr.consts[name])
            return lambda args: v
        e = _resolve(defs, ir, name)
        if e is None:
            return None
        if isinstance(e, ir.Arg):
            k = e.index
            if _is_scalar(types.unliteral(tr.vtype(name))):
                return lambda args: int(args[k])
            return None
        if isinstance(e, (ir.Const, ir.Global, ir.FreeVar)):
            if isinstance(e.value, (int, np.integer)) and not isinstance(e.value, bool):
                v = int(e.value)
                return lambda args: v
            return None
        if not isinstance(e, ir.Expr):
            return None
        if e.op in ("static_getitem", "getitem"):
            base = _resolve(defs, ir, e.value.name)
            if (isinstance(base, ir.Expr) and base.op == "getattr" and base.attr == "shape"):
                arr = _resolve(defs, ir, base.value.name)
                idx = e.index if e.op == "static_getitem" else None
                if isinstance(arr, ir.Arg) and isinstance(idx, int):
                    k = arr.index
                    return lambda args: args[k].shape[idx]
            return None
        if e.op == "call":
            try:
                fn = tr.callee(e.func)
            except Exception:
                return None
            if fn is len and len(e.args) == 1:
                arr = _resolve(defs, ir, e.args[0].name)
                if isinstance(arr, ir.Arg):
                    k = arr.index
                    return lambda args: args[k].shape[0]
            return None
        if e.op == "getattr" and e.attr == "size":
            arr = _resolve(defs, ir, e.value.name)
            if isinstance(arr, ir.Arg):
                k = arr.index
                return lambda args: args[k].size
            return None
        if e.op in ("binop", "inplace_binop") and e.fn in (op.add, op.sub, op.mul, op.floordiv,
                                                           op.iadd, op.isub, op.imul, op.ifloordiv):
            a, b = sym(e.lhs, depth + 1), sym(e.rhs, depth + 1)
            if a is None or b is None:
                return None
            f = {op.iadd: op.add, op.isub: op.sub, op.imul: op.mul, op.ifloordiv: op.floordiv}.get(e.fn, e.fn)
            return lambda args: f(a(args), b(args))
        return None

    parts = [sym(a) for a in call_expr.args]
    if any(p is None for p in parts):
        return None
    if len(parts) == 1:
        return lambda args: parts[0](args)
    if len(parts) == 2:
        return lambda args: parts[1](args) - parts[0](args)

    def trip(args):
        lo, hi, st = (f(args) for f in parts)
        return len(range(lo, hi, st))

    return trip


def compile_parfor(py_func, args, fastmath=False, index32=False):
    """njit function with `prange` loops -> one CUDA kernel.

    The reference turns every parallel loop nest of an njit function into a
    `gpu.launch` (mlir/tests/test_gpu.py:1523-1613: ConvertParallelLoopToGpu).
    Here the function becomes one kernel: the outermost `prange` is
    grid-strided over the y (or only) grid dimension; a `prange` directly
    inside it is grid-strided over x when its iterations are independent and
    nothing else in the outer body has side effects; deeper loops run
    sequentially in the thread.  Statements before the loop run in every
    thread, so they may only compute scalars."""
    from numba.core import types
    from numba.core.analysis import compute_cfg_from_blocks, compute_live_map, compute_use_defs

    from . import kernel_impl as K

    argtypes = [_argtype_of(a) for a in args]
    tir = typed_ir(py_func, argtypes)
    returns_scalar = _is_scalar(types.unliteral(tir.return_type))
    if not returns_scalar and not isinstance(tir.return_type, types.NoneType):
        raise UnsupportedError(
            f"{py_func.__name__}: a function with prange loops returns None or a scalar (array "
            "results go to array arguments)")
    tr = Translator(tir, "parfor", "nmb_parfor", index32=index32, fastmath=fastmath)
    ir = tr.ir
    blocks = tir.func_ir.blocks
    cfg = compute_cfg_from_blocks(blocks)
    loops = cfg.loops()
    defs = _single_defs(blocks, ir)
    usedefs = compute_use_defs(blocks)
    live = compute_live_map(cfg, blocks, usedefs.usemap, usedefs.defmap)

    def prange_call_of(loop):
        """(name of the range variable, call expression) when `loop` iterates a prange."""
        for inst in blocks[loop.header].body:
            if (isinstance(inst, ir.Assign) and isinstance(inst.value, ir.Expr)
                    and inst.value.op == "iternext"):
                it = _resolve(defs, ir, inst.value.value.name)
                if not (isinstance(it, ir.Expr) and it.op == "getiter"):
                    return None
                name = it.value.name
                while True:  # the variable the call was assigned to
                    d = defs.get(name)
                    if d is None or len(d) != 1:
                        return None
                    if isinstance(d[0], ir.Var):
                        name = d[0].name
                        continue
                    break
                call = d[0]
                if not (isinstance(call, ir.Expr) and call.op == "call"):
                    return None
                fn = tr.callee(call.func)
                if getattr(fn, "__name__", "") == "prange":
                    return name, call
                return None
        return None

    def side_effects(labels):
        for lb in labels:
            for inst in blocks[lb].body:
                if isinstance(inst, (ir.SetItem, ir.StaticSetItem)):
                    return True
                if (isinstance(inst, ir.Assign) and isinstance(inst.value, ir.Expr)
                        and inst.value.op == "call"):
                    try:
                        fn = tr.callee(inst.value.func)
                    except Exception:
                        return True
                    if fn in (K.atomic_add, K.atomic_sub, K.barrier, K.mem_fence) or fn in K.GROUP_REDUCE:
                        return True
        return False

    def body_defs(loop):
        out = set()
        for lb in loop.body:
            out |= usedefs.defmap[lb]
        return out

    def independent(loop):
        """No scalar is carried from one iteration to the next or out of the loop."""
        d = body_defs(loop)
        carried = {v for v in live[loop.header] & d}
        escaping = set()
        for ex in loop.exits:
            escaping |= live[ex] & d
        return carried, escaping

    top = [lp for lp in loops.values()
           if not any(lp.header in o.body and o is not lp for o in loops.values())]
    par_top = [(lp, prange_call_of(lp)) for lp in top]
    par_top = [(lp, pc) for lp, pc in par_top if pc is not None]
    if len(par_top) != 1:
        raise UnsupportedError(
            f"{py_func.__name__}: exactly one outermost prange loop per function is supported "
            f"(found {len(par_top)})")
    outer, (outer_name, outer_call) = par_top[0]
    carried, escaping = independent(outer)
    reductions = _find_reductions(tr, blocks, defs, outer, carried, escaping)
    if reductions is None:
        raise UnsupportedError(
            f"{py_func.__name__}: scalar(s) {sorted(carried | escaping)} are carried across or out of "
            "the prange loop in a form that is not a reduction (supported: s += x, s -= x, s *= x, "
            "s = min(s, x), s = max(s, x), with s not read otherwise inside the loop)")
    before = set()  # blocks that can run before the loop: every thread executes them
    work = list(outer.entries)
    while work:
        lb = work.pop()
        if lb not in before:
            before.add(lb)
            work.extend(p_ for p_, _ in cfg.predecessors(lb))
    if side_effects(before):
        raise UnsupportedError(
            f"{py_func.__name__}: array stores before the prange loop are not supported (every "
            "thread runs that code)")
    after = set(blocks) - set(outer.body) - before
    # Code after the loop must run once, after every thread has finished: it is
    # left to the last thread block to arrive (a ticket), which also combines
    # the reduction partials.
    needs_epilogue = bool(reductions) or returns_scalar or side_effects(after)

    inner = None
    level2 = [lp for lp in loops.values() if lp is not outer and lp.header in outer.body
              and not any(lp.header in o.body and o is not lp and o is not outer for o in loops.values())]
    cands = [(lp, prange_call_of(lp)) for lp in level2]
    cands = [(lp, pc) for lp, pc in cands if pc is not None]
    if len(cands) == 1 and len(level2) == 1:
        lp, (nm, call) = cands[0]
        c2, e2 = independent(lp)
        if not c2 and not e2 and not side_effects(set(outer.body) - set(lp.body)):
            inner = (lp, nm, call)

    if needs_epilogue:
        inner = None  # the epilogue assumes a one-dimensional grid
    if inner is not None:
        tr.par_ranges[outer_name] = ("nmb_oid", "nmb_on")
        tr.par_ranges[inner[1]] = ("nmb_iid", "nmb_in")
        ids = ("const int64_t nmb_oid = (int64_t)blockIdx.y * blockDim.y + threadIdx.y, "
               "nmb_on = (int64_t)gridDim.y * blockDim.y, "
               "nmb_iid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, "
               "nmb_in = (int64_t)gridDim.x * blockDim.x;")
    else:
        tr.par_ranges[outer_name] = ("nmb_oid", "nmb_on")
        ids = ("const int64_t nmb_oid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, "
               "nmb_on = (int64_t)gridDim.x * blockDim.x;")

    epilogue_bytes = None
    if needs_epilogue:
        epilogue_bytes = _install_epilogue(tr, outer, reductions)
        if returns_scalar:
            tr.return_store = f"*({c_scalar_type(tir.return_type)}*)nmb_ret"
    pnames = [f"p{i}" for i in range(len(argtypes))]
    body = tr.translate(pnames)
    if (tr.shared_decls and not needs_epilogue) or tr.uses_barrier:
        raise UnsupportedError("work-group local memory and barriers belong to @kernel functions")
    written = {int(r[6:-1]) for r in tr.written_params if r.startswith("<param")}
    kparams, layout = [], []
    for i, t in enumerate(argtypes):
        t = types.unliteral(t)
        if isinstance(t, types.Array):
            ct = c_scalar_type(t.dtype)
            # no __restrict__: the same buffer may be passed as input and output
            kparams.append(f"{ct}* p{i}_p" if i in written else f"const {ct}* p{i}_p")
            kparams += [f"int64_t p{i}_s{d}" for d in range(t.ndim)]
            if t.layout != "C":
                kparams += [f"int64_t p{i}_t{d}" for d in range(t.ndim)]
            layout.append(("array", t.ndim, t.layout))
        else:
            kparams.append(f"{c_scalar_type(t)} p{i}")
            layout.append(("scalar", np.dtype(str(t))))
    if needs_epilogue:
        kparams += ["unsigned char* nmb_partials", "unsigned int* nmb_ticket", "void* nmb_ret"]
    opts = "\n#define NMB_FASTMATH 1" if fastmath else " --fmad=false"
    src = f"""//NMB200:CUDA-SOURCE
//NMB200:OPTIONS{opts}
#include "nmb_device.cuh"
extern "C" __global__ void __launch_bounds__(256) nmb_parfor({', '.join(kparams)}) {{
    {ids}
    const int64_t nmb_gs[3] = {{1, 1, 1}};
    (void)nmb_gs;
    {' '.join(tr.shared_decls)}
    {chr(10).join('    ' + d for d in tr.decls)}
    {(chr(10) + '    ').join(body)}
}}
"""
    fns = [_extent_fn(tr, defs, outer_call)]
    if inner is not None:
        fns.append(_extent_fn(tr, defs, inner[2]))
    from numba.np.numpy_support import as_dtype

    return CompiledParfor(src, "nmb_parfor", layout, inner is not None, fns, epilogue=epilogue_bytes,
                          return_dtype=as_dtype(tir.return_type) if returns_scalar else None)


_REDUCTION_OPS = {operator.add: ("OpAdd", "add"), operator.iadd: ("OpAdd", "add"),
                  operator.sub: ("OpAdd", "add"), operator.isub: ("OpAdd", "add"),
                  operator.mul: ("OpMul", "mul"), operator.imul: ("OpMul", "mul")}


def _find_reductions(tr, blocks, defs, loop, carried, escaping):
    """Reduction variables of a parallel loop: [(variable, op struct, neutral name)], or
    None when a carried or escaping scalar is anything else.

    After SSA and phi stripping a reduction `s += x` reads
        s.2 = s              (before the loop)
        t = s.2 + x ; s.1 = t ; s.2 = s.1      (in the body)
    i.e. the carried variable is assigned once in the body, from a value
    computed by one + - * (or min / max call) that has the carried variable as
    an operand, and is not read anywhere else in the body."""
    ir, types = tr.ir, tr.types
    if escaping - carried:
        return None
    body_insts = [inst for lb in loop.body for inst in blocks[lb].body]
    found = []
    for v in sorted(carried):
        if not _is_scalar(types.unliteral(tr.vtype(v))):
            return None
        assigns = [inst for inst in body_insts if isinstance(inst, ir.Assign) and inst.target.name == v]
        if len(assigns) != 1 or not isinstance(assigns[0].value, ir.Var):
            return None
        # the update expression, through single-assignment copies made in the body
        name, upd, chain = assigns[0].value.name, None, []
        for _ in range(8):
            chain.append(name)
            d = [inst.value for inst in body_insts if isinstance(inst, ir.Assign) and inst.target.name == name]
            if len(d) != 1:
                return None
            if isinstance(d[0], ir.Var):
                name = d[0].name
                continue
            upd = d[0]
            break
        # the running value must not be observed on its way (that would be a scan)
        for c in chain:
            uses = sum(1 for inst in body_insts for u in inst.list_vars() if u.name == c)
            if uses != 2 or c in escaping:  # its definition and the copy onwards
                return None
        if not isinstance(upd, ir.Expr):
            return None
        if upd.op in ("binop", "inplace_binop") and upd.fn in _REDUCTION_OPS:
            operands = [upd.lhs.name, upd.rhs.name]
            if upd.fn in (operator.sub, operator.isub) and upd.lhs.name != v:
                return None
            opinfo = _REDUCTION_OPS[upd.fn]
        elif upd.op == "call" and len(upd.args) == 2 and not upd.kws:
            fn = tr.callee(upd.func)
            if fn is min:
                opinfo = ("OpMin", "min")
            elif fn is max:
                opinfo = ("OpMax", "max")
            else:
                return None
            operands = [a.name for a in upd.args]
        else:
            return None
        if operands.count(v) != 1:
            return None
        reads = sum(1 for inst in body_insts for u in inst.list_vars() if u.name == v) - 1  # its own assignment
        if reads != 1:
            return None
        found.append((v, opinfo[0], opinfo[1]))
    return found


def _install_epilogue(tr, loop, reductions):
    """Hooks the grid-wide epilogue of a prange kernel into the translation and
    returns the bytes of partials one thread block contributes.

    Before the loop every thread swaps each reduction variable for the neutral
    element and keeps the incoming value.  At the loop exit the block reduces
    its threads' partials, thread 0 publishes them and draws a ticket; every
    block but the last to arrive leaves.  The last block combines the
    published partials in block order (so the result does not depend on
    scheduling), applies the incoming value, resets the ticket and its thread
    0 alone runs what follows the loop."""
    types = tr.types
    pre, post = [], []
    slot = 0
    tr.decls.append("bool nmb_last_block;")
    tr.shared_decls.append("__shared__ bool nmb_is_last;")
    for k, (v, opname, neutral) in enumerate(reductions):
        t = types.unliteral(tr.vtype(v))
        ct = c_scalar_type(t)
        tr.declare(v)
        c = tr.cname(v)
        tr.decls.append(f"{ct} nmb_init{k};")
        tr.shared_decls.append(f"__shared__ {ct} nmb_rs{k}[32];")
        pre.append(f"nmb_init{k} = {c}; {c} = nmb::neutral_{neutral}<{ct}>();")
        post.append(f"{c} = nmb::block_reduce(({ct}){c}, nmb::{opname}(), nmb::neutral_{neutral}<{ct}>(), nmb_rs{k});")
        post.append(f"if (threadIdx.x == 0) (({ct}*)(nmb_partials + {slot} * (size_t)gridDim.x))[blockIdx.x] = {c};")
        slot += 8
    post.append("if (threadIdx.x == 0) { __threadfence(); "
                "nmb_is_last = atomicAdd(nmb_ticket, 1u) == gridDim.x - 1; }")
    post.append("__syncthreads(); nmb_last_block = nmb_is_last; if (!nmb_last_block) return; __threadfence();")
    slot = 0
    for k, (v, opname, neutral) in enumerate(reductions):
        t = types.unliteral(tr.vtype(v))
        ct = c_scalar_type(t)
        c = tr.cname(v)
        post.append(f"{c} = nmb::neutral_{neutral}<{ct}>(); "
                    f"for (unsigned nmb_b = threadIdx.x; nmb_b < gridDim.x; nmb_b += blockDim.x) "
                    f"{c} = nmb::{opname}()({c}, __ldcg((const {ct}*)(nmb_partials + {slot} * (size_t)gridDim.x) + nmb_b)); "
                    f"{c} = nmb::block_reduce(({ct}){c}, nmb::{opname}(), nmb::neutral_{neutral}<{ct}>(), nmb_rs{k}); "
                    f"{c} = nmb::{opname}()(nmb_init{k}, {c});")
        slot += 8
    post.append("if (threadIdx.x != 0) return; *nmb_ticket = 0u;")
    for lb in loop.entries:
        tr.block_epilogue.setdefault(lb, []).extend(pre)
    for lb in loop.exits:
        tr.block_prologue.setdefault(lb, []).extend(post)
    return max(slot, 8)
