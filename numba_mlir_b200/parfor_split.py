"""Functions with several parallel loops, or loops mixed with array expressions.

The reference compiles such a function into one host function holding one
`gpu.launch` per parallel loop nest, with the scalar code between them on the
host (numba_mlir/mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940; tests
mlir/tests/test_gpu.py:1523-1613), and `njit_replace_parfors` leaves the host
code to Numba and offloads only the loops (numba_mlir/mlir/passes.py:332-416).

Here the function's source is rewritten once: every outermost `prange` loop
becomes a call to a helper function that holds just that loop (its live-in
names as parameters, a scalar it carries out as return value), and each
helper is compiled as a whole into one kernel by
`codegen_ir.compile_parfor`.  What is left -- array expressions, scalar
arithmetic, control flow on host values -- runs as the ordinary traced
function around those calls.
"""

import ast
import inspect
import textwrap

_PRANGE_NAMES = ("prange",)


class SplitError(TypeError):
    """The function's loops cannot be cut out (no source, unsupported form)."""


def _is_prange_loop(node):
    if not isinstance(node, ast.For) or not isinstance(node.iter, ast.Call):
        return False
    f = node.iter.func
    name = f.id if isinstance(f, ast.Name) else f.attr if isinstance(f, ast.Attribute) else None
    return name in _PRANGE_NAMES


def _function_ast(py_func):
    try:
        src = textwrap.dedent(inspect.getsource(py_func))
    except (OSError, TypeError) as e:
        raise SplitError(f"{getattr(py_func, '__name__', py_func)}: source not available ({e})") from None
    tree = ast.parse(src)
    fn = tree.body[0]
    if not isinstance(fn, ast.FunctionDef):
        raise SplitError("only plain `def` functions can be split into loops and host code")
    return fn


def count_outer_prange_loops(py_func):
    """Number of `prange` loops that are not nested in another loop; 0 when the
    source cannot be read."""
    try:
        fn = _function_ast(py_func)
    except SplitError:
        return 0
    count = 0

    def visit(stmts):
        nonlocal count
        for st in stmts:
            if _is_prange_loop(st):
                count += 1
            elif isinstance(st, (ast.For, ast.While)):
                continue  # a sequential loop around prange loops is not split
            elif isinstance(st, (ast.If, ast.With, ast.Try)):
                for field in ("body", "orelse", "finalbody"):
                    visit(getattr(st, field, []))

    visit(fn.body)
    return count


def _names(nodes, ctx):
    out = set()
    for n in nodes:
        for sub in ast.walk(n):
            if isinstance(sub, ast.Name) and isinstance(sub.ctx, ctx):
                out.add(sub.id)
    return out


def _stores(nodes):
    """Names bound by the statements: plain, augmented and loop-target stores."""
    return _names(nodes, ast.Store)


def _subscript_roots(nodes):
    """Names whose elements are written (`x[i] = ...`, `x[i] += ...`)."""
    out = set()
    for n in nodes:
        for sub in ast.walk(n):
            targets = []
            if isinstance(sub, ast.Assign):
                targets = sub.targets
            elif isinstance(sub, (ast.AugAssign, ast.AnnAssign)):
                targets = [sub.target]
            for t in targets:
                while isinstance(t, (ast.Subscript, ast.Attribute)):
                    t = t.value
                    if isinstance(t, ast.Name):
                        out.add(t.id)
    return out


def split(py_func, make_loop_function):
    """Rewrites `py_func`.  `make_loop_function(helper)` wraps each loop helper
    (a plain function holding one prange loop) into what the rewritten function
    calls in its place.  Returns (rewritten function, number of loops cut out).
    """
    fn = _function_ast(py_func)
    params = [a.arg for a in fn.args.posonlyargs + fn.args.args + fn.args.kwonlyargs]
    if fn.args.vararg or fn.args.kwarg:
        raise SplitError("*args / **kwargs are not supported in offloaded functions")
    local_names = set(params) | _stores(fn.body)
    helpers = []

    def cut(loop, bound_before):
        """Replaces one outermost prange loop by a call to its helper."""
        index = len(helpers)
        name = f"__nmb_loop{index}_{fn.name}"
        used = _names([loop], ast.Load)
        stored = _stores([loop])
        loop_targets = _stores([loop.target])
        # parameters: local names the loop reads (or updates) that exist before it
        live_in = sorted((used | stored) & local_names & bound_before)
        # carried out: scalars bound before the loop and rebound inside it
        written_elements = _subscript_roots([loop])
        carried = sorted((stored - loop_targets) & bound_before - written_elements)
        if len(carried) > 1:
            raise SplitError(
                f"{fn.name}: the prange loop at line {loop.lineno} carries several scalars out "
                f"({', '.join(carried)}); one per loop is supported")
        body = [loop]
        if carried:
            body.append(ast.Return(value=ast.Name(id=carried[0], ctx=ast.Load())))
        helper = ast.FunctionDef(
            name=name,
            args=ast.arguments(posonlyargs=[], args=[ast.arg(arg=a) for a in live_in], vararg=None,
                               kwonlyargs=[], kw_defaults=[], kwarg=None, defaults=[]),
            body=body, decorator_list=[], returns=None, type_comment=None)
        try:
            helper.type_params = []
        except Exception:
            pass
        helpers.append((name, helper))
        call = ast.Call(func=ast.Name(id=name, ctx=ast.Load()),
                        args=[ast.Name(id=a, ctx=ast.Load()) for a in live_in], keywords=[])
        if carried:
            return ast.Assign(targets=[ast.Name(id=carried[0], ctx=ast.Store())], value=call)
        return ast.Expr(value=call)

    def rewrite(stmts, bound):
        """Rewrites a statement list in order, tracking the names bound so far."""
        out = []
        for st in stmts:
            if _is_prange_loop(st):
                out.append(cut(st, set(bound)))
                bound |= _stores([st]) - _stores([st.target])
            elif isinstance(st, (ast.If, ast.With, ast.Try)):
                for field in ("body", "orelse", "finalbody"):
                    if getattr(st, field, None):
                        setattr(st, field, rewrite(getattr(st, field), bound))
                out.append(st)
                bound |= _stores([st])
            else:
                out.append(st)
                bound |= _stores([st])
        return out

    fn.decorator_list = []
    fn.body = rewrite(fn.body, set(params))
    if not helpers:
        raise SplitError(f"{fn.name}: no outermost prange loop found")
    module = ast.Module(body=[h for _n, h in helpers] + [fn], type_ignores=[])
    ast.fix_missing_locations(module)
    namespace = dict(py_func.__globals__)
    if py_func.__closure__:
        for cell_name, cell in zip(py_func.__code__.co_freevars, py_func.__closure__):
            try:
                namespace[cell_name] = cell.cell_contents
            except ValueError:
                pass
    filename = f"<numba_mlir_b200 split of {py_func.__name__}>"
    source = ast.unparse(module)
    # the helpers' source must be retrievable: Numba's front end and tracebacks read it
    import linecache

    linecache.cache[filename] = (len(source), None, source.splitlines(True), filename)
    exec(compile(source, filename, "exec"), namespace)
    for name, _h in helpers:
        namespace[name] = make_loop_function(namespace[name])
    return namespace[fn.name], len(helpers)
