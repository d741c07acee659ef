"""The array front end without a device: every function of the GPU suite's
tables is traced on shape-only arrays and each generated kernel is compiled
for sm_100a by NVRTC (library loaded, no GPU needed)."""

import numpy as np
import pytest

import test_numpy_reference_suite_gpu as suite


def _trace_and_compile(py_func, shapes_dtypes, scalars=()):
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy, runtime

    args = [lazy.fake_array(shape, dt) for shape, dt in shapes_dtypes] + list(scalars)
    trace, _plan = nm.njit(py_func).trace_dry(*args)
    launches = [s for s in trace.steps if s[0] == "launch"]
    for step in launches:
        assert len(runtime.compile_to_cubin(step[1])) > 0
    return trace, launches


@pytest.mark.parametrize("src", suite._unary)
def test_unary_functions_generate_valid_kernels(runtime_lib, src):
    _trace, launches = _trace_and_compile(eval("lambda a: " + src), [((2, 3), np.float32)])
    assert len(launches) <= 1  # one fused kernel per expression (none for the identity)


@pytest.mark.parametrize("src", suite._binary)
@pytest.mark.parametrize("dtype", [np.int32, np.float32])
def test_binary_functions_generate_valid_kernels(runtime_lib, src, dtype):
    _trace, launches = _trace_and_compile(eval("lambda a, b: " + src), [((2, 3), dtype), ((2, 3), dtype)])
    assert len(launches) == 1


@pytest.mark.parametrize("src", suite._bitwise)
def test_bitwise_functions_generate_valid_kernels(runtime_lib, src):
    _trace_and_compile(eval("lambda a, b: " + src), [((2, 3), np.int32), ((2, 3), np.int32)])


@pytest.mark.parametrize("src", suite._reduce_axis_funcs())
def test_reductions_record_reduce_steps(runtime_lib, src):
    trace, launches = _trace_and_compile(eval(src), [((2, 3), np.float32)])
    # a library reduction kernel, or a generated one when a chain feeds the reduction
    assert any(s[0] == "reduce" for s in trace.steps) or any(s[2] == "nmb_fused_reduce" for s in launches)


def test_black_scholes_chain_is_one_kernel(runtime_lib):
    from numba_mlir_b200 import workloads

    arrs = [((1 << 16,), np.float32)] * 3
    outs = [((1 << 16,), np.float32)] * 2
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy, runtime

    args = ([lazy.fake_array(s, d) for s, d in arrs] + [np.float32(0.1), np.float32(0.2)]
            + [lazy.fake_array(s, d) for s, d in outs])
    trace, plan = workloads.black_scholes.trace_dry(*args)
    launches = [s for s in trace.steps if s[0] == "launch"]
    assert len(launches) == 1 and plan is not None
    assert len(runtime.compile_to_cubin(launches[0][1])) > 0
    # the chain runs for two options at once: its own +, -, *, the library's log
    # and the @vectorize function that is nothing but erf use packed instructions
    src = bytes(launches[0][1]).decode()
    assert "nmb::log_pair(" in src and src.count("nmb::erf_pair(") == 2
    assert "nmb::sub2(" in src and "nmb::add2(" in src and "nmb::mul2(" in src


def test_fastmath_selects_the_approximate_division_and_sqrt(runtime_lib):
    """fastmath=True compiles without --fmad=false, with the approximate
    division and square root, and folds 1/sqrt(x) into one rsqrt
    (numba_mlir/mlir/tests/test_gpu.py:1900-1934 checks the flag reaches the
    device code); the default keeps the IEEE forms."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy, runtime

    def f(a, b):
        return a / b + np.float32(1.0) / np.sqrt(a)

    args = [lazy.fake_array((64,), np.float32), lazy.fake_array((64,), np.float32)]
    for fast in (False, True):
        trace, _plan = nm.njit(f, fastmath=fast).trace_dry(*args)
        (step,) = [s for s in trace.steps if s[0] == "launch"]
        src = bytes(step[1]).decode()
        assert ("#define NMB_FASTMATH 1" in src) == fast
        assert ("--fmad=false" in src) != fast
        assert ("nmb::f_rsqrt" in src) == fast
        assert len(runtime.compile_to_cubin(step[1])) > 0


def test_float32_arithmetic_is_emitted_for_two_elements_at_once(runtime_lib):
    """float32 +, - and * of a fused chain are emitted once per two adjacent
    elements (add/sub/mul.rn.f32x2); everything else and other element types
    keep the scalar form, and so does a multiply whose product something may
    add to (the assembler would merge the packed pair into a fused
    multiply-add) unless fastmath allows that contraction."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy, runtime

    def f(a, b):
        return np.sqrt((a - b) * (a + b)) + b

    def g(a, b):
        return a * b - a  # a product that feeds a subtraction stays a scalar multiply

    for dt, fast, packed in ((np.float32, False, True), (np.float64, False, False), (np.float32, True, True)):
        args = [lazy.fake_array((4096,), dt), lazy.fake_array((4096,), dt)]
        trace, _plan = nm.njit(f, fastmath=fast).trace_dry(*args)
        (step,) = [s for s in trace.steps if s[0] == "launch"]
        src = bytes(step[1]).decode()
        assert ("nmb::mul2(" in src and "nmb::sub2(" in src and "nmb::add2(" in src) == packed
        if packed:
            assert src.count("nmb::f_sqrt(") == 3  # both elements of the pair, and the one-element form
            assert "if constexpr (V % 2 == 0)" in src
        assert len(runtime.compile_to_cubin(step[1])) > 0
    args = [lazy.fake_array((4096,), np.float32), lazy.fake_array((4096,), np.float32)]
    trace, _plan = nm.njit(g).trace_dry(*args)
    (step,) = [s for s in trace.steps if s[0] == "launch"]
    src = bytes(step[1]).decode()
    assert "nmb::sub2(" in src and "nmb::mul2(" not in src
    trace, _plan = nm.njit(g, fastmath=True).trace_dry(*args)
    (step,) = [s for s in trace.steps if s[0] == "launch"]
    assert "nmb::mul2(" in bytes(step[1]).decode()


def test_array_building_functions_trace_and_compile(runtime_lib):
    """hstack / vstack / dstack, flip, outer, tril and triu of the reference's
    NumPy table (numba_mlir/mlir/numpy/funcs.py) become stores into slices,
    views with negative strides, a broadcast product and a select against row
    and column numbers: every kernel they generate compiles."""
    shapes = [((6, 8), np.float32), ((6, 8), np.float32), ((8,), np.float32), ((5,), np.float32)]
    for fn in (lambda a, b, v, w: np.vstack((a, b + 1)),
               lambda a, b, v, w: np.hstack((v, w)),
               lambda a, b, v, w: np.dstack((a, b)),
               lambda a, b, v, w: np.flip(a, axis=1) * 2,
               lambda a, b, v, w: np.outer(v, w),
               lambda a, b, v, w: np.triu(a, 1) + np.tril(b, -2)):
        _trace, launches = _trace_and_compile(fn, shapes)
        assert launches


def test_out_arguments_store_into_the_given_array(runtime_lib):
    """np.add(a, b, c) and np.clip(a, lo, hi, out=c) are one kernel each that
    writes c; no temporary is allocated."""
    shapes = [((6, 8), np.float32)] * 3
    for fn in (lambda a, b, c: np.add(a, b, c),
               lambda a, b, c: np.multiply(a, b, out=c),
               lambda a, b, c: np.clip(a, np.float32(0), np.float32(1), c),
               lambda a, b, c: np.clip(a, b, b + 1, out=c)):
        trace, launches = _trace_and_compile(fn, shapes)
        assert len(launches) == 1 and not [s for s in trace.steps if s[0] == "alloc"]


def test_index_arrays_become_a_gather_launch(runtime_lib):
    """a[m] with an integer array is one gather launch into a temporary of
    m's shape (plus a's trailing dimensions); views that the kernel cannot
    address directly are copied first."""
    trace, launches = _trace_and_compile(lambda a, m: a[m], [((16,), np.float32), ((3,), np.int32)])
    assert [s[2] for s in launches] == ["nmb_gather"]
    trace, launches = _trace_and_compile(lambda a, m: a[m] * 2, [((16, 4), np.float64), ((2, 3), np.int64)])
    assert [s[2] for s in launches] == ["nmb_gather", "nmb_fused"]
    trace, launches = _trace_and_compile(lambda a, m: a.T[m[::-1]], [((16, 4), np.float32), ((3,), np.int32)])
    assert [s[2] for s in launches].count("nmb_gather") == 1 and len(launches) == 3


def test_scalar_arguments_as_indices(runtime_lib):
    """a[b] = 42; return a[b] with b a scalar argument (numba_mlir/mlir/tests/
    test_numpy.py: test_setitem1, test_setitem2): views at the argument's
    value, one store; assignment through an index array is refused."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy

    def f(a, b):
        a[b] = 42
        return a[b]

    def g(a, b, c):
        a[b, c] = 42
        return a[b, c]

    for fn, args in ((f, [lazy.fake_array((3,), np.int64), -2]),
                     (g, [lazy.fake_array((2, 3), np.int64), 1, 2])):
        trace, _plan = nm.njit(fn).trace_dry(*args)
        assert [s[0] for s in trace.steps] == ["launch"]

    def scatter(a, m):
        a[m] = 1

    with pytest.raises(TypeError, match="index array"):
        nm.njit(scatter).trace_dry(lazy.fake_array((8,), np.float32), lazy.fake_array((3,), np.int32))


def _batchnorm(x, eps=1e-5):
    mean = np.empty(x.shape, dtype=x.dtype)
    mean[:] = np.sum(x, axis=0) / x.shape[0]
    std = np.empty(x.shape, dtype=x.dtype)
    std[:] = np.sqrt(np.sum((x - mean) ** 2, axis=0) / x.shape[0])
    return (x - mean) / np.sqrt(std + eps)


def _write_through_a_view(a, b):
    e = b[1:]
    c = a + b
    e[:] = c[1:]
    d = a - b
    return c, d


def _self_alias(n):
    a = np.arange(n)
    a[:] += 3 * np.flip(a)
    return a


def _atleast_2d_then_transpose(m, rowvar):
    m_arr = np.atleast_2d(m)
    if not rowvar:
        m_arr = m_arr.T
    return m_arr


_F32, _I32 = np.float32, np.int32
_BODIES = [
    # bodies of the reference's array tests (numba_mlir/mlir/tests/test_numpy.py), on shape-only arrays
    (_batchnorm, [((8, 14, 14, 32), _F32)], ()),
    (_write_through_a_view, [((12,), np.int64), ((12,), np.int64)], ()),
    (_self_alias, [], (1000,)),
    (_atleast_2d_then_transpose, [((4, 5), _F32)], (False,)),
    (lambda a, b, c: np.dot(a, b, out=c), [((8, 16), _F32), ((16, 8), _F32), ((8, 8), _F32)], ()),
    (lambda a: a * np.pi + np.e, [((16,), _F32)], ()),
    (lambda a, b: a.size / b, [((2, 3, 1), _F32)], (3,)),
    (lambda a: np.sum(a, dtype=np.int16, axis=0), [((4, 5), _I32)], ()),
    (lambda a: np.prod(a, dtype=np.int16), [((4, 5), _I32)], ()),
    (lambda a: np.mean(a, axis=0, keepdims=True) + np.var(a, axis=0), [((4, 8), _F32)], ()),
    (lambda a: np.std(a) + a.sum(axis=0), [((4, 8), _F32)], ()),
    (lambda a: a ** 2 + a ** 0.5, [((16,), _F32)], ()),
    (lambda a: a.astype(np.int32), [((16,), _F32)], ()),
    (lambda a: a[::-1] + a[1:3, None].sum(), [((16,), _F32)], ()),
    (lambda a: a[1:3, :, ::2] * 2 + a[..., 0][1:3, :, None], [((4, 5, 6), _F32)], ()),
    (lambda a, b: a // b + a % b, [((16,), _F32), ((16,), _F32)], ()),
    (lambda a, b: (a << 1) + (b >> 1) + (a & b) + (a | b) + (a ^ b) + ~a, [((16,), _I32), ((16,), _I32)], ()),
    (lambda a, b: np.logical_and(a > 0, b > 0) | np.logical_not(a > b), [((16,), _F32), ((16,), _F32)], ()),
    (lambda a: np.any(a > 0) & np.all(a > 0), [((16,), _F32)], ()),
    (lambda a: np.count_nonzero(a) + np.argmax(a), [((4, 16), _F32)], ()),
    (lambda a: np.tanh(a) + np.arctan2(a, a) + np.hypot(a, a) + np.floor(a) + np.ceil(a) + np.trunc(a)
     + np.sign(a), [((16,), _F32)], ()),
    (lambda a: np.isfinite(a) | np.isinf(a) | np.isnan(a), [((16,), _F32)], ()),
    (lambda a: a.flatten() + np.ravel(a) + a.reshape(-1), [((4, 4), _F32)], ()),
    (lambda a: (a + a.size + a.itemsize + a.strides[0] + len(a), a.shape, a.T), [((8, 16), _F32)], ()),
    (lambda a, m: a[m] + a[m[::-1]], [((16,), _F32), ((3,), _I32)], ()),
    # axis views: new, dropped, permuted and stretched axes
    (lambda a: np.expand_dims(a, 0) + np.expand_dims(a, -1), [((16,), _F32)], ()),
    (lambda a: np.squeeze(a * 2, axis=0) + np.squeeze(a, axis=(0, 2))[:, None], [((1, 16, 1), _F32)], ()),
    (lambda a: np.broadcast_to(a, (3, 4, 5)) * 2, [((4, 1), _F32)], ()),
    (lambda a: np.swapaxes(a, 0, 2) + np.transpose(a, (2, 1, 0)), [((3, 4, 5), _F32)], ()),
]


@pytest.mark.parametrize("case", range(len(_BODIES)))
def test_bodies_of_the_reference_array_tests_trace_and_compile(runtime_lib, case):
    py_func, arrays, scalars = _BODIES[case]
    _trace_and_compile(py_func, arrays, scalars)


def test_view_operations_give_numpy_shapes_and_strides():
    """The views a recorded plan re-applies to new arguments (transpose,
    permutation, broadcast, indexing, reshape) have NumPy's shape and strides."""
    from numba_mlir_b200 import lazy

    host = np.zeros((3, 1, 5), np.float32)
    dev = lazy.fake_array(host.shape, host.dtype)
    for op, want in ((("T",), host.T),
                     (("transpose", (2, 0, 1)), host.transpose(2, 0, 1)),
                     (("broadcast", (4, 3, 6, 5)), np.broadcast_to(host, (4, 3, 6, 5))),
                     (("getitem", (slice(1, None), 0, slice(None, None, -2))), host[1:, 0, ::-2]),
                     (("reshape", (5, 3)), host.reshape(5, 3))):
        got = lazy._apply_view(dev, op)
        assert got.shape == want.shape and tuple(got.strides) == want.strides, op


def test_argmin_of_a_chain_along_the_last_axis_is_one_kernel(runtime_lib):
    """np.argmin / np.argmax of an elementwise chain along the last axis is
    one generated kernel (a warp per row keeps value and position); along
    another axis the chain goes to a temporary and the library kernel."""
    _trace, launches = _trace_and_compile(lambda a, b: np.argmin(a * a - b, axis=1),
                                          [((512, 256), np.float32), ((512, 256), np.float32)])
    assert [s[2] for s in launches] == ["nmb_fused_reduce"] and len(_trace.steps) == 2  # alloc + launch
    assert "reduce_rows_arg_fused<256, 4, 4, true>" in bytes(launches[0][1]).decode()
    trace, launches = _trace_and_compile(lambda a: np.argmax(a * 2, axis=0), [((512, 256), np.float32)])
    assert [s[0] for s in trace.steps].count("reduce") == 1 and [s[2] for s in launches] == ["nmb_fused"]


def test_arrays_created_inside_a_function_are_device_temporaries(runtime_lib):
    """np.empty / zeros / ones / full called with a shape inside a traced
    function (numba_mlir/mlir/numpy/funcs.py types numpy.empty, zeros, ones)
    give device temporaries, so `out = np.empty(n); out[:] = ...; return out`
    works and the call is recorded as a replayable plan; outside a trace the
    same names are NumPy's."""
    import numba_mlir_b200 as nm
    from numba_mlir_b200 import lazy

    def f(a):
        out = np.empty(a.shape, a.dtype)
        out[:] = a + np.float32(1)
        acc = np.zeros(a.shape[0], np.float32)
        acc += out
        return acc * np.ones(a.shape, dtype=np.float32) + np.full(a.shape, 2.5, np.float32)

    trace, plan = nm.njit(f).trace_dry(lazy.fake_array((256,), np.float32))
    assert plan is not None and [s[0] for s in trace.steps].count("alloc") >= 4
    assert isinstance(lazy.with_device_creators(f)(np.ones(3, np.float32)), np.ndarray)  # no trace: plain NumPy


def test_large_local_arrays_move_to_the_local_memory_parameter(runtime_lib):
    """Local arrays stay static shared memory while the kernel's static total
    fits 48 KB; above that the kernel takes an offset parameter and the launch carries a local-memory
    request of the arrays' total size (16-byte aligned pieces)."""
    from numba_mlir_b200 import codegen_ir, lazy, runtime
    from numba_mlir_b200.kernel import get_local_id, local

    def small(a):
        t = local.array(1024, np.float32)
        t[get_local_id(0)] = a[get_local_id(0)]

    def big(a):
        t = local.array(20000, np.float32)
        u = local.array(3, np.int32)
        t[get_local_id(0)] = a[get_local_id(0)]
        u[0] = 1

    args = [lazy.fake_array((256,), np.float32)]
    ck = codegen_ir.compile_kernel(small, args, 1)
    assert ck.local_bytes == 0 and "nmb_local_off" not in ck.source
    assert ck.kinds(3)[-1] == np.dtype(np.int64)
    ck = codegen_ir.compile_kernel(big, args, 1)
    assert ck.local_bytes == 80000 + 16 and "unsigned long long nmb_local_off" in ck.source
    assert ck.kinds(3)[-1] == ("local", 80016)
    assert len(runtime.compile_to_cubin(ck.source.encode())) > 0


# ---------------------------------------------------- ordering of reads/writes ---
def _dry(py_func, arrays):
    import numba_mlir_b200 as nm

    trace, _plan = nm.njit(py_func).trace_dry(*arrays)
    return trace


def test_store_after_an_unevaluated_read_keeps_the_old_values():
    """`b = a + 1; a[:] = 0; a.sum(); o[:] = b`: b is evaluated from the
    values a had when b was written down, not from the zeros."""
    from numba_mlir_b200 import lazy

    def g(a, o):
        b = a + np.float32(1)
        a[:] = np.float32(0)
        s = a.sum()
        o[:] = b
        return s

    a, o = lazy.fake_array((64,), np.float32), lazy.fake_array((64,), np.float32)
    trace = _dry(g, [a, o])
    launches = [s for s in trace.steps if s[0] == "launch"]
    # first launch: the temporary for b (reads a) together with the zeroing of a
    first = [p[1] for p in launches[0][5] if p[0] == "slot"]
    assert 0 in first and any(trace.slots[s][0] == "tmp" for s in first)
    # the launch that writes o reads that temporary, not a
    last = [p[1] for p in launches[-1][5] if p[0] == "slot"]
    assert 1 in last and 0 not in last
    assert any(trace.slots[s][0] == "tmp" for s in last)


def test_shifted_self_assignment_goes_through_a_temporary():
    """`a[1:] = a[:-1]`: two kernels (NumPy copies on overlap), never one
    kernel reading and writing shifted views of one buffer."""

    from numba_mlir_b200 import lazy

    def shift(a):
        a[1:] = a[:-1]

    def rev(a):
        b = a[::-1] + np.float32(1)
        a[:] = np.float32(0)
        return b

    for fn in (shift, rev):
        trace = _dry(fn, [lazy.fake_array((64,), np.float32)])
        launches = [s for s in trace.steps if s[0] == "launch"]
        assert len(launches) == 2, fn.__name__
        for step in launches:
            slots = [p[1] for p in step[5] if p[0] == "slot"]
            for x in slots:
                for y in slots:
                    assert trace.overlap(x, y) != 2


def test_in_place_update_stays_one_kernel_without_restrict():
    from numba_mlir_b200 import lazy

    def f(a, b):
        a[:] = a * np.float32(2) + b

    trace = _dry(f, [lazy.fake_array((256,), np.float32), lazy.fake_array((256,), np.float32)])
    (step,) = [s for s in trace.steps if s[0] == "launch"]
    src = bytes(step[1]).decode()
    assert "const float* in0," in src and "float* out0," in src  # a: read and written
    assert "const float* __restrict__ in1" in src


def test_plan_key_sees_overlapping_arguments():
    from numba_mlir_b200 import lazy

    a = lazy.fake_array((64,), np.float32)
    b = lazy.fake_array((64,), np.float32)
    assert lazy.signature_of((a, b)) != lazy.signature_of((a, a))
    assert lazy.signature_of((a[1:], a[:-1])) != lazy.signature_of((a[1:], b[:-1]))


# ------------------------------------------------ gpu_use_64bit_index=False ---
def test_32bit_index_mode_narrows_index_values_only(runtime_lib):
    """With gpu_use_64bit_index=False ids, loop counters, shapes and what is
    computed from them are 32-bit C variables; values read from arrays and
    scalar arguments keep their 64 bits
    (numba_mlir/mlir/lib/Conversion/GpuToGpuRuntime.cpp:976-1030 types `index`
    as i32 under that flag)."""
    import re

    from numba_mlir_b200 import codegen_ir, lazy, runtime
    from numba_mlir_b200.kernel import get_global_id

    def body(a, table, big, out):
        i = get_global_id(0)
        n = a.shape[0]
        acc = 0
        for j in range(n // 4):
            acc += table[(i + j) % n]      # a value read from an int64 array: wide
        out[i] = acc + big                 # big: a scalar int64 argument: wide

    args = [lazy.fake_array((64,), np.float32), lazy.fake_array((64,), np.int64), np.int64(1 << 40),
            lazy.fake_array((64,), np.int64)]
    wide = codegen_ir.compile_kernel(body, args, 1).source
    narrow = codegen_ir.compile_kernel(body, args, 1, index32=True).source
    assert "int32_t v" not in wide
    decl = {m.group(2): m.group(1) for m in re.finditer(r"\b(int32_t|int64_t) (v\d+_\w+?)(?:, |;)", narrow)}
    kinds = {name.split("_", 1)[1]: ct for name, ct in decl.items()}
    assert kinds["i"] == "int32_t" and kinds["n"] == "int32_t"
    assert any(k.startswith("j") and ct == "int32_t" for k, ct in kinds.items())
    assert any(k.startswith("acc") and ct == "int64_t" for k, ct in kinds.items())
    assert "(int32_t)(" in narrow and "int32_t v1_table_s0" in narrow.replace("  ", " ")
    for src in (wide, narrow):
        assert len(runtime.compile_to_cubin(src)) > 0


# ------------------------------------------------------- packed inner loops ---
def test_independent_constant_loops_are_emitted_two_iterations_at_a_time(runtime_lib):
    """A `for q in range(2)` loop over private arrays whose iterations do not
    depend on one another is emitted as straight-line code with the float32
    subtraction and addition of the two iterations packed (nmb::sub2 / add2);
    the multiply that feeds the addition stays scalar, because the assembler
    would merge a packed multiply into a dependent packed add.  Loops that
    carry a value from one iteration to the next keep their loop form."""
    from numba_mlir_b200 import codegen_ir, lazy, runtime
    from numba_mlir_b200.kernel import get_global_id, private

    def independent(x, c, out):
        i = get_global_id(0)
        p = private.array((2, 4), np.float32)
        d = private.array(2, np.float32)
        for q in range(2):
            for j in range(4):
                p[q, j] = x[2 * i + q, j]
            d[q] = np.float32(0.0)
        for j in range(4):
            cj = c[j]
            for q in range(2):
                t = p[q, j] - cj
                d[q] += t * t
        out[2 * i] = d[0]
        out[2 * i + 1] = d[1]

    def carried(x, out):
        i = get_global_id(0)
        d = private.array(4, np.float32)
        s = np.float32(0.0)
        for q in range(4):
            s = s + x[4 * i + q]      # a running value: iteration q reads iteration q - 1
            d[q] = s * np.float32(2.0)
        out[i] = d[3]

    def shifted(x, out):
        i = get_global_id(0)
        d = private.array(5, np.float32)
        d[0] = x[i]
        for q in range(4):
            d[q + 1] = d[q] + np.float32(1.0)   # not indexed by the loop variable itself
        out[i] = d[4]

    x2 = lazy.fake_array((64, 4), np.float32)
    c = lazy.fake_array((4,), np.float32)
    x1 = lazy.fake_array((64,), np.float32)
    out = lazy.fake_array((64,), np.float32)
    ck = codegen_ir.compile_kernel(independent, [x2, c, out], 1)
    assert ck.source.count("nmb::sub2(") == 1 and ck.source.count("nmb::add2(") == 1
    assert "nmb::mul2(" not in ck.source
    assert len(runtime.compile_to_cubin(ck.source.encode())) > 0
    for fn, args in ((carried, [x1, out]), (shifted, [x1, out])):
        ck = codegen_ir.compile_kernel(fn, args, 1)
        assert "nmb::add2(" not in ck.source and "nmb::mul2(" not in ck.source
        assert len(runtime.compile_to_cubin(ck.source.encode())) > 0
