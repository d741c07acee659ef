"""Kernel cases shared by the simulator pin (CPU) and the device parity test
(GPU): the same bodies, inputs and launch shapes as tests/golden/make_golden.py
ran through the reference's own simulator.  Every case yields
(golden key, function, global size, local size, arguments, index of the output
argument, exact?)."""

import math
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden import BINARY_OPS, MATH_UNARY, SCALAR_VALUES  # noqa: E402


def cases(for_device=False):
    """`for_device`: helper functions called from kernels are wrapped in
    `kernel_func`, which the code generator needs and the simulator must not see."""
    from numba_mlir_b200.kernel import (DEFAULT_LOCAL_SIZE, get_global_id, get_global_size, get_group_id,
                                        get_local_id, get_local_size, kernel_func, private)

    private_array = private.array
    for dtype in ("int32", "int64", "float32", "float64"):
        a = np.arange(-6, 6, dtype=dtype)
        for vi, val in enumerate(SCALAR_VALUES):
            def k_scalar(a, b, c):
                i = get_global_id(0)
                c[i] = a[i] + b

            yield f"scalar_{dtype}_{vi}", k_scalar, a.shape, DEFAULT_LOCAL_SIZE, [a, val, np.zeros_like(a)], 2, True

    for dtype in ("float32", "float64"):
        a = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9], dtype)
        for op in MATH_UNARY:
            f = getattr(math, op)

            def make(f):
                def k_unary(a, b):
                    i = get_global_id(0)
                    b[i] = f(a[i])
                return k_unary

            yield f"unary_{op}_{dtype}", make(f), a.shape, DEFAULT_LOCAL_SIZE, [a, np.zeros_like(a)], 1, False

    for dtype in ("int32", "float32", "float64"):
        a = np.array([11, 12, 13, 14, 15], dtype)
        b = np.array([1, 2, 3, 4, 5], dtype)
        for name, op in BINARY_OPS.items():
            def make(op):
                f = eval(f"lambda a, b: a {op} b")
                if for_device:
                    f = kernel_func(f)

                def k_binary(a, b, c):
                    i = get_global_id(0)
                    c[i] = f(a[i], b[i])
                return k_binary

            yield (f"binary_{name}_{dtype}", make(op), a.shape, DEFAULT_LOCAL_SIZE,
                   [a, b, np.zeros_like(a)], 2, False)

    def k_inner(a, b, c):
        i = get_global_id(0)
        res = 0.0
        for j in range(a[i]):
            res = res + b[j]
        c[i] = res

    a = np.array([1, 2, 3, 4], np.int32)
    b = np.array([5, 6, 7, 8, 9], np.float32)
    yield "inner_loop", k_inner, a.shape, DEFAULT_LOCAL_SIZE, [a, b, np.zeros(a.shape, b.dtype)], 2, True

    def k_slice(a, b):
        i = get_global_id(0)
        b1 = b[i]
        j = get_global_id(1)
        b2 = b1[j]
        k = get_global_id(2)
        b2[k] = a[i, j, k]

    a = np.arange(3 * 4 * 5).reshape((3, 4, 5))
    yield "slice", k_slice, a.shape, DEFAULT_LOCAL_SIZE, [a, np.zeros_like(a)], 1, True

    for blocksize in (1, 10, 17, 64, 67, 101):
        for priv_size in (1, 11, 27):
            def make(priv_size):
                def k_private(A):
                    i = get_global_id(0)
                    prvt_mem = private_array(priv_size, np.float32)
                    for j in range(priv_size):
                        prvt_mem[j] = j + i
                    res = 0
                    for j in range(priv_size):
                        res += prvt_mem[(j + i) % priv_size]
                    A[i] = res
                return k_private

            yield (f"private3_{blocksize}_{priv_size}", make(priv_size), (blocksize,), (blocksize,),
                   [np.zeros(blocksize, np.float32)], 0, True)

    def k_ids3(gid, lid, grp, gsz, lsz):
        i = get_global_id(0)
        j = get_global_id(1)
        k = get_global_id(2)
        gid[i, j, k] = i + j * 100 + k * 10000
        lid[i, j, k] = get_local_id(0) + get_local_id(1) * 100 + get_local_id(2) * 10000
        grp[i, j, k] = get_group_id(0) + get_group_id(1) * 100 + get_group_id(2) * 10000
        gsz[i, j, k] = get_global_size(0) + get_global_size(1) * 100 + get_global_size(2) * 10000
        lsz[i, j, k] = get_local_size(0) + get_local_size(1) * 100 + get_local_size(2) * 10000

    arrs = [np.zeros((7, 13, 23), np.int32) for _ in range(5)]
    for n, name in enumerate(("gid", "lid", "grp", "gsz", "lsz")):
        yield f"ids3d_7x13x23_2x4x8_{name}", k_ids3, (7, 13, 23), (2, 4, 8), arrs, n, True
