"""Generates tests/golden/kernel_sim.npz by running the REFERENCE's own kernel
simulator (numba_mlir/numba_mlir/mlir/kernel_sim_impl.py, loaded by file path
from a checkout of the reference) on the inputs of the reference's GPU tests.

    python tests/golden/make_golden.py /path/to/numba-mlir

The reference checkout is only needed to regenerate the file; the tests read
the committed .npz.  Each case re-derives its inputs from the cited test.
"""

import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# Shared with the tests that replay these cases.
SCALAR_VALUES = [True, False, -3, 0, 2, -2.5, -0.0, 0.5]
MATH_UNARY = ["sqrt", "log", "exp", "sin", "cos", "erf", "tanh", "floor", "ceil", "acos"]
BINARY_OPS = {"add": "+", "sub": "-", "mul": "*", "truediv": "/", "floordiv": "//", "mod": "%", "pow": "**"}


def load_sim(ref_root):
    path = os.path.join(ref_root, "numba_mlir", "numba_mlir", "mlir", "kernel_sim_impl.py")
    spec = importlib.util.spec_from_file_location("ref_kernel_sim_impl", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    sim = load_sim(ref_root)
    out = {}

    def run(func, gs, ls, args):
        sim.execute_kernel(tuple(gs), tuple(ls), func, args, False, lambda g: g)

    # atomics: mlir/tests/test_gpu.py:820-954; the simulator's read-modify-write
    # (kernel_sim.py:24-35) is restated inline because kernel_sim.py itself needs
    # the native extension.
    def atomic_add(arr, ind, val):
        new = arr[ind] + val
        arr[ind] = new
        return new

    def atomic_sub(arr, ind, val):
        new = arr[ind] - val
        arr[ind] = new
        return new

    for dtype in ("int32", "int64", "float32"):
        a = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9], dtype)
        for opname, op in (("add", atomic_add), ("sub", atomic_sub)):
            def k_simple(a, b):
                i = sim.get_global_id(0)
                op(b, 0, a[i])

            def k_offset(a, b):
                i = sim.get_global_id(0)
                op(b, i % 2, a[i])

            res = np.zeros([1], dtype)
            run(k_simple, a.shape, (), (a, res))
            out[f"atomic_{opname}_{dtype}"] = res
            res = np.zeros([2], dtype)
            run(k_offset, a.shape, (), (a, res))
            out[f"atomic_{opname}_offset_{dtype}"] = res

        a2 = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], dtype)

        def k_2d(a, b):
            i = sim.get_global_id(0)
            j = sim.get_global_id(1)
            atomic_add(b, (i % 2, j % 2), a[i, j])

        res = np.zeros((2, 2), dtype)
        run(k_2d, a2.shape, (), (a2, res))
        out[f"atomic_add_2d_{dtype}"] = res

    # ids and sizes: mlir/tests/test_gpu.py:580-803, (global, local) pairs of
    # :1077-1078 where the global size is not a multiple of the local size
    for gsize, lsize in ((27, 7), (67, 17), (101, 33), (4, 2)):
        def k_ids(gid, lid, grp, gsz, lsz):
            i = sim.get_global_id(0)
            gid[i] = i
            lid[i] = sim.get_local_id(0)
            grp[i] = sim.get_group_id(0)
            gsz[i] = sim.get_global_size(0)
            lsz[i] = sim.get_local_size(0)

        arrs = [np.full(gsize, -1, np.int64) for _ in range(5)]
        run(k_ids, (gsize,), (lsize,), tuple(arrs))
        for name, arr in zip(("gid", "lid", "grp", "gsz", "lsz"), arrs):
            out[f"ids_{gsize}_{lsize}_{name}"] = arr

    def k_ids2(out2):
        i = sim.get_global_id(0)
        j = sim.get_global_id(1)
        out2[i, j] = 1000 * sim.get_group_id(0) + 100 * sim.get_group_id(1) + \
            10 * sim.get_local_id(0) + sim.get_local_id(1)

    res = np.zeros((5, 7), np.int64)
    run(k_ids2, (5, 7), (2, 3), (res,))
    out["ids2d_5x7_2x3"] = res

    # pairwise distance kernel: mlir/tests/test_gpu.py:1396-1430
    def k_pair(X1, X2, D):
        i = sim.get_global_id(0)
        j = sim.get_global_id(1)
        d = 0.0
        for k in range(X1.shape[1]):
            tmp = X1[i, k] - X2[j, k]
            d += tmp * tmp
        D[i, j] = np.sqrt(d)

    a = np.arange(128 * 3, dtype=np.float32).reshape(128, 3)
    b = a + 5
    res = np.zeros((128, 128), np.float32)
    run(k_pair, (128, 128), (), (a, b, res))
    out["pairwise1"] = res

    # scalar argument / captured scalar: mlir/tests/test_gpu.py:288-345
    for dtype in ("int32", "int64", "float32", "float64"):
        a = np.arange(-6, 6, dtype=dtype)
        for vi, val in enumerate(SCALAR_VALUES):
            def k_scalar(a, b, c):
                i = sim.get_global_id(0)
                c[i] = a[i] + b

            res = np.zeros(a.shape, a.dtype)
            run(k_scalar, a.shape, (), (a, val, res))
            out[f"scalar_{dtype}_{vi}"] = res

    # unary math: mlir/tests/test_gpu.py:484-556
    import math

    for dtype in ("float32", "float64"):
        a = np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9], dtype)
        for op in MATH_UNARY:
            f = getattr(math, op)

            def k_unary(a, b):
                i = sim.get_global_id(0)
                b[i] = f(a[i])

            res = np.zeros(a.shape, dtype)
            run(k_unary, a.shape, (), (a, res))
            out[f"unary_{op}_{dtype}"] = res

    # binary operators: mlir/tests/test_gpu.py:559-575
    for dtype in ("int32", "float32", "float64"):
        a = np.array([11, 12, 13, 14, 15], dtype)
        b = np.array([1, 2, 3, 4, 5], dtype)
        for name, op in BINARY_OPS.items():
            f = eval(f"lambda a, b: a {op} b")

            def k_binary(a, b, c):
                i = sim.get_global_id(0)
                c[i] = f(a[i], b[i])

            res = np.zeros(a.shape, dtype)
            run(k_binary, a.shape, (), (a, b, res))
            out[f"binary_{name}_{dtype}"] = res

    # inner loop with a data-dependent trip count: mlir/tests/test_gpu.py:455-481
    def k_inner(a, b, c):
        i = sim.get_global_id(0)
        res = 0.0
        for j in range(a[i]):
            res = res + b[j]
        c[i] = res

    a = np.array([1, 2, 3, 4], np.int32)
    b = np.array([5, 6, 7, 8, 9], np.float32)
    res = np.zeros(a.shape, b.dtype)
    run(k_inner, a.shape, (), (a, b, res))
    out["inner_loop"] = res

    # sub-array views: mlir/tests/test_gpu.py:429-452
    def k_slice(a, b):
        i = sim.get_global_id(0)
        b1 = b[i]
        j = sim.get_global_id(1)
        b2 = b1[j]
        k = sim.get_global_id(2)
        b2[k] = a[i, j, k]

    a = np.arange(3 * 4 * 5).reshape((3, 4, 5))
    res = np.zeros(a.shape, a.dtype)
    run(k_slice, a.shape, (), (a, res))
    out["slice"] = res

    # private arrays: mlir/tests/test_gpu.py:1255-1287 (the simulator's
    # private.array is local_array's zero-filled buffer per work-item)
    for blocksize in (1, 10, 17, 64, 67, 101):
        for priv_size in (1, 11, 27):
            def k_private(A):
                i = sim.get_global_id(0)
                prvt_mem = sim.private_array(priv_size, np.float32)
                for j in range(priv_size):
                    prvt_mem[j] = j + i
                res = 0
                for j in range(priv_size):
                    res += prvt_mem[(j + i) % priv_size]
                A[i] = res

            res = np.zeros(blocksize, np.float32)
            run(k_private, (blocksize,), (blocksize,), (res,))
            out[f"private3_{blocksize}_{priv_size}"] = res

    # ids and sizes in three dimensions with a (2, 4, 8) group: mlir/tests/test_gpu.py:578-803
    def k_ids3(gid, lid, grp, gsz, lsz):
        i = sim.get_global_id(0)
        j = sim.get_global_id(1)
        k = sim.get_global_id(2)
        gid[i, j, k] = i + j * 100 + k * 10000
        lid[i, j, k] = sim.get_local_id(0) + sim.get_local_id(1) * 100 + sim.get_local_id(2) * 10000
        grp[i, j, k] = sim.get_group_id(0) + sim.get_group_id(1) * 100 + sim.get_group_id(2) * 10000
        gsz[i, j, k] = sim.get_global_size(0) + sim.get_global_size(1) * 100 + sim.get_global_size(2) * 10000
        lsz[i, j, k] = sim.get_local_size(0) + sim.get_local_size(1) * 100 + sim.get_local_size(2) * 10000

    arrs = [np.zeros((7, 13, 23), np.int32) for _ in range(5)]
    run(k_ids3, (7, 13, 23), (2, 4, 8), tuple(arrs))
    for name, arr in zip(("gid", "lid", "grp", "gsz", "lsz"), arrs):
        out[f"ids3d_7x13x23_2x4x8_{name}"] = arr

    np.savez_compressed(os.path.join(HERE, "kernel_sim.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a numba-mlir checkout>")
    main(sys.argv[1])
