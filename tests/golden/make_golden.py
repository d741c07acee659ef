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

    np.savez_compressed(os.path.join(HERE, "kernel_sim.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a numba-mlir checkout>")
    main(sys.argv[1])
