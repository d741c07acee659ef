"""Host dispatch of the tensor-core contraction entry points.

`gemm` is what `np.dot` on device arrays reaches in the reference
(numba_mlir/mlir/numpy/funcs.py:752-812 -> "mkl_gemm_float32_device");
`pairwise_distance` is the fused distance routine surfaced as a device library
call next to it.  Both go through the C-ABI symbols of the runtime library.
"""

import ctypes

import numpy as np

from . import runtime as _rt
from .device_array import empty


def _memref(a, dtype=np.float32):
    if a.dtype != dtype or a.ndim != 2:
        raise TypeError(f"this routine takes 2-D {np.dtype(dtype).name} device arrays")
    it = a.dtype.itemsize
    m = _rt.Memref2f()
    m.userData = None
    m.data = a.ptr
    m.offset = 0
    m.dims[0], m.dims[1] = a.shape
    st = [s // it for s in a.strides]
    if any(s < 0 for s in st):
        raise ValueError("negative strides are not supported")
    m.strides[0], m.strides[1] = st
    return m


def gemm(a, b, c, alpha=1.0, beta=0.0, blocking=True):
    """c = alpha * a @ b + beta * c.  Blocking like the reference's call by
    default; `blocking=False` only enqueues it on the queue's stream."""
    lib = _rt.load()
    if a.dtype == np.float64:
        # the float64 entry (CUDA cores; B200 has no fast float64 tensor path)
        ma, mb, mc = (_memref(x, np.float64) for x in (a, b, c))
        sync, enqueue, scalar = (lib._mlir_ciface_mkl_gemm_float64_device,
                                 lib._mlir_ciface_nmb_gemm_float64_device_async, ctypes.c_double)
    else:
        ma, mb, mc = _memref(a), _memref(b), _memref(c)
        sync, enqueue, scalar = (lib._mlir_ciface_mkl_gemm_float32_device,
                                 lib._mlir_ciface_nmb_gemm_float32_device_async, ctypes.c_float)
    if blocking:
        sync(c.queue.handle, ctypes.byref(ma), ctypes.byref(mb), scalar(alpha), scalar(beta), ctypes.byref(mc))
        _rt.check()
        return c
    ev = enqueue(c.queue.handle, ctypes.byref(ma), ctypes.byref(mb), scalar(alpha), scalar(beta),
                 ctypes.byref(mc))
    if not ev:
        _rt.check()
        raise _rt.GpuRuntimeError("gemm launch failed")
    lib.gpuxDestroyEvent(c.queue.handle, ev)
    return c


TERM_NONE, TERM_NORMS, TERM_VECTOR = 0, 1, 2
FUNC_IDENTITY, FUNC_SQRT_MAX0 = 0, 1


def contract_rowcol(x, y, out, alpha=1.0, row=None, col=None, func=FUNC_IDENTITY):
    """out[i, j] = func(alpha * x[i] . y[j] + row[i] + col[j]) for float32
    x (M, K), y (N, K): the contraction with its surrounding elementwise chain
    as the epilogue.  `row` / `col`: None, the string "norms" (squared norms of
    the operand's rows, from the packing prepass) or a contiguous float32
    device vector."""
    def term(t, n):
        if t is None:
            return TERM_NONE, None
        if isinstance(t, str):
            if t != "norms":
                raise ValueError("a term is None, 'norms' or a device vector")
            return TERM_NORMS, None
        if t.dtype != np.float32 or t.size != n or not t.is_c_contiguous:
            raise ValueError("a row/column term must be a contiguous float32 vector of matching length")
        return TERM_VECTOR, t.ptr

    rk, rp = term(row, x.shape[0])
    ck, cp = term(col, y.shape[0])
    lib = _rt.load()
    mx, my, mo = _memref(x), _memref(y), _memref(out)
    ev = lib._mlir_ciface_nmb_contract_rowcol_float32_device(
        out.queue.handle, ctypes.byref(mx), ctypes.byref(my), ctypes.c_float(alpha), rk, rp, ck, cp, func,
        ctypes.byref(mo))
    if not ev:
        _rt.check()
        raise _rt.GpuRuntimeError("contraction launch failed")
    lib.gpuxDestroyEvent(out.queue.handle, ev)
    return out


def pairwise_distance(x, y, out=None):
    """out[i, j] = ||x[i] - y[j]||_2 for float32 x (M, K), y (N, K)."""
    if x.ndim != 2 or y.ndim != 2 or x.shape[1] != y.shape[1]:
        raise ValueError("pairwise_distance needs x (M, K) and y (N, K)")
    if out is None:
        out = empty((x.shape[0], y.shape[0]), np.float32, queue=x.queue)
    lib = _rt.load()
    mx, my, mo = _memref(x), _memref(y), _memref(out)
    ev = lib._mlir_ciface_nmb_pairwise_distance_float32_device(
        out.queue.handle, ctypes.byref(mx), ctypes.byref(my), ctypes.byref(mo))
    if not ev:
        _rt.check()
        raise _rt.GpuRuntimeError("pairwise distance launch failed")
    lib.gpuxDestroyEvent(out.queue.handle, ev)
    return out
