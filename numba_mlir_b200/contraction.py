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


def _memref(a):
    if a.dtype != np.float32 or a.ndim != 2:
        raise TypeError("the tensor-core contraction takes 2-D float32 device arrays")
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


def gemm(a, b, c, alpha=1.0, beta=0.0):
    """c = alpha * a @ b + beta * c (blocking, like the reference's call)."""
    lib = _rt.load()
    ma, mb, mc = _memref(a), _memref(b), _memref(c)
    lib._mlir_ciface_mkl_gemm_float32_device(c.queue.handle, ctypes.byref(ma), ctypes.byref(mb),
                                             ctypes.c_float(alpha), ctypes.c_float(beta),
                                             ctypes.byref(mc))
    _rt.check()
    return c


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
