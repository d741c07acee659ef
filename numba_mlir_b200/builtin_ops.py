"""Host dispatch of the hand-written kernels linked into the runtime.

Each function does what the reference's generated host code does around one
outlined GPU kernel (numba_mlir/mlir_compiler/lib/pipelines/LowerToGpu.cpp:742-940,
mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:444-628): fetch the cached kernel
handle, build the GPUParamDesc array and call gpuxLaunchKernel.  Everything
goes through the C-ABI; nothing here computes on the host.
"""

import numpy as np

from .device_array import empty

_I64 = np.int64


def _aligned16(*arrays):
    return all(a.ptr % 16 == 0 for a in arrays)


def _check_contig(*arrays):
    for a in arrays:
        if not a.is_c_contiguous:
            raise ValueError("builtin kernels need C-contiguous arrays")


def bcast_add_f32(a, b, out=None):
    """out[i, j] = a[i, j] + b[0, j] for float32 a (M, N), b (1, N)."""
    _check_contig(a, b)
    if a.dtype != np.float32 or b.dtype != np.float32:
        raise TypeError("bcast_add_f32 needs float32 operands")
    if a.ndim != 2 or b.shape != (1, a.shape[1]):
        raise ValueError("bcast_add_f32 needs shapes (M, N) and (1, N)")
    q = a.queue
    if out is None:
        out = empty(a.shape, np.float32, queue=q)
    n, inner = a.size, a.shape[1]
    if n == 0:
        return out
    vec = _aligned16(a, b, out) and inner % 4 == 0
    kernel = q.builtin("nmb_bcast_add_f32" if vec else "nmb_bcast_add_f32_v1")
    tile = 256 * (4 if vec else 1) * 4
    q.launch(kernel, ((n + tile - 1) // tile,), (256,),
             [("ptr", a.ptr), ("ptr", b.ptr), ("ptr", out.ptr), _I64(n), _I64(inner)])
    return out


def black_scholes_f32(price, strike, t, rate, volatility, call, put):
    """Fused Black-Scholes chain over float32 arrays of equal length."""
    arrays = (price, strike, t, call, put)
    _check_contig(*arrays)
    if any(x.dtype != np.float32 for x in arrays):
        raise TypeError("black_scholes_f32 needs float32 arrays")
    n = price.size
    if any(x.size != n for x in arrays):
        raise ValueError("black_scholes_f32 needs arrays of equal length")
    if n == 0:
        return
    q = price.queue
    vec = _aligned16(*arrays)
    kernel = q.builtin("nmb_black_scholes_f32" if vec else "nmb_black_scholes_f32_v1")
    tile = 256 * (4 if vec else 1) * 2
    q.launch(kernel, ((n + tile - 1) // tile,), (256,),
             [("ptr", price.ptr), ("ptr", strike.ptr), ("ptr", t.ptr), np.float32(rate),
              np.float32(volatility), ("ptr", call.ptr), ("ptr", put.ptr), _I64(n)])
