"""Chunked host -> device -> host execution with the copies hidden.

The reference leaves host/device movement to `dpctl` (its tests copy whole
arrays before and after a call: numba_mlir/mlir/tests/test_gpu.py:52-87), so a
call on host data costs copy-in + kernel + copy-out one after the other.  For
an elementwise function with out-parameters the three can overlap: the input
is cut into chunks, and while chunk c is computed chunk c+1 travels to the
device on a second queue and chunk c-1 travels back on a third, so both
directions of the host link are busy at once.  Ordering between the queues is
expressed with the event lists of the gpux* C-ABI; nothing blocks on the host
until the end.
"""

import numpy as np

from . import runtime as _rt
from .device_array import empty

_H2D, _D2H = _rt.COPY_H2D, _rt.COPY_D2H


class HostPipeline:
    """`func(*inputs, *scalars, *outputs)` over 1-D host arrays, chunk by chunk.

    `func` is an `njit` function (or any callable taking device arrays) that
    reads its input arrays and writes its output arrays elementwise.  Host
    arrays should come from `pinned_empty` (pageable memory still works but the
    copies then serialise).  The device side holds `slots` chunk-sized buffers
    per array, whatever the total length."""

    def __init__(self, func, in_dtypes, out_dtypes, chunk=1 << 22, slots=3, queue=None):
        if chunk <= 0 or slots < 2:
            raise ValueError("chunk must be positive and slots >= 2")
        self.func = func
        self.chunk = int(chunk)
        self.slots = int(slots)
        self.q = queue if queue is not None else _rt.get_queue()
        name = f"cuda:{self.q.device}"
        self.q_in = _rt.Queue(name)    # own streams: the copies run beside the kernels
        self.q_out = _rt.Queue(name)
        self.in_dtypes = [np.dtype(d) for d in in_dtypes]
        self.out_dtypes = [np.dtype(d) for d in out_dtypes]
        self.d_in = [[empty(self.chunk, d, self.q) for d in self.in_dtypes] for _ in range(self.slots)]
        self.d_out = [[empty(self.chunk, d, self.q) for d in self.out_dtypes] for _ in range(self.slots)]

    @staticmethod
    def _check(arrays, dtypes, what):
        if len(arrays) != len(dtypes):
            raise TypeError(f"expected {len(dtypes)} {what} arrays, got {len(arrays)}")
        n = None
        for a, d in zip(arrays, dtypes):
            if not isinstance(a, np.ndarray) or a.ndim != 1 or not a.flags.c_contiguous:
                raise TypeError(f"{what} arrays must be contiguous 1-D NumPy arrays")
            if a.dtype != d:
                raise TypeError(f"{what} array has dtype {a.dtype}, pipeline was built for {d}")
            if n is not None and a.shape[0] != n:
                raise ValueError(f"{what} arrays differ in length")
            n = a.shape[0]
        return n

    def run(self, inputs, scalars, outputs):
        """Blocks until every output chunk is back in host memory."""
        n = self._check(inputs, self.in_dtypes, "input")
        n_out = self._check(outputs, self.out_dtypes, "output")
        if n is None or n_out != n:
            raise ValueError("inputs and outputs must have the same length")
        q, q_in, q_out = self.q, self.q_in, self.q_out
        S = self.slots
        cmp_done = [None] * S   # event on q: the slot's inputs have been read, outputs written
        out_done = [None] * S   # event on q_out: the slot's outputs are back on the host
        in_base = [a.ctypes.data for a in inputs]
        out_base = [a.ctypes.data for a in outputs]
        try:
            for c, lo in enumerate(range(0, n, self.chunk)):
                m = min(self.chunk, n - lo)
                s = c % S
                # copy-in, once the kernel that last read this slot is done
                q_in.wait_events([cmp_done[s]])
                for d, base, dt in zip(self.d_in[s], in_base, self.in_dtypes):
                    q_in.memcpy(d.ptr, base + lo * dt.itemsize, m * dt.itemsize, _H2D)
                in_done = q_in.record()
                # compute, once the inputs are there and the slot's old outputs have left
                q.wait_events([in_done, out_done[s]])
                q_in.destroy_event(in_done)
                full = m == self.chunk
                ins = self.d_in[s] if full else [d[:m] for d in self.d_in[s]]
                outs = self.d_out[s] if full else [d[:m] for d in self.d_out[s]]
                self.func(*ins, *scalars, *outs)
                if cmp_done[s]:
                    q.destroy_event(cmp_done[s])
                cmp_done[s] = q.record()
                # copy-out
                q_out.wait_events([cmp_done[s]])
                for d, base, dt in zip(self.d_out[s], out_base, self.out_dtypes):
                    q_out.memcpy(base + lo * dt.itemsize, d.ptr, m * dt.itemsize, _D2H)
                if out_done[s]:
                    q_out.destroy_event(out_done[s])
                out_done[s] = q_out.record()
            q_out.synchronize()
            q.synchronize()
        finally:
            for ev in cmp_done:
                if ev:
                    q.destroy_event(ev)
            for ev in out_done:
                if ev:
                    q_out.destroy_event(ev)
        q.check_status()


_pipelines = {}


def auto_chunk(n):
    """About four chunks per call (enough for the copy-in of one to hide behind
    the copy-out of another), between 2^18 and 2^22 elements, a multiple of 1024."""
    c = -(-int(n) // 4)
    c = max(1 << 18, min(1 << 22, c))
    return -(-c // 1024) * 1024


def map_host(func, inputs, outputs, scalars=(), chunk=None, queue=None):
    """One call: `func(*inputs, *scalars, *outputs)` with host arrays in and
    out, copies overlapped with the kernels.  Pipelines (device buffers and
    queues) are kept per function, dtype list and chunk size (`chunk=None`
    picks one from the length)."""
    if chunk is None:
        chunk = auto_chunk(inputs[0].shape[0] if inputs else outputs[0].shape[0])
    key = (id(func), tuple(a.dtype.str for a in inputs), tuple(a.dtype.str for a in outputs), int(chunk),
           None if queue is None else id(queue))
    entry = _pipelines.get(key)
    if entry is None:
        pipe = HostPipeline(func, [a.dtype for a in inputs], [a.dtype for a in outputs], chunk=chunk,
                            queue=queue)
        entry = _pipelines[key] = (pipe, func)  # keeps func alive so that id(func) stays unique
    entry[0].run(inputs, scalars, outputs)
