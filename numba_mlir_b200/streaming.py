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
    """`func(*inputs, *resident, *scalars, *outputs)` over host arrays, cut into
    chunks of rows (axis 0).

    `func` is an `njit` function (or any callable taking device arrays) whose
    output rows depend only on the same rows of its inputs: an elementwise
    chain, a row reduction, the distance rows of a block of points.  Inputs and
    outputs share their leading dimension; the trailing dimensions are free
    (`in_shapes` / `out_shapes`, one tuple per array, () for 1-D arrays).
    `resident` arrays are needed whole by every chunk (the second operand of a
    distance matrix): they are copied to the device once per call.  Host
    arrays should come from `pinned_empty` (pageable memory still works but the
    copies then serialise).  The device side holds `slots` chunk-sized buffers
    per array, whatever the total length."""

    def __init__(self, func, in_dtypes, out_dtypes, chunk=1 << 22, slots=3, queue=None,
                 in_shapes=None, out_shapes=None):
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
        self.in_shapes = [tuple(t) for t in (in_shapes or [()] * len(self.in_dtypes))]
        self.out_shapes = [tuple(t) for t in (out_shapes or [()] * len(self.out_dtypes))]
        self.d_in = [[empty((self.chunk,) + t, d, self.q) for d, t in zip(self.in_dtypes, self.in_shapes)]
                     for _ in range(self.slots)]
        self.d_out = [[empty((self.chunk,) + t, d, self.q) for d, t in zip(self.out_dtypes, self.out_shapes)]
                      for _ in range(self.slots)]
        self._resident = {}

    @staticmethod
    def _check(arrays, dtypes, shapes, what):
        if len(arrays) != len(dtypes):
            raise TypeError(f"expected {len(dtypes)} {what} arrays, got {len(arrays)}")
        n = None
        for a, d, t in zip(arrays, dtypes, shapes):
            if not isinstance(a, np.ndarray) or a.ndim != 1 + len(t) or not a.flags.c_contiguous:
                raise TypeError(f"{what} arrays must be contiguous NumPy arrays of {1 + len(t)} dimension(s)")
            if a.dtype != d or a.shape[1:] != t:
                raise TypeError(f"{what} array is {a.dtype}{a.shape[1:]} per row, the pipeline was built for {d}{t}")
            if n is not None and a.shape[0] != n:
                raise ValueError(f"{what} arrays differ in length")
            n = a.shape[0]
        return n

    def _resident_arrays(self, resident):
        """Device copies of the whole-array operands (buffers kept per shape)."""
        out = []
        for i, h in enumerate(resident):
            if not isinstance(h, np.ndarray) or not h.flags.c_contiguous:
                raise TypeError("resident arrays must be contiguous NumPy arrays")
            key = (i, h.shape, h.dtype.str)
            d = self._resident.get(key)
            if d is None:
                d = self._resident[key] = empty(h.shape, h.dtype, self.q)
            self.q.memcpy(d.ptr, h.ctypes.data, h.nbytes, _H2D)
            out.append(d)
        return out

    def run(self, inputs, scalars, outputs, resident=()):
        """Blocks until every output chunk is back in host memory."""
        n = self._check(inputs, self.in_dtypes, self.in_shapes, "input")
        n_out = self._check(outputs, self.out_dtypes, self.out_shapes, "output")
        if n is None or n_out != n:
            raise ValueError("inputs and outputs must have the same length")
        q, q_in, q_out = self.q, self.q_in, self.q_out
        S = self.slots
        cmp_done = [None] * S   # event on q: the slot's inputs have been read, outputs written
        out_done = [None] * S   # event on q_out: the slot's outputs are back on the host
        in_base = [a.ctypes.data for a in inputs]
        out_base = [a.ctypes.data for a in outputs]
        in_row = [int(np.prod(t, dtype=np.int64)) * d.itemsize for d, t in zip(self.in_dtypes, self.in_shapes)]
        out_row = [int(np.prod(t, dtype=np.int64)) * d.itemsize for d, t in zip(self.out_dtypes, self.out_shapes)]
        whole = self._resident_arrays(resident)
        try:
            for c, lo in enumerate(range(0, n, self.chunk)):
                m = min(self.chunk, n - lo)
                s = c % S
                # copy-in, once the kernel that last read this slot is done
                q_in.wait_events([cmp_done[s]])
                for d, base, row in zip(self.d_in[s], in_base, in_row):
                    q_in.memcpy(d.ptr, base + lo * row, m * row, _H2D)
                in_done = q_in.record()
                # compute, once the inputs are there and the slot's old outputs have left
                q.wait_events([in_done, out_done[s]])
                q_in.destroy_event(in_done)
                full = m == self.chunk
                ins = self.d_in[s] if full else [d[:m] for d in self.d_in[s]]
                outs = self.d_out[s] if full else [d[:m] for d in self.d_out[s]]
                self.func(*ins, *whole, *scalars, *outs)
                if cmp_done[s]:
                    q.destroy_event(cmp_done[s])
                cmp_done[s] = q.record()
                # copy-out
                q_out.wait_events([cmp_done[s]])
                for d, base, row in zip(self.d_out[s], out_base, out_row):
                    q_out.memcpy(base + lo * row, d.ptr, m * row, _D2H)
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


def auto_chunk(n, row_bytes=4):
    """About four chunks per call (enough for the copy-in of one to hide behind
    the copy-out of another), between 1 MB and 16 MB of the widest array, a
    multiple of 1024 rows where a row is small."""
    c = -(-int(n) // 4)
    lo, hi = max(1, (1 << 20) // row_bytes), max(1, (1 << 24) // row_bytes)
    c = max(lo, min(hi, c))
    unit = 1024 if row_bytes <= 1024 else 8
    return -(-c // unit) * unit


def map_host(func, inputs, outputs, scalars=(), chunk=None, queue=None, resident=()):
    """One call: `func(*inputs, *resident, *scalars, *outputs)` with host arrays
    in and out, copies overlapped with the kernels.  Inputs and outputs are cut
    along axis 0; `resident` arrays go to the device whole.  Pipelines (device
    buffers and queues) are kept per function, per-row layout and chunk size
    (`chunk=None` picks one from the length)."""
    lead = inputs[0] if inputs else outputs[0]
    if chunk is None:
        row_bytes = max(int(np.prod(a.shape[1:], dtype=np.int64)) * a.dtype.itemsize
                        for a in list(inputs) + list(outputs))
        chunk = auto_chunk(lead.shape[0], row_bytes)
    key = (id(func), tuple((a.dtype.str, a.shape[1:]) for a in inputs),
           tuple((a.dtype.str, a.shape[1:]) for a in outputs), int(chunk),
           None if queue is None else id(queue))
    entry = _pipelines.get(key)
    if entry is None:
        pipe = HostPipeline(func, [a.dtype for a in inputs], [a.dtype for a in outputs], chunk=chunk,
                            queue=queue, in_shapes=[a.shape[1:] for a in inputs],
                            out_shapes=[a.shape[1:] for a in outputs])
        entry = _pipelines[key] = (pipe, func)  # keeps func alive so that id(func) stays unique
    entry[0].run(inputs, scalars, outputs, resident)
