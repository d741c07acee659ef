"""Device arrays for the CUDA offload path.

Replaces the role `dpctl.tensor.usm_ndarray` plays for the reference
(numba_mlir/numba_mlir/mlir/dpctl_interop.py:77-262): the array type whose
presence in a call's arguments selects offload.  Memory comes from gpuxAlloc
and is released with gpuxDeAlloc when the last view dies, the contract the
reference implements with a meminfo destructor
(mlir/lib/Conversion/GpuRuntimeToLlvm.cpp:717-720).  Interop is through
`__cuda_array_interface__` version 3 (strides in BYTES, unlike the element
strides of `__sycl_usm_array_interface__`, python_runtime/lib/Boxing.cpp:122-128).
"""

import ctypes

import numpy as np

from . import runtime as _rt


class _Buffer:
    """Owner of one gpuxAlloc allocation."""

    __slots__ = ("queue", "ptr", "nbytes", "kind", "__weakref__")

    def __init__(self, queue, nbytes, kind):
        self.queue = queue
        self.nbytes = int(nbytes)
        self.kind = kind
        self.ptr = queue.alloc(max(self.nbytes, 1), kind)

    def __del__(self):
        try:
            if self.ptr:
                self.queue.free(self.ptr)
                self.ptr = None
        except Exception:
            pass


class _Foreign:
    """Keeps a foreign exporter of __cuda_array_interface__ alive."""

    __slots__ = ("obj", "ptr", "nbytes", "queue", "kind")

    def __init__(self, obj, ptr, nbytes, queue):
        self.obj = obj
        self.ptr = ptr
        self.nbytes = nbytes
        self.queue = queue
        self.kind = _rt.ALLOC_DEVICE


def _c_strides(shape, itemsize):
    strides = []
    acc = itemsize
    for dim in reversed(shape):
        strides.append(acc)
        acc *= max(int(dim), 1)
    return tuple(reversed(strides))


class DeviceArray:
    """N-dimensional strided view of device (or managed) memory."""

    def __init__(self, buffer, shape, dtype, strides=None, offset=0):
        self._buf = buffer
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.strides = tuple(strides) if strides is not None else _c_strides(self.shape, self.dtype.itemsize)
        self._offset = int(offset)
        self._addr = (buffer.ptr or 0) + self._offset  # device address, read by the native launch path
        self._contig = None if strides is not None else True
        self._call_sig = None
        self._trace_sig = None
        self._extent = None

    # -- basic properties ------------------------------------------------------
    @property
    def queue(self):
        return self._buf.queue

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def itemsize(self):
        return self.dtype.itemsize

    @property
    def nbytes(self):
        return self.size * self.dtype.itemsize

    @property
    def ptr(self):
        return self._buf.ptr + self._offset

    @property
    def usm_type(self):
        """'device' or 'shared', the reference's placement attribute
        (dpctl_interop.py:210-234)."""
        return "shared" if self._buf.kind == _rt.ALLOC_SHARED else "device"

    @property
    def trace_sig(self):
        """Everything a recorded plan is specialised on (a cache key)."""
        sig = self._trace_sig
        if sig is None:
            sig = self._trace_sig = ("arr", self.dtype.name, self.shape, self.strides, self.ptr % 16 == 0,
                                     getattr(self.queue, "device", None))
        return sig

    @property
    def extent(self):
        """Byte range (lo, hi) of device addresses the view can touch."""
        ext = self._extent
        if ext is None:
            lo = hi = self.ptr
            if self.size:
                for n, st in zip(self.shape, self.strides):
                    if st >= 0:
                        hi += (n - 1) * st
                    else:
                        lo += (n - 1) * st
                hi += self.dtype.itemsize
            ext = self._extent = (lo, hi)
        return ext

    @property
    def call_sig(self):
        """What generated code depends on: dtype, rank, contiguity (a cache key)."""
        sig = self._call_sig
        if sig is None:
            sig = self._call_sig = ("arr", self.dtype.name, len(self.shape), self.is_c_contiguous)
        return sig

    @property
    def is_c_contiguous(self):
        c = self._contig
        if c is None:
            c = self._contig = self._compute_contiguity()
        return c

    def _compute_contiguity(self):
        return self.size <= 1 or self.strides == _c_strides(self.shape, self.dtype.itemsize) or all(
            st == cst for s, st, cst in zip(self.shape, self.strides, _c_strides(self.shape, self.dtype.itemsize)) if s != 1
        )

    @property
    def __cuda_array_interface__(self):
        return {
            "shape": self.shape,
            "typestr": self.dtype.str,
            "data": (self.ptr if self.size else 0, False),
            "version": 3,
            "strides": None if self.is_c_contiguous else self.strides,
            "stream": int(self.queue.stream) or None,
        }

    def __len__(self):
        if not self.shape:
            raise TypeError("len() of a 0-d array")
        return self.shape[0]

    def __repr__(self):
        return f"DeviceArray(shape={self.shape}, dtype={self.dtype}, device={self.queue.device})"

    # -- views -------------------------------------------------------------------
    @property
    def T(self):
        return DeviceArray(self._buf, self.shape[::-1], self.dtype, self.strides[::-1], self._offset)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if not self.is_c_contiguous:
            raise ValueError("reshape needs a C-contiguous array")
        shape = list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.size // max(known, 1)
        n = 1
        for s in shape:
            n *= s
        if n != self.size:
            raise ValueError("cannot reshape array of size %d into %s" % (self.size, tuple(shape)))
        return DeviceArray(self._buf, shape, self.dtype, None, self._offset)

    def __getitem__(self, idx):
        """Basic indexing (ints, slices, None, Ellipsis) as views."""
        if not isinstance(idx, tuple):
            idx = (idx,)
        if any(i is Ellipsis for i in idx):
            pos = idx.index(Ellipsis)
            fill = self.ndim - sum(1 for i in idx if i is not None and i is not Ellipsis)
            idx = idx[:pos] + (slice(None),) * fill + idx[pos + 1 :]
        shape, strides, offset = [], [], self._offset
        dim = 0
        for i in idx:
            if i is None:
                shape.append(1)
                strides.append(0)
                continue
            if dim >= self.ndim:
                raise IndexError("too many indices")
            n, st = self.shape[dim], self.strides[dim]
            if isinstance(i, slice):
                start, stop, step = i.indices(n)
                length = max(0, (stop - start + (step - (1 if step > 0 else -1))) // step)
                offset += start * st
                shape.append(length)
                strides.append(st * step)
            else:
                i = int(i)
                if i < 0:
                    i += n
                if not 0 <= i < n:
                    raise IndexError("index out of range")
                offset += i * st
            dim += 1
        shape.extend(self.shape[dim:])
        strides.extend(self.strides[dim:])
        return DeviceArray(self._buf, shape, self.dtype, strides, offset)

    def __setitem__(self, idx, value):
        """`arr[:] = value` style assignment is handled by the expression
        front-end; see numba_mlir_b200.lazy."""
        from . import lazy

        lazy.assign(self[idx] if idx != slice(None) else self, value)

    # -- data movement -------------------------------------------------------------
    def copy_from_host(self, host, wait=True):
        host = np.ascontiguousarray(host, dtype=self.dtype)
        if host.shape != self.shape:
            raise ValueError(f"shape mismatch {host.shape} vs {self.shape}")
        if not self.is_c_contiguous:
            raise ValueError("copy_from_host needs a C-contiguous destination")
        self.queue.memcpy(self.ptr, host.ctypes.data, self.nbytes, _rt.COPY_H2D, wait=wait)
        return self

    def copy_to_host(self, out=None, wait=True):
        src = self if self.is_c_contiguous else self.copy()
        if out is None:
            out = np.empty(self.shape, self.dtype)
        if out.shape != self.shape or out.dtype != self.dtype or not out.flags.c_contiguous:
            raise ValueError("copy_to_host needs a C-contiguous host array of the same shape/dtype")
        src.queue.memcpy(out.ctypes.data, src.ptr, src.nbytes, _rt.COPY_D2H, wait=wait)
        return out

    def copy(self):
        """C-contiguous device copy."""
        out = empty(self.shape, self.dtype, queue=self.queue)
        if self.is_c_contiguous:
            self.queue.memcpy(out.ptr, self.ptr, self.nbytes, _rt.COPY_D2D)
        else:
            from . import lazy

            lazy.assign(out, self)
        return out

    def __array__(self, dtype=None, copy=None):
        host = self.copy_to_host()
        return host.astype(dtype) if dtype is not None else host

    def item(self):
        return self.copy_to_host().item()


def empty(shape, dtype=np.float32, queue=None, usm_type="device"):
    if isinstance(shape, (int, np.integer)):
        shape = (int(shape),)
    queue = queue or _rt.get_queue()
    dtype = np.dtype(dtype)
    n = 1
    for s in shape:
        n *= int(s)
    kind = {"device": _rt.ALLOC_DEVICE, "shared": _rt.ALLOC_SHARED}[usm_type]
    return DeviceArray(_Buffer(queue, n * dtype.itemsize, kind), shape, dtype)


def zeros(shape, dtype=np.float32, queue=None, usm_type="device"):
    arr = empty(shape, dtype, queue, usm_type)
    if arr.nbytes:
        arr.queue.memset(arr.ptr, 0, arr.nbytes)
    return arr


def from_host(host, queue=None, usm_type="device", wait=True):
    """Host -> device copy (what dpctl's `usm_ndarray.usm_data.copy_from_host`
    does for the reference's tests, mlir/tests/test_gpu.py:52-75)."""
    host = np.ascontiguousarray(host)
    arr = empty(host.shape, host.dtype, queue, usm_type)
    if arr.nbytes:
        arr.queue.memcpy(arr.ptr, host.ctypes.data, arr.nbytes, _rt.COPY_H2D, wait=wait)
    return arr


def as_device_array(obj, queue=None):
    """Zero-copy view of any exporter of __cuda_array_interface__ (torch, cupy,
    numba.cuda ...).  When the exporter names the stream its data is ready on
    (version 3 of the interface), the queue is ordered after that stream."""
    if isinstance(obj, DeviceArray):
        return obj
    iface = obj.__cuda_array_interface__
    queue = queue or _rt.get_queue()
    stream = iface.get("stream")
    if stream is not None and int(stream) != int(queue.stream or 0):
        queue.wait_stream(stream)
    dtype = np.dtype(iface["typestr"])
    shape = tuple(iface["shape"])
    ptr = iface["data"][0] or 0
    n = 1
    for s in shape:
        n *= s
    return DeviceArray(_Foreign(obj, ptr, n * dtype.itemsize, queue), shape, dtype, iface.get("strides"))


class _PinnedOwner:
    def __init__(self, queue, nbytes):
        self.queue = queue
        self.ptr = queue.alloc(max(int(nbytes), 1), _rt.ALLOC_HOST)

    def __del__(self):
        try:
            self.queue.free(self.ptr)
        except Exception:
            pass


def pinned_empty(shape, dtype=np.float32, queue=None):
    """Page-locked host array (gpuxAlloc with GpuAllocType::Host) for fast
    asynchronous transfers."""
    queue = queue or _rt.get_queue()
    dtype = np.dtype(dtype)
    if isinstance(shape, (int, np.integer)):
        shape = (int(shape),)
    n = 1
    for s in shape:
        n *= int(s)
    owner = _PinnedOwner(queue, n * dtype.itemsize)
    raw = (ctypes.c_char * max(n * dtype.itemsize, 1)).from_address(owner.ptr)
    # The ctypes view is the buffer object every NumPy view keeps alive; it
    # carries the allocation's owner.
    raw._owner = owner
    return np.frombuffer(raw, dtype=dtype, count=n).reshape(shape)


def is_device_array(obj):
    return isinstance(obj, DeviceArray)
