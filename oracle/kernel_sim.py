"""CPU simulator of the `@kernel` programming model (test infrastructure only).

Restates numba_mlir/numba_mlir/mlir/kernel_sim_impl.py:193-234 and
kernel_sim.py:24-117: work-groups are visited in row-major order, the
work-items of a group likewise; the last group of a dimension is clipped to the
global size (kernel_sim_impl.py:203-209); the API names found in the kernel's
globals and closure are swapped for simulator versions for the duration of the
call.  Atomics are plain read-modify-write that return the NEW value
(kernel_sim.py:24-35); mem_fence does nothing; local.array is shared by the
work-items of a group and zero filled, private.array zero filled per call
(kernel_sim_impl.py:155-168).  Barriers and group reductions need coroutines in
the reference (greenlet); here they are supported for the common case where
the kernel body is run in lock step by generator-free code: not at all --
kernels that call them are rejected.
"""

from itertools import product

import numpy as np

from numba_mlir_b200 import kernel_impl as K

_state = None


class _State:
    def __init__(self, global_size, local_size):
        self.global_size = global_size
        self.local_size = local_size
        self.indices = [0] * len(global_size)
        self.local_arrays = []
        self.cursor = 0
        self.first_item = True


def _get_global_id(i):
    return _state.indices[i]


def _get_local_id(i):
    return _state.indices[i] % _state.local_size[i]


def _get_group_id(i):
    return _state.indices[i] // _state.local_size[i]


def _get_global_size(i):
    return _state.global_size[i]


def _get_local_size(i):
    return _state.local_size[i]


def _atomic_add(arr, ind, val):
    new = arr[ind] + val
    arr[ind] = new
    return arr[ind]


def _atomic_sub(arr, ind, val):
    new = arr[ind] - val
    arr[ind] = new
    return arr[ind]


class _Atomic:
    add = staticmethod(_atomic_add)
    sub = staticmethod(_atomic_sub)


def _local_array(shape, dtype):
    st = _state
    if st.first_item:
        arr = np.zeros(shape, dtype)
        st.local_arrays.append(arr)
    else:
        arr = st.local_arrays[st.cursor]
    st.cursor += 1
    return arr


def _private_array(shape, dtype):
    return np.zeros(shape, dtype)


class _Local:
    array = staticmethod(_local_array)


class _Private:
    array = staticmethod(_private_array)


def _unsupported(*_a, **_k):
    raise NotImplementedError("barrier/group operations are not simulated")


_REPLACE = [
    (K.get_global_id, _get_global_id), (K.get_local_id, _get_local_id),
    (K.get_group_id, _get_group_id), (K.get_global_size, _get_global_size),
    (K.get_local_size, _get_local_size), (K.atomic, _Atomic), (K.atomic_add, _atomic_add),
    (K.atomic_sub, _atomic_sub), (K.local, _Local), (K.private, _Private),
    (K.local_array, _local_array), (K.private_array, _private_array),
    (K.barrier, _unsupported), (K.group, _unsupported), (K.mem_fence, lambda *a: None),
]


def _swap(obj):
    for old, new in _REPLACE:
        if obj is old:
            return new
    return obj


class SimKernel:
    def __init__(self, func):
        self.py_func = func
        self.global_size = ()
        self.local_size = ()

    def __getitem__(self, args):
        if not isinstance(args, tuple):
            args = (args,)
        k = SimKernel(self.py_func)
        k.global_size = K._process_dims(args[0])
        ls = K._process_dims(args[1]) if len(args) > 1 else ()
        if ls and len(ls) < len(k.global_size):
            ls = tuple(ls) + (1,) * (len(k.global_size) - len(ls))
        k.local_size = ls
        return k

    def __call__(self, *args):
        global _state
        func = self.py_func
        gs = self.global_size
        ls = self.local_size or (1,) * len(gs)
        saved_globals = {n: v for n, v in func.__globals__.items() if _swap(v) is not v}
        for n, v in saved_globals.items():
            func.__globals__[n] = _swap(v)
        saved_cells = []
        for cell in func.__closure__ or ():
            saved_cells.append(cell.cell_contents)
            cell.cell_contents = _swap(cell.cell_contents)
        _state = _State(gs, ls)
        try:
            groups = tuple((g + l - 1) // l for g, l in zip(gs, ls))
            for gid in product(*(range(g) for g in groups)):
                offset = tuple(g * l for g, l in zip(gid, ls))
                size = tuple(min(g - o, l) for o, g, l in zip(offset, gs, ls))
                _state.local_arrays = []
                _state.first_item = True
                for idx in product(*(range(o, o + s) for o, s in zip(offset, size))):
                    _state.indices[:] = idx
                    _state.cursor = 0
                    func(*args)
                    _state.first_item = False
        finally:
            _state = None
            func.__globals__.update(saved_globals)
            for cell, v in zip(func.__closure__ or (), saved_cells):
                cell.cell_contents = v


def kernel_sim(func):
    return SimKernel(func)
