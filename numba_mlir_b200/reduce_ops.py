"""Host dispatch of the reduction kernels (sum/prod/min/max/argmin/argmax).

Full and row reductions of sum/prod/min/max run on the direct-load kernels
(csrc/kernels/reduce_direct.cu), as do argmin/argmax along rows when there are
enough rows; column reductions and argmin/argmax of a few long rows run on the
TMA-staged ring (reduce_ws.cuh), which measured faster there (float32
(16384, 4096) min(axis=0): 47 us against 61-65 us for direct-load column
kernels), anything unaligned or strided on the generic
kernels.  Result dtypes follow the reference's _array_reduce
(numba_mlir/numba_mlir/mlir/numpy/funcs.py:163-214): sum and prod of an integer
array are int64, of a float array the array's dtype; min/max keep the dtype;
argmin/argmax are int64 (NumPy's intp).  Everything runs on the device through
gpuxLaunchKernel; there is no host-side combination step (the reference reduces
work-group partials in a host loop, mlir/lib/Conversion/GpuToGpuRuntime.cpp:2232-2273).
"""

import numpy as np

from .device_array import empty

_TY = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64",
       np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}
OPS = ("sum", "prod", "min", "max", "argmin", "argmax")
_CTAS_PER_SM = 3  # three 65 KB CTAs fit one SM
_TILE_BYTES = 16384
_COL_FANIN = 16  # rows merged per ticket of the column merge tree (at most 32)
_I64 = np.int64


def out_dtype(op, dtype):
    dtype = np.dtype(dtype)
    if op in ("argmin", "argmax"):
        return np.dtype(np.int64)
    if op in ("sum", "prod") and dtype.kind in "iu":
        return np.dtype(np.int64)
    return dtype


def _acc_bytes(op, dtype):
    if op in ("argmin", "argmax"):
        return 16
    return out_dtype(op, dtype).itemsize


def _kernel_type(dtype):
    try:
        return _TY[np.dtype(dtype)]
    except KeyError:
        raise TypeError(f"reductions support float32/float64/int32/int64, not {dtype}") from None


_NO_PEERS = [("ptr", 0), np.int32(0), np.int32(0)]
_EXCHANGED_OPS = ("sum", "prod", "min", "max")


def _peer_params(q, op, nbytes):
    """Kernel arguments of the exchange between the GPUs' shards that ends a
    reduction over the sharded axis (numba_mlir_b200.sharding.across), or the
    arguments that switch it off.  Returns (params, exchange still owed)."""
    ex = getattr(q, "shard_exchange", None)
    if ex is None:
        return _NO_PEERS, None
    group = ex.group
    if op in _EXCHANGED_OPS and group is not None and 0 < nbytes <= ex.slot_bytes:
        return [("ptr", group.table.ptr), np.int32(group.rank), np.int32(group.world)], None
    return _NO_PEERS, ex


def reduce(a, op, axis=None, out=None):
    """Reduces DeviceArray `a` with `op` over `axis` (None = all elements).

    Returns a DeviceArray; a 0-d one for axis=None.  Inside
    `numba_mlir_b200.sharding.across(...)` the array is one GPU's shard of rows:
    a full reduction or a reduction over axis 0 ends with the all-reduce of the
    GPUs' results, inside the same kernel when the result fits a mailbox slot."""
    if op not in OPS:
        raise ValueError(f"unknown reduction {op}")
    ty = _kernel_type(a.dtype)
    odt = out_dtype(op, a.dtype)
    q = a.queue
    ex = getattr(q, "shard_exchange", None)
    if ex is not None:
        if axis is not None and int(axis) % max(a.ndim, 1) != 0:
            raise ValueError("inside sharding.across only reductions over axis 0 (the sharded axis) or over "
                             "all elements are exchanged; reduce along other axes outside it")
        if op not in _EXCHANGED_OPS:
            raise ValueError(f"{op} over a sharded axis is not supported (the shards' offsets are needed)")
    if axis is None:
        if a.size == 0:
            raise ValueError("zero-size array to reduction operation")
        flat = a if a.is_c_contiguous else a.copy()
        if out is None:
            out = empty((), odt, queue=q)
        _launch_all(q, flat, out, op, ty)
        return out
    axis = int(axis)
    if axis < 0:
        axis += a.ndim
    if not 0 <= axis < a.ndim:
        raise ValueError("axis out of range")
    oshape = a.shape[:axis] + a.shape[axis + 1:]
    if a.shape[axis] == 0:
        raise ValueError("zero-size reduction axis")
    if out is None:
        out = empty(oshape, odt, queue=q)
    if out.size == 0:
        return out
    outer = int(np.prod(a.shape[:axis], dtype=np.int64))
    K = a.shape[axis]
    inner = int(np.prod(a.shape[axis + 1:], dtype=np.int64))
    it = a.dtype.itemsize
    vec = 16 // it
    aligned = a.is_c_contiguous and a.ptr % 16 == 0
    if aligned and inner == 1 and K % vec == 0:
        _launch_rows(q, a, out, op, ty, outer, K)
    elif aligned and outer == 1 and inner % vec == 0:
        _launch_cols(q, a, out, op, ty, K, inner)
    else:
        _launch_generic(q, a, out, op, ty, axis, outer, K, inner)
    return out


_DIRECT_OPS = ("sum", "prod", "min", "max")
# the direct kernels hand out rows and tiles round robin and are compiled for a
# fixed number of resident blocks per multiprocessor (float32 rows: eight;
# other rows, full and argmin/argmax: six):
# one block per residency slot keeps the shares equal
_DIRECT_ROWS_BLOCKS_PER_SM = 8
_DIRECT_BLOCKS_PER_SM = 6


def _launch_rows(q, a, out, op, ty, rows, cols):
    if op in _DIRECT_OPS:
        # plain 128-bit loads, one warp per row (the whole block for few long
        # rows): measured faster than the TMA ring for these reductions
        resident = _DIRECT_ROWS_BLOCKS_PER_SM if ty == "f32" else _DIRECT_BLOCKS_PER_SM
        block_row = cols >= 8192 and rows < q.sm_count * resident
        k = q.builtin(f"nmb_reduce_rows_direct_{'blockrow_' if block_row else ''}{op}_{ty}")
        units = rows if block_row else (rows + 7) // 8
        q.launch(k, (max(1, min(units, q.sm_count * resident)),), (256,),
                 [("ptr", a.ptr), ("ptr", out.ptr), _I64(rows), _I64(cols)])
        return
    if rows >= q.sm_count * 2:
        # argmin / argmax: one warp per row over plain loads (few long rows stay
        # on the ring kernel below, which spreads a row over a whole block)
        k = q.builtin(f"nmb_reduce_rows_direct_{op}_{ty}")
        q.launch(k, (max(1, min((rows + 7) // 8, q.sm_count * _DIRECT_BLOCKS_PER_SM)),), (256,),
                 [("ptr", a.ptr), ("ptr", out.ptr), _I64(rows), _I64(cols)])
        return
    k = q.builtin(f"nmb_reduce_rows_{op}_{ty}")
    it = a.dtype.itemsize
    if cols * it > 2048:
        units = (rows + 7) // 8              # blocks of 8 rows
    else:
        units = (rows + (_TILE_BYTES // (cols * it)) - 1) // (_TILE_BYTES // (cols * it))
    grid = max(1, min(units, q.sm_count * _CTAS_PER_SM))
    q.launch(k, (grid,), (256,),
             [("ptr", a.ptr), ("ptr", out.ptr), _I64(rows), _I64(cols), ("ptr", q.status_ptr)])


def _launch_cols(q, a, out, op, ty, rows, cols):
    peers, owed = _peer_params(q, op, out.nbytes)
    k = q.builtin(f"nmb_reduce_cols_{op}_{ty}")
    it = a.dtype.itemsize
    # column slabs of 2 KB: a stage of the ring is then 8 row segments, one bulk
    # copy for each of the block's 8 warps, and the per-CTA partial rows stay
    # short (for (16384, 4096) float32, sum: 50.3 us against 56.2 us with 4 KB
    # slabs and three blocks per multiprocessor)
    tile_cols = min(cols, 2048 // it)
    col_tiles = (cols + tile_cols - 1) // tile_cols
    rows_per_stage = _TILE_BYTES // (tile_cols * it)
    # two blocks per multiprocessor instead of the three that fit: min measured
    # 48.5 us against 51.4 us (min and max meet in `out` through one atomic per
    # column and row block: a third fewer atomics, the same bytes in flight),
    # the merge tree of the other reductions has a third fewer rows
    per_sm = 2
    row_blocks = max(1, min((q.sm_count * per_sm + col_tiles - 1) // col_tiles,
                            (rows + rows_per_stage - 1) // rows_per_stage, 65535))
    # merge tree: level buffers and tickets for the fan-in handed to the kernel
    level_rows, tickets, n = 0, 0, row_blocks
    while n > 1:
        level_rows += n
        n = (n + _COL_FANIN - 1) // _COL_FANIN
        tickets += n
    if col_tiles * tickets * 4 > q.COUNTER_BYTES - 4:  # the last word is the exchange's ticket
        raise ValueError("too many column tiles for the counter region")
    counters, partials = q.scratch(max(level_rows, 1) * cols * _acc_bytes(op, a.dtype))
    q.launch(k, (col_tiles, row_blocks), (256,),
             [("ptr", a.ptr), ("ptr", out.ptr), ("ptr", partials), ("ptr", counters),
              _I64(rows), _I64(cols), _I64(tile_cols), _I64(_COL_FANIN), ("ptr", q.status_ptr)] + peers)
    if owed is not None:
        owed.allreduce(out, op)


def _launch_all(q, a, out, op, ty):
    n = a.size
    if a.ptr % 16 != 0:
        _launch_generic(q, a.reshape(n), out, op, ty, 0, 1, n, 1)
        return
    peers, owed = _peer_params(q, op, out.nbytes)
    if op in _DIRECT_OPS:
        tile = 256 * (16 // a.dtype.itemsize) * 4  # elements a block takes per step
        grid = max(1, min(q.sm_count * _DIRECT_BLOCKS_PER_SM, (n + tile - 1) // tile))
        counters, partials = q.scratch(grid * 8)
        q.launch(q.builtin(f"nmb_reduce_all_direct_{op}_{ty}"), (grid,), (256,),
                 [("ptr", a.ptr), ("ptr", out.ptr), ("ptr", partials), ("ptr", counters), _I64(n),
                  ("ptr", q.status_ptr)] + peers)
        if owed is not None:
            owed.allreduce(out, op)
        return
    k = q.builtin(f"nmb_reduce_all_{op}_{ty}")
    tile = _TILE_BYTES // a.dtype.itemsize
    grid = max(1, min(q.sm_count * _CTAS_PER_SM, (n + tile - 1) // tile))
    span = (n + grid - 1) // grid
    span = (span + tile - 1) // tile * tile
    counters, partials = q.scratch(grid * 16)
    q.launch(k, (grid,), (256,),
             [("ptr", a.ptr), ("ptr", out.ptr), ("ptr", partials), ("ptr", counters),
              _I64(n), _I64(span), ("ptr", q.status_ptr)] + peers)
    if owed is not None:
        owed.allreduce(out, op)


def _launch_generic(q, a, out, op, ty, axis, outer, K, inner):
    """Any strides / alignment.  The (outer, K, inner) decomposition needs the
    outer and inner index groups to be addressable with one stride each, which
    holds for 1-D/2-D arrays and C-contiguous N-D arrays; other layouts are
    copied to C order first."""
    it = a.dtype.itemsize
    if a.ndim <= 2 or a.is_c_contiguous:
        src = a
    else:
        src = a.copy()
    st = [s // it for s in src.strides]
    sk = st[axis]
    if src.ndim == 1:
        so, si = 0, 0
    elif src.ndim == 2:
        so, si = (st[0], 0) if axis == 1 else (0, st[1])
    else:
        so = st[axis - 1] if axis > 0 else 0
        si = 1
    k = q.builtin(f"nmb_reduce_generic_{op}_{ty}")
    nout = outer * inner
    mode = 0 if (abs(sk) == 1 and K >= 64) or inner == 1 else 1
    threads = nout * 32 if mode == 0 else nout
    q.launch(k, ((threads + 255) // 256,), (256,),
             [("ptr", src.ptr), ("ptr", out.ptr), _I64(outer), _I64(K), _I64(inner),
              _I64(so), _I64(sk), _I64(si), np.int32(mode)])
    ex = getattr(q, "shard_exchange", None)
    if ex is not None:
        ex.allreduce(out, op)
