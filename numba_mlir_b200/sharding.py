"""Row sharding across the GPUs of one box and the few exchanges it needs.

The reference has no multi-device code (one queue per device,
mlir/lib/Conversion/GpuToGpuRuntime.cpp:169-197).  The benchmark workloads
shard along axis 0 -- one process per GPU, every process runs the same
single-GPU kernels on its rows -- and only three results span shards: a full
sum, a column-wise min, and the per-cluster sums/counts of a k-means
iteration.  Those partials are all-reduced with torch.distributed (NCCL over
NVLink on GPUs, gloo in the CPU tests); they are at most a few KB, so the
exchange is latency bound and no custom kernel is warranted.
"""

import numpy as np


def row_range(n_rows, world, rank):
    """Contiguous balanced split of `n_rows` rows: rows [begin, end) of `rank`."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    begin = n_rows * rank // world
    end = n_rows * (rank + 1) // world
    return begin, end


def shard_rows(array, world, rank):
    """View of this rank's rows of a host or device array."""
    begin, end = row_range(array.shape[0], world, rank)
    return array[begin:end]


_REDUCE_OPS = ("sum", "min", "max")


def allreduce(partial, op="sum", dist=None):
    """In-place all-reduce of a partial result (DeviceArray or NumPy array).

    `dist` is an initialised torch.distributed module (or None / world 1: the
    partial already is the result).  A DeviceArray is shared with torch through
    __cuda_array_interface__ and the collective is enqueued on the array's own
    queue (stream)."""
    if op not in _REDUCE_OPS:
        raise ValueError(f"unsupported reduction {op}")
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return partial
    import torch

    rop = {"sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}[op]
    if isinstance(partial, np.ndarray):
        t = torch.from_numpy(partial)
        dist.all_reduce(t, op=rop)
        return partial
    # Run the collective in stream order behind the kernels that produced the
    # partial: torch adopts the queue's stream for the duration of the call, so
    # no host synchronisation is needed on either side.
    stream = _external_stream(partial.queue)
    with torch.cuda.stream(stream):
        dist.all_reduce(_torch_view(partial), op=rop)
    return partial


_streams = {}
_views = {}


def _torch_view(array):
    """torch tensor over the array's memory; kept (with the array) per buffer so
    that a step repeated every iteration does not rebuild it."""
    import torch

    key = (array.ptr, array.shape, array.strides, array.dtype.str)
    hit = _views.get(key)
    if hit is None or hit[0]._buf is not array._buf:
        if len(_views) > 64:
            _views.clear()
        hit = _views[key] = (array, torch.as_tensor(array, device=f"cuda:{array.queue.device}"))
    return hit[1]


def _external_stream(queue):
    import torch

    key = (queue.device, int(queue.stream))
    s = _streams.get(key)
    if s is None:
        s = torch.cuda.ExternalStream(int(queue.stream), device=f"cuda:{queue.device}")
        _streams[key] = s
    return s


def offset_argmin(local_index, begin):
    """Row-sharded argmin over axis 0 needs the shard offset added back."""
    return local_index + begin
