"""Row sharding across the GPUs of one box and the few exchanges it needs.

The reference has no multi-device code (one queue per device,
mlir/lib/Conversion/GpuToGpuRuntime.cpp:169-197).  The benchmark workloads
shard along axis 0 -- one process per GPU, every process runs the same
single-GPU kernels on its rows -- and only three results span shards: a full
sum, a column-wise min, and the per-cluster sums/counts of a k-means
iteration.  Those partials are a few KB, so the exchange is latency bound.  On
GPUs it is the library's own peer-memory routine (csrc/kernels/peer_exchange.cuh:
every rank publishes its partial in a mailbox the others map over NVLink,
waits for their flags and combines all partials in rank order).  Inside
`across(dist)` the library's reductions over the sharded axis run it in the
block that finishes the reduction, so reduction and exchange are one launch;
`allreduce` / `allreduce_many` launch it on its own for partials produced by
other kernels (one flag round trip for up to four arrays).  torch.distributed
carries only the one-time exchange of the mailbox handles, and remains the
path for host arrays (gloo in the CPU tests), for partials above 64 KB and when
peer mapping is unavailable (NCCL).
"""

import contextlib

import ctypes
import os

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
    group = peer_group(partial.queue, dist)
    if group is not None and group.accepts(partial):
        group.allreduce(partial, op)
        return partial
    # Run the collective in stream order behind the kernels that produced the
    # partial: torch adopts the queue's stream for the duration of the call, so
    # no host synchronisation is needed on either side.
    stream = _external_stream(partial.queue)
    with torch.cuda.stream(stream):
        dist.all_reduce(_torch_view(partial), op=rop)
    return partial


class _ShardExchange:
    """State a queue carries inside `across`: how reductions over the sharded
    axis reach the other GPUs' results."""

    slot_bytes = 65536

    def __init__(self, dist, queue):
        self.dist = dist
        self.group = peer_group(queue, dist)  # None: NCCL through torch.distributed

    def allreduce(self, out, op):
        allreduce(out, op, self.dist)


@contextlib.contextmanager
def across(dist, queue=None):
    """Inside the block, arrays on `queue` are the process's shard of rows of a
    larger array split over the ranks of `dist`: a full reduction or a reduction
    over axis 0 (np.sum(a), np.min(a, axis=0) in an `njit` function, or
    `reduce_ops.reduce`) returns the result over ALL shards, identical on every
    rank.  Sums, products, minima and maxima whose result fits 64 KB are
    exchanged by the reduction kernel itself (its last block runs the
    peer-memory all-reduce); anything else is followed by `allreduce`.  With
    `dist` None or a world of one the block changes nothing.  Every rank must
    run the same reductions in the same order."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        yield
        return
    from . import runtime as _rt

    queue = queue if queue is not None else _rt.get_queue()
    previous = getattr(queue, "shard_exchange", None)
    queue.shard_exchange = _ShardExchange(dist, queue)
    try:
        yield
    finally:
        queue.shard_exchange = previous


def allreduce_many(partials, dist=None):
    """In-place all-reduce of up to four partial results `[(array, op), ...]`
    (device arrays on one queue) behind a single flag round trip; falls back to
    one `allreduce` per array when the peer mailboxes cannot carry them."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return
    arrays = [a for a, _op in partials]
    group = peer_group(arrays[0].queue, dist) if arrays and not isinstance(arrays[0], np.ndarray) else None
    if group is not None and len(partials) <= 4 and all(group.accepts(a) for a in arrays) and \
            sum(-(-a.nbytes // 16) * 16 for a in arrays) <= PEER_SLOT_BYTES and \
            all(op in _REDUCE_OPS for _a, op in partials):
        group.allreduce_many(partials)
        return
    for a, op in partials:
        allreduce(a, op, dist)


PEER_SLOT_BYTES = 65536                       # payload one call can carry
# header + 2 slots x 16 source ranks x the payload as tagged 8-byte words
PEER_MAILBOX_BYTES = 256 + 2 * 16 * 2 * PEER_SLOT_BYTES
_PEER_TYPES = {"float32": "f32", "float64": "f64", "int32": "i32", "int64": "i64"}


class PeerGroup:
    """The mailboxes of one queue's ranks for the peer-memory all-reduce.

    Built collectively (every rank of `dist` constructs it at the same point):
    each rank allocates its mailbox, the 64-byte handles travel through
    `dist.all_gather_object`, and every rank maps the others' mailboxes.
    `ok` is False on every rank if any rank failed to map a peer."""

    def __init__(self, queue, dist):
        from .device_array import from_host

        self.queue = queue
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self.seq = 0
        self.ok = False
        self._opened = []
        lib = queue.lib
        self._lib = lib
        self.mailbox = lib.gpuxPeerAlloc(queue.handle, PEER_MAILBOX_BYTES)
        handle = (ctypes.c_ubyte * 64)()
        mine = None
        if self.mailbox and self.world <= 16 and lib.gpuxPeerExport(self.mailbox, handle) == 0:
            mine = bytes(handle)
        lib.gpuxClearLastError()
        handles = [None] * self.world
        dist.all_gather_object(handles, mine)
        bases = [0] * self.world
        good = all(h is not None for h in handles)
        if good:
            for r, h in enumerate(handles):
                if r == self.rank:
                    bases[r] = self.mailbox
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                p = lib.gpuxPeerOpen(queue.handle, buf)
                if not p:
                    good = False
                    lib.gpuxClearLastError()
                    break
                self._opened.append(p)
                bases[r] = p
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(good))
        if all(flags):
            self.table = from_host(np.asarray(bases, dtype=np.uint64), queue=queue)
            self.ok = True
        else:
            self.close()

    def accepts(self, partial):
        return (self.ok and partial.dtype.name in _PEER_TYPES and partial.is_c_contiguous
                and 0 < partial.nbytes <= PEER_SLOT_BYTES and partial.queue is self.queue)

    def allreduce(self, partial, op):
        """One launch on the partial's queue; the result is bit-identical on
        every rank (the partials are combined in rank order).  The call number
        lives in the mailbox, so the launch can be recorded in a CUDA graph;
        `seq` here only counts the calls submitted from the host."""
        self.seq += 1
        q = self.queue
        k = q.builtin(f"nmb_peer_allreduce_{op}_{_PEER_TYPES[partial.dtype.name]}")
        q.launch(k, (1,), (1024,),
                 [("ptr", partial.ptr), np.int64(partial.size), ("ptr", self.table.ptr),
                  np.int32(self.rank), np.int32(self.world), ("ptr", q.status_ptr)])

    def allreduce_many(self, partials):
        """One launch for up to four (array, op) pairs: all payloads travel
        behind one flag."""
        self.seq += 1
        q = self.queue
        k = q.builtin("nmb_peer_allreduce_multi")
        args = []
        for i in range(4):
            if i < len(partials):
                a, op = partials[i]
                code = list(_PEER_TYPES).index(a.dtype.name) + 4 * _REDUCE_OPS.index(op)
                args += [("ptr", a.ptr), np.int64(a.size), np.int32(code)]
            else:
                args += [("ptr", 0), np.int64(0), np.int32(0)]
        q.launch(k, (1,), (1024,), args + [("ptr", self.table.ptr), np.int32(self.rank), np.int32(self.world),
                                           ("ptr", q.status_ptr)])

    def close(self):
        for p in self._opened:
            self._lib.gpuxPeerClose(self.queue.handle, p)
        self._opened = []
        if self.mailbox:
            self._lib.gpuxPeerFree(self.queue.handle, self.mailbox)
            self.mailbox = None
        self.ok = False


_peer_groups = {}


def peer_group(queue, dist):
    """The queue's PeerGroup, built on first use (collectively: every rank
    reaches its first device all-reduce at the same point of the program), or
    None when NUMBA_MLIR_B200_PEER_ALLREDUCE=0 or the mapping failed."""
    if os.environ.get("NUMBA_MLIR_B200_PEER_ALLREDUCE", "1") == "0":
        return None
    g = _peer_groups.get(queue)
    if g is None:
        g = _peer_groups[queue] = PeerGroup(queue, dist)
    return g if g.ok else None


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


def bind_host_to_gpu(device_index):
    """Runs this process on the CPU cores next to GPU `device_index`, so that
    host buffers allocated afterwards, page-locked ones included, land in that
    socket's memory and the copies of several ranks do not all cross one
    socket's memory and links.  The cores come from NVML's CPU affinity of
    the device (or, failing that, from the NUMA node sysfs names for its PCIe
    slot); only this process's CPU affinity changes.  Returns the number of
    cores the process is bound to, or None when the topology is not visible
    or names every core anyway (nothing is changed then)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        idx = int(device_index)
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            if idx < len(ids) and ids[idx].isdigit():
                idx = int(ids[idx])
        handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        allowed = os.sched_getaffinity(0)
        cpus = set()
        try:
            words = (max(allowed) + 64) // 64
            for w, mask in enumerate(pynvml.nvmlDeviceGetCpuAffinity(handle, words)):
                cpus.update(64 * w + b for b in range(64) if (int(mask) >> b) & 1)
        except Exception:
            cpus = set()
        if not cpus:
            bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
            bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
            if len(bus.split(":")[0]) == 8:  # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
                bus = bus[4:]
            with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
                node = int(f.read().strip())
            if node < 0:
                return None
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
        target = cpus & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
        return len(target)
    except Exception:
        return None


def offset_argmin(local_index, begin):
    """Row-sharded argmin over axis 0 needs the shard offset added back."""
    return local_index + begin
