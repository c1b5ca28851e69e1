"""Data-parallel use of the convolution path: batch shards on several GPUs, one exchange.

The reference parallelises CorrMM over the batch inside one process with OpenMP and adds
the per-thread filter-gradient partials at the end (theano/tensor/nnet/c_code/corr_gemm.c:304,
397-455).  Across GPUs the same decomposition holds: forward and gradInputs need nothing
from other ranks, gradWeights is summed over ranks with one all-reduce.  One process per
GPU; the collective runs inside ``libb200conv`` on NCCL.  A second communicator built on a
``torch.distributed`` process group (gloo on CPU) carries the same host logic where no GPU
is present.
"""
import os
import time

import numpy as np


def shard_bounds(n, rank, world):
    """Contiguous batch slice of a rank: the first ``n % world`` ranks take one extra image."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank %d of %d" % (rank, world))
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def file_exchange(path, timeout=60.0):
    """Returns ``exchange(rank, payload)``: rank 0 publishes bytes through a file, the others
    wait for it (bounded).  Enough to hand the NCCL unique id to the other ranks of one node."""
    def exchange(rank, payload=None):
        if rank == 0:
            tmp = path + ".tmp.%d" % os.getpid()
            with open(tmp, "wb") as f:
                f.write(payload)
            os.replace(tmp, path)
            return payload
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > timeout:
                raise TimeoutError("rank %d: no unique id from rank 0 after %.0f s" % (rank, timeout))
            time.sleep(0.02)
        with open(path, "rb") as f:
            return f.read()
    return exchange


def plan_buckets(elems, itemsize, min_bytes=4 << 20, align=256):
    """Lay the filter gradients of a network out in one flat buffer, in the order in which the
    backward pass produces them (`elems[i]` = element count of the i-th gradient to become ready),
    and cut the buffer into buckets of at least `min_bytes` (the last one takes what is left).

    Returns ``(offsets, buckets, total)``: the element offset of every gradient (multiples of
    `align` bytes), buckets as ``(first_element, n_elements, last_gradient_index)`` and the total
    element count.  One collective per bucket replaces one per layer: per-layer tensors of the
    benchmark networks run from 9 kB to 9 MB, and a small all-reduce costs its launch latency."""
    if itemsize <= 0 or align % itemsize:
        raise ValueError("alignment must be a multiple of the item size")
    step = align // itemsize
    offsets, buckets = [], []
    pos = start = 0
    for i, n in enumerate(elems):
        if n < 0:
            raise ValueError("negative gradient size")
        offsets.append(pos)
        pos += (int(n) + step - 1) // step * step
        if (pos - start) * itemsize >= min_bytes:
            buckets.append((start, pos - start, i))
            start = pos
    if pos > start:
        buckets.append((start, pos - start, len(elems) - 1))
    return offsets, buckets, pos


class GradBuckets(object):
    """Filter gradients of many layers in flat device buckets that are all-reduced while the
    backward pass goes on (the sum the reference forms over its OpenMP threads,
    theano/tensor/nnet/c_code/corr_gemm.c:443-455, formed over GPUs).

    ``ptr(i)`` is where gradWeights of the i-th layer (in backward order) writes its result:
    the split-K reduction kernel stores straight into the bucket.  ``ready(i)`` is called once
    that call has been enqueued; when it completes a bucket, the bucket's all-reduce is queued on
    the library's communication stream and runs beside the remaining layers.  ``wait()`` orders
    the main stream after all of them."""

    def __init__(self, ctx, elems, dtype, min_bytes=4 << 20, world=1):
        self.ctx, self.dtype, self.world = ctx, np.dtype(dtype), world
        self.offsets, self.buckets, self.total = plan_buckets(elems, self.dtype.itemsize, min_bytes)
        self.base = ctx.malloc(max(self.total, 1) * self.dtype.itemsize)
        ctx.memset(self.base, 0, max(self.total, 1) * self.dtype.itemsize)   # alignment gaps are summed too
        self._bucket_of_last = {last: k for k, (_, _, last) in enumerate(self.buckets)}
        self.elems = [int(n) for n in elems]

    def ptr(self, i):
        return self.base + self.offsets[i] * self.dtype.itemsize

    def ready(self, i):
        k = self._bucket_of_last.get(i)
        if k is not None and self.world > 1:
            first, n, _ = self.buckets[k]
            self.ctx.allreduce_sum_async(self.base + first * self.dtype.itemsize, n, self.dtype)
        return k

    def wait(self):
        if self.world > 1:
            self.ctx.comm_wait()

    def to_host(self, i):
        """Gradient i as a flat host array (synchronises)."""
        out = np.empty(self.elems[i], self.dtype)
        self.ctx.d2h(out, self.ptr(i))
        self.ctx.sync()
        return out

    def free(self):
        if self.base:
            self.ctx.free(self.base)
            self.base = None


class HostGradBuckets(object):
    """The same bucketing on host arrays over a ``torch.distributed`` process group: the CPU
    stand-in that carries the bucket logic where no GPU is present (asynchronous all-reduces,
    joined by ``wait``)."""

    def __init__(self, comm, elems, dtype=np.float32, min_bytes=4 << 20):
        self.comm, self.dtype = comm, np.dtype(dtype)
        self.offsets, self.buckets, self.total = plan_buckets(elems, self.dtype.itemsize, min_bytes)
        self.flat = np.zeros(max(self.total, 1), self.dtype)
        self.elems = [int(n) for n in elems]
        self._bucket_of_last = {last: k for k, (_, _, last) in enumerate(self.buckets)}
        self._pending = []

    def view(self, i):
        return self.flat[self.offsets[i]:self.offsets[i] + self.elems[i]]

    def ready(self, i):
        k = self._bucket_of_last.get(i)
        if k is not None:
            import torch
            first, n, _ = self.buckets[k]
            t = torch.from_numpy(self.flat[first:first + n])       # shares the memory
            self._pending.append(self.comm.dist.all_reduce(t, op=self.comm.dist.ReduceOp.SUM,
                                                           group=self.comm.group, async_op=True))
        return k

    def wait(self):
        for w in self._pending:
            w.wait()
        self._pending = []


class NcclCommunicator(object):
    """Sum-all-reduce of device buffers through the library's NCCL entry points."""

    def __init__(self, ctx, rank, world, exchange):
        self.ctx, self.rank, self.world = ctx, rank, world
        if world > 1:
            uid = exchange(rank, ctx.nccl_unique_id() if rank == 0 else None)
            ctx.nccl_init(world, rank, uid)

    def allreduce_device(self, tensor):
        if self.world > 1:
            self.ctx.allreduce_sum(tensor.ptr, int(np.prod(tensor.shape)), tensor.dtype)
        return tensor

    def barrier(self):
        self.ctx.barrier()


class ProcessGroupCommunicator(object):
    """Same contract on host arrays over a ``torch.distributed`` process group (gloo)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def allreduce_host(self, arr):
        import torch
        t = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32))
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)
        return t.numpy().astype(arr.dtype, copy=False)

    def barrier(self):
        self.dist.barrier(group=self.group)


class DataParallel(object):
    """One training-style step of a convolution layer on this rank's batch shard.

    ``kernels`` supplies the three directions on host arrays (default: the CUDA path of
    ``theano_b200.shim``); ``comm`` is a communicator with ``allreduce_host``.
    """

    def __init__(self, comm, kernels=None, **conv_kwargs):
        self.comm, self.kw = comm, conv_kwargs
        if kernels is None:
            from . import shim
            kernels = (shim.conv2d_forward, shim.conv2d_grad_inputs, shim.conv2d_grad_weights)
        self.fwd, self.gi, self.gw = kernels

    def shard(self, arr):
        a, b = shard_bounds(arr.shape[0], self.comm.rank, self.comm.world)
        return arr[a:b]

    def step(self, x_shard, w, dy_shard):
        y = self.fwd(x_shard, w, **self.kw)
        dx = self.gi(w, dy_shard, x_shard.shape[2:], **self.kw)
        dw = self.gw(x_shard, dy_shard, w.shape[2:], **self.kw)
        return y, dx, self.comm.allreduce_host(dw)
