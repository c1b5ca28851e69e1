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
