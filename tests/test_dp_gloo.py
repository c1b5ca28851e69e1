"""Data-parallel host logic with two CPU ranks over gloo: batch sharding, the all-reduce of
the filter gradients, and what the survivors see when a rank never shows up."""
import datetime
import os
import socket
import tempfile

import numpy as np
import pytest

from theano_b200 import dp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_kernels():
    from oracle import corr_oracle as O
    return (lambda x, w, **k: O.conv2d(x, w, **k),
            lambda w, dy, shp, **k: O.conv2d_grad_inputs(w, dy, shp, **k),
            lambda x, dy, shp, **k: O.conv2d_grad_weights(x, dy, shp, **k))


def _worker(rank, world, port, outdir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    rs = np.random.RandomState(21)
    x = rs.standard_normal((7, 4, 9, 9)).astype(np.float32)          # 7 images on 2 ranks: 4 + 3
    w = rs.standard_normal((6, 4, 3, 3)).astype(np.float32)
    dy = rs.standard_normal((7, 6, 9, 9)).astype(np.float32)
    layer = dp.DataParallel(dp.ProcessGroupCommunicator(), kernels=_oracle_kernels(), border_mode="half")
    y, dx, dw = layer.step(layer.shard(x), w, layer.shard(dy))
    np.savez(os.path.join(outdir, "rank%d.npz" % rank), y=y, dx=dx, dw=dw)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_bounds():
    assert [dp.shard_bounds(7, r, 2) for r in range(2)] == [(0, 4), (4, 7)]
    assert [dp.shard_bounds(8, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert dp.shard_bounds(1, 1, 2) == (1, 1)                          # an empty shard is legal
    with pytest.raises(ValueError):
        dp.shard_bounds(4, 2, 2)


def test_two_ranks_equal_the_full_batch():
    import torch.multiprocessing as mp
    from oracle import corr_oracle as O
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, port, d), nprocs=2, join=True)
        r0, r1 = (np.load(os.path.join(d, "rank%d.npz" % r)) for r in range(2))
        rs = np.random.RandomState(21)
        x = rs.standard_normal((7, 4, 9, 9)).astype(np.float32)
        w = rs.standard_normal((6, 4, 3, 3)).astype(np.float32)
        dy = rs.standard_normal((7, 6, 9, 9)).astype(np.float32)
        assert O.rel_err(np.concatenate([r0["y"], r1["y"]]), O.conv2d(x, w, border_mode="half")) < 1e-6
        assert O.rel_err(np.concatenate([r0["dx"], r1["dx"]]), O.conv2d_grad_inputs(w, dy, (9, 9), border_mode="half")) < 1e-6
        full = O.conv2d_grad_weights(x, dy, (3, 3), border_mode="half")
        assert O.rel_err(r0["dw"], full) < 1e-5 and np.array_equal(r0["dw"], r1["dw"])


def _lonely_worker(rank, world, port, outdir):
    """Rank 1 never joins; rank 0 must get an error within the group's timeout, not hang."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if rank == 1:
        return
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        dp.ProcessGroupCommunicator().allreduce_host(np.ones(4, np.float32))
        outcome = "no error"
    except Exception as e:               # the failure is seen on the host, before any launch
        outcome = type(e).__name__
    open(os.path.join(outdir, "outcome"), "w").write(outcome)


def test_missing_rank_is_detected_on_the_host():
    import torch.multiprocessing as mp
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_lonely_worker, args=(2, port, d), nprocs=2, join=True)
        assert open(os.path.join(d, "outcome")).read() != "no error"


def test_file_exchange_times_out_and_delivers():
    with tempfile.TemporaryDirectory() as d:
        ex = dp.file_exchange(os.path.join(d, "uid"), timeout=0.2)
        with pytest.raises(TimeoutError):
            ex(1)
        assert ex(0, b"x" * 128) == b"x" * 128
        assert ex(1) == b"x" * 128
