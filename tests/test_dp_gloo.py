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


def test_bucket_plan_covers_every_gradient_once():
    elems = [2048 * 512, 512 * 512 * 9, 512 * 2048, 10, 0, 64 * 3 * 49]
    offsets, buckets, total = dp.plan_buckets(elems, 2, min_bytes=4 << 20)
    assert offsets[0] == 0 and all(o * 2 % 256 == 0 for o in offsets)
    for i in range(len(elems) - 1):
        assert offsets[i + 1] >= offsets[i] + elems[i]
    assert total >= offsets[-1] + elems[-1]
    # buckets tile the buffer in order, each but the last at least min_bytes
    assert buckets[0][0] == 0 and sum(b[1] for b in buckets) == total
    for (s0, n0, _), (s1, _, _) in zip(buckets, buckets[1:]):
        assert s1 == s0 + n0
    assert all(n * 2 >= (4 << 20) for _, n, _ in buckets[:-1])
    assert [b[2] for b in buckets] == sorted(b[2] for b in buckets) and buckets[-1][2] == len(elems) - 1
    with pytest.raises(ValueError):
        dp.plan_buckets([4], 3)


def _bucket_worker(rank, world, port, outdir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from oracle import corr_oracle as O
    comm = dp.ProcessGroupCommunicator()
    rs = np.random.RandomState(5)
    layers = []                                            # three small layers, gradients in backward order
    for (c, k, ks) in ((4, 6, 3), (6, 8, 1), (8, 5, 3)):
        x = rs.standard_normal((6, c, 7, 7)).astype(np.float32)
        dy = rs.standard_normal((6, k, 7, 7)).astype(np.float32)
        layers.append((x, dy, ks))
    order = [2, 1, 0]
    elems = [layers[i][1].shape[1] * layers[i][0].shape[1] * layers[i][2] ** 2 for i in order]
    buckets = dp.HostGradBuckets(comm, elems, min_bytes=1024)      # two buckets: the collectives overlap the loop
    a, b = dp.shard_bounds(6, rank, world)
    for j, i in enumerate(order):
        x, dy, ks = layers[i]
        g = O.conv2d_grad_weights(x[a:b], dy[a:b], (ks, ks), border_mode="half")
        buckets.view(j)[...] = g.ravel()
        buckets.ready(j)
    buckets.wait()
    np.savez(os.path.join(outdir, "b%d.npz" % rank), nb=len(buckets.buckets), **{"g%d" % j: buckets.view(j) for j in range(3)})
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_gradients_of_two_ranks_equal_the_full_batch():
    import torch.multiprocessing as mp
    from oracle import corr_oracle as O
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_bucket_worker, args=(2, port, d), nprocs=2, join=True)
        r0, r1 = (np.load(os.path.join(d, "b%d.npz" % r)) for r in range(2))
        assert int(r0["nb"]) >= 2
        rs = np.random.RandomState(5)
        shapes = ((4, 6, 3), (6, 8, 1), (8, 5, 3))
        full = []
        for (c, k, ks) in shapes:
            x = rs.standard_normal((6, c, 7, 7)).astype(np.float32)
            dy = rs.standard_normal((6, k, 7, 7)).astype(np.float32)
            full.append(O.conv2d_grad_weights(x, dy, (ks, ks), border_mode="half"))
        for j, i in enumerate([2, 1, 0]):
            assert O.rel_err(r0["g%d" % j].reshape(full[i].shape), full[i]) < 1e-5
            assert np.array_equal(r0["g%d" % j], r1["g%d" % j])
