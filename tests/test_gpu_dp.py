"""NCCL path of the library on real GPUs: a one-rank communicator (identity) and, where two
GPUs are visible, two ranks whose all-reduced filter gradient equals the full-batch result."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, numpy as np
sys.path.insert(0, %(root)r)
from theano_b200 import shim, dp
rank, world, d = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
os.environ["NCCL_NVLS_ENABLE"] = "0"
ctx = shim.Context(rank)
comm = dp.NcclCommunicator(ctx, rank, world, dp.file_exchange(os.path.join(d, "uid"), timeout=120))
rs = np.random.RandomState(33)
x = rs.standard_normal((10, 32, 12, 12)).astype(np.float32)
dy = rs.standard_normal((10, 48, 12, 12)).astype(np.float32)
a, b = dp.shard_bounds(10, rank, world)
X = shim.DeviceTensor.from_host(ctx, x[a:b], "nhwc")
DY = shim.DeviceTensor.from_host(ctx, dy[a:b], "nhwc")
DW = shim.device_grad_weights(X, DY, (3, 3), border_mode="half")
comm.allreduce_device(DW)
comm.barrier()
np.save(os.path.join(d, "dw%%d.npy" %% rank), DW.to_host())
"""


def _device_count():
    out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True)
    return len([l for l in out.stdout.splitlines() if l.startswith("GPU ")]) if out.returncode == 0 else 0


def test_single_rank_communicator_is_identity():
    from theano_b200 import dp, shim
    ctx = shim.get_context(0)
    with tempfile.TemporaryDirectory() as d:
        uid = ctx.nccl_unique_id()
        assert len(uid) == 128
        ctx.nccl_init(1, 0, uid)
        a = np.arange(1000, dtype=np.float32)
        t = shim.DeviceTensor.from_host(ctx, a.reshape(1, 1, 10, 100))
        ctx.allreduce_sum(t.ptr, a.size, np.float32)
        ctx.barrier()
        assert np.array_equal(t.to_host().ravel(), a)
        ctx.lib.b200conv_nccl_destroy(ctx.h)


def test_two_ranks_allreduce_gradweights():
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import corr_oracle as O
    with tempfile.TemporaryDirectory() as d:
        script = os.path.join(d, "worker.py")
        open(script, "w").write(WORKER % {"root": ROOT})
        procs = [subprocess.Popen([sys.executable, script, str(r), "2", d]) for r in range(2)]
        try:
            for p in procs:
                assert p.wait(timeout=300) == 0
        finally:
            for p in procs:                      # no worker outlives the test
                if p.poll() is None:
                    p.kill()
        rs = np.random.RandomState(33)
        x = rs.standard_normal((10, 32, 12, 12)).astype(np.float32)
        dy = rs.standard_normal((10, 48, 12, 12)).astype(np.float32)
        full = O.conv2d_grad_weights(x, dy, (3, 3), border_mode="half")
        dw0, dw1 = (np.load(os.path.join(d, "dw%d.npy" % r)) for r in range(2))
        assert np.array_equal(dw0, dw1)
        assert O.rel_err(dw0, full) < 5e-3


def test_two_devices_in_one_process():
    """Kernel attributes are per device: a context on device 1 opened after device 0 ran must
    launch the tensor-core kernels too (skipped with fewer than two GPUs)."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import corr_oracle as O
    from theano_b200 import shim
    rs = np.random.RandomState(8)
    x = rs.standard_normal((4, 32, 10, 10)).astype(np.float32)
    w = (rs.standard_normal((48, 32, 3, 3)) * 0.1).astype(np.float32)
    dy = rs.standard_normal((4, 48, 10, 10)).astype(np.float32)
    kw = dict(border_mode="half")
    for dev in (0, 1):
        ctx = shim.Context(dev)
        assert O.rel_err(shim.conv2d_forward(x, w, ctx=ctx, **kw), O.conv2d(x, w, **kw)) < 5e-3
        assert ctx.last_algo == "umma"
        assert O.rel_err(shim.conv2d_grad_inputs(w, dy, (10, 10), ctx=ctx, **kw), O.conv2d_grad_inputs(w, dy, (10, 10), **kw)) < 5e-3
        assert O.rel_err(shim.conv2d_grad_weights(x, dy, (3, 3), ctx=ctx, **kw), O.conv2d_grad_weights(x, dy, (3, 3), **kw)) < 5e-3
        ctx.close()


def _fake_nccl(tmpdir):
    so = os.path.join(tmpdir, "libfakenccl.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", so, os.path.join(ROOT, "tests", "fake_nccl.c"), "-ldl"])
    return so


@pytest.mark.parametrize("mode, needle", [("1", "asynchronous error"), ("2", "deadline")], ids=["nccl_error", "stalled_collective"])
def test_watchdog_aborts_a_failed_collective(mode, needle):
    """A collective that fails or stalls must end in an error on the host, not in a blocked
    process.  The failure is made on the host: a stand-in NCCL library whose all-reduce keeps the
    stream waiting on a sleeping host function (no GPU kernel spins) and whose error state reports
    a failure.  The context must keep working afterwards."""
    import time
    from oracle import corr_oracle as O
    from theano_b200 import shim
    old = {k: os.environ.get(k) for k in ("B200CONV_NCCL_LIB", "FAKE_NCCL_MODE")}
    with tempfile.TemporaryDirectory() as d:
        try:
            os.environ["B200CONV_NCCL_LIB"] = _fake_nccl(d)
            os.environ["FAKE_NCCL_MODE"] = mode
            ctx = shim.Context(0)
            ctx.nccl_init(1, 0, ctx.nccl_unique_id())
            if mode == "2":
                ctx.set_comm_timeout(50)
            buf = ctx.malloc(64)
            ctx.allreduce_sum(buf, 4, np.float32)
            t0 = time.time()
            with pytest.raises(shim.B200Error) as err:
                ctx.sync()
            assert "error %d" % shim.E_NCCL in str(err.value) and needle in str(err.value)
            assert time.time() - t0 < 5.0
            rs = np.random.RandomState(8)
            x = rs.standard_normal((2, 16, 8, 8)).astype(np.float32)
            w = (rs.standard_normal((16, 16, 3, 3)) * 0.1).astype(np.float32)
            assert O.rel_err(shim.conv2d_forward(x, w, ctx=ctx, border_mode="half"), O.conv2d(x, w, border_mode="half")) < 5e-3
            ctx.close()
        finally:
            for k, v in old.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
