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
        for p in procs:
            assert p.wait(timeout=300) == 0
        rs = np.random.RandomState(33)
        x = rs.standard_normal((10, 32, 12, 12)).astype(np.float32)
        dy = rs.standard_normal((10, 48, 12, 12)).astype(np.float32)
        full = O.conv2d_grad_weights(x, dy, (3, 3), border_mode="half")
        dw0, dw1 = (np.load(os.path.join(d, "dw%d.npy" % r)) for r in range(2))
        assert np.array_equal(dw0, dw1)
        assert O.rel_err(dw0, full) < 5e-3
