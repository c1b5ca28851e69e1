"""The allocation-free gradWeights entry point (``b200conv_wgrad_static``).

Some users of the library are not allowed to call ``cudaMalloc`` once they are running: a
host program that has handed the whole GPU memory to its own allocator, a loop that must
not stall on the device-wide synchronisation of ``cudaMalloc``/``cudaFree``, or a deployment
whose memory budget is fixed after warm-up.  For them the split-K scratch lives in a fixed
array inside the library.  The test calls the entry point through the C ABI twice in a row
(the array keeps the previous call's contents, so the second call must not be disturbed by
the first) and compares each result with the regular ``b200conv_wgrad``.

The file name makes pytest collect it last, so a run that stops at the first failure has
already gone through every other test.
"""
import numpy as np
import pytest

from theano_b200 import hostlogic, shim

pytestmark = pytest.mark.gpu

TOL = 5e-3   # float32 on TF32 tensor cores, the tolerance of the other float32 parity tests


def rel_err(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / max(np.abs(b).max(), 1e-30))


def _case(ctx, rs, xshape, kshape, border, sub, K):
    x = rs.standard_normal(xshape).astype(np.float32)
    wshape = (K, xshape[1]) + kshape
    yshape, pads = hostlogic.forward_shape(xshape, wshape, border, sub, (1, 1))
    dy = rs.standard_normal(yshape).astype(np.float32)
    X = shim.DeviceTensor.from_host(ctx, x, "nhwc")
    DY = shim.DeviceTensor.from_host(ctx, dy, "nhwc")
    d = shim.make_desc(xshape, wshape, yshape, pads, sub, (1, 1), 1, True, np.float32)
    return X, DY, d, wshape


def test_static_scratch_wgrad_matches_pooled_wgrad_twice():
    ctx = shim.get_context(0)
    rs = np.random.RandomState(77)
    # two different layers back to back: the second reuses the array the first one wrote
    layers = [((6, 48, 14, 14), (3, 3), (1, 1), (1, 1), 40),
              ((4, 24, 17, 15), (3, 3), "half", (2, 2), 56)]
    for xshape, kshape, border, sub, K in layers:
        X, DY, d, wshape = _case(ctx, rs, xshape, kshape, border, sub, K)
        ref = shim.DeviceTensor(ctx, wshape, np.float32)
        got = shim.DeviceTensor(ctx, wshape, np.float32)
        ctx.wgrad(d, X.ptr, DY.ptr, ref.ptr, shim.IN_NHWC | shim.IN2_NHWC)
        ctx.memset(got.ptr, 0xFF, got.nbytes)
        ctx.wgrad_static(d, X.ptr, DY.ptr, got.ptr)
        a, b = got.to_host(), ref.to_host()
        assert np.isfinite(a).all()
        assert rel_err(a, b) < TOL
        for t in (X, DY, ref, got):
            t.free()


def test_static_scratch_rejects_oversized_gradient():
    ctx = shim.get_context(0)
    # 7x7 filters, 1024 -> 1024 channels: one slab is 196 MiB, far beyond the 32 MiB array
    xshape, wshape = (1, 1024, 8, 8), (1024, 1024, 7, 7)
    yshape, pads = hostlogic.forward_shape(xshape, wshape, "half", (1, 1), (1, 1))
    d = shim.make_desc(xshape, wshape, yshape, pads, (1, 1), (1, 1), 1, True, np.float32)
    X = shim.DeviceTensor(ctx, xshape, np.float32, "nhwc")
    DY = shim.DeviceTensor(ctx, yshape, np.float32, "nhwc")
    with pytest.raises(ValueError, match="static scratch"):
        ctx.wgrad_static(d, X.ptr, DY.ptr, X.ptr)
    X.free()
    DY.free()
