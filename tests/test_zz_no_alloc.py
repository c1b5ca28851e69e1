"""The allocation-free gradWeights entry point (``b200conv_wgrad_static``).

Some users of the library are not allowed to call ``cudaMalloc`` once they are running: a
host program that has handed the whole GPU memory to its own allocator, a loop that must
not stall on the device-wide synchronisation of ``cudaMalloc``/``cudaFree``, or a deployment
whose memory budget is fixed after warm-up.  For them the split-K scratch lives in a fixed
array inside the library.  The test calls the entry point through the C ABI several times in a
row (the array keeps the previous call's contents, so a call must not be disturbed by the one
before) and compares each result with the regular ``b200conv_wgrad`` and with the CPU oracle.

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


def _case(ctx, rs, xshape, kshape, border, sub, K, groups=1, dtype=np.float32):
    x = rs.standard_normal(xshape).astype(dtype)
    wshape = (K, xshape[1] // groups) + kshape
    yshape, pads = hostlogic.forward_shape(xshape, wshape, border, sub, (1, 1), groups)
    dy = (rs.standard_normal(yshape) * 0.1).astype(dtype)
    X = shim.DeviceTensor.from_host(ctx, x, "nhwc")
    DY = shim.DeviceTensor.from_host(ctx, dy, "nhwc")
    d = shim.make_desc(xshape, wshape, yshape, pads, sub, (1, 1), groups, True, dtype)
    return x, dy, X, DY, d, wshape


# (input shape, filter size, border, stride, filters, groups, dtype, flags)
LAYERS = [((6, 48, 14, 14), (3, 3), (1, 1), (1, 1), 40, 1, np.float32, 0),
          ((4, 24, 17, 15), (3, 3), "half", (2, 2), 56, 1, np.float32, 0),
          ((5, 3, 20, 20), (3, 3), "half", (1, 1), 32, 1, np.float32, 0),            # three channels: one tap per work item, no row folding here
          ((4, 64, 9, 9), (3, 3), "half", (1, 1), 64, 2, np.float32, 0),             # two groups of 32 channels
          ((6, 64, 12, 12), (3, 3), "half", (1, 1), 96, 1, np.float16, 0),           # float16
          ((6, 48, 14, 14), (3, 3), (1, 1), (1, 1), 40, 1, np.float32, shim.ATOMIC_SPLITK),   # adds into the array: it must be cleared first
          ((3, 16, 1, 9), (3, 3), "half", (2, 2), 24, 1, np.float32, 0),             # stride 2 on one image row: a stride class without pixels, its taps are dropped
          ((2, 512, 7, 7), (3, 3), "half", (1, 1), 512, 1, np.float32, 0)]           # 9.4 MB per slab: three of them fit the 32 MiB


def test_static_scratch_wgrad_matches_pooled_wgrad_and_the_oracle():
    """Back to back on one context, so that every call finds the array as the previous one left it:
    results equal b200conv_wgrad's within the float tolerance and the CPU oracle's too, and from
    the second call on neither the context's pool nor the device's free memory changes."""
    from oracle import corr_oracle as O
    ctx = shim.get_context(0)
    rs = np.random.RandomState(77)
    for n, (xshape, kshape, border, sub, K, groups, dtype, flags) in enumerate(LAYERS):
        tol = TOL if dtype == np.float32 else 2e-2
        x, dy, X, DY, d, wshape = _case(ctx, rs, xshape, kshape, border, sub, K, groups, dtype)
        ref = shim.DeviceTensor(ctx, wshape, dtype)
        got = shim.DeviceTensor(ctx, wshape, dtype)
        ctx.wgrad(d, X.ptr, DY.ptr, ref.ptr, shim.IN_NHWC | shim.IN2_NHWC | flags)
        assert ctx.last_algo == "umma"
        for rep in range(2):
            ctx.memset(got.ptr, 0xFF, got.nbytes)
            ctx.sync()
            before = ctx.memory_info()
            ctx.wgrad_static(d, X.ptr, DY.ptr, got.ptr, flags)
            ctx.sync()
            if n > 0 or rep > 0:                 # the very first call on a device loads the module and its array
                assert ctx.memory_info() == before
            a, b = got.to_host(), ref.to_host()
            assert np.isfinite(a).all()
            assert rel_err(a, b) < tol, (n, rep)
            want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), kshape, border_mode=border,
                                         subsample=sub, num_groups=groups)
            assert rel_err(a, want) < tol, (n, rep)
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
