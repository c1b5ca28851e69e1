"""Safety nets on the GPU that stand in for a memory checker: a device-side wait that runs out
on purpose (bounded, reported, context still usable) and outputs framed by canary bytes.

Nothing here faults, traps or hangs the GPU: the wait that runs out is a one-CTA kernel with a
limit of about a millisecond on a barrier nobody arrives on; it writes a status word and returns.
"""
import numpy as np
import pytest

from oracle import corr_oracle as O
from theano_b200 import shim

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return shim.get_context(0)


def _small_case(dtype=np.float32, seed=3):
    rs = np.random.RandomState(seed)
    x = rs.standard_normal((5, 32, 12, 12)).astype(dtype)
    w = (rs.standard_normal((48, 32, 3, 3)) * 0.1).astype(dtype)
    return x, w


def test_wait_that_runs_out_is_reported_and_the_context_survives(ctx):
    x, w = _small_case()
    kw = dict(border_mode="half")
    want = O.conv2d(x, w, **kw)
    ctx.set_wait_limit(2000000)                      # about a millisecond
    try:
        with pytest.raises(shim.B200Error) as err:
            ctx.selftest_wait()
        assert "error %d" % shim.E_TIMEOUT in str(err.value) and "wait ran out" in str(err.value)
        # the status word was reset: the same context computes again, also with the short limit
        assert O.rel_err(shim.conv2d_forward(x, w, ctx=ctx, **kw), want) < 5e-3
        with pytest.raises(shim.B200Error):
            ctx.selftest_wait()                      # and reports again
    finally:
        ctx.set_wait_limit(4000000000)
    assert O.rel_err(shim.conv2d_forward(x, w, ctx=ctx, **kw), want) < 5e-3
    with pytest.raises(ValueError):
        ctx.set_wait_limit(10)


CANARY, GUARD = 0x5A, 1 << 16


def _framed(ctx, nbytes):
    """Device buffer of nbytes with GUARD canary bytes on each side; returns (base, payload ptr)."""
    base = ctx.malloc(nbytes + 2 * GUARD)
    ctx.memset(base, CANARY, nbytes + 2 * GUARD)
    return base, base + GUARD


def _canaries_intact(ctx, base, nbytes):
    lo, hi = np.empty(GUARD, np.uint8), np.empty(GUARD, np.uint8)
    ctx.d2h(lo, base)
    ctx.d2h(hi, base + GUARD + nbytes)
    ctx.sync()
    return bool((lo == CANARY).all() and (hi == CANARY).all())


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["float32", "float16"])
@pytest.mark.parametrize("shape", [((6, 64, 14, 14), (64, 64, 3, 3), (1, 1), 1),      # TMA-store epilogue
                                   ((3, 24, 9, 11), (40, 24, 3, 2), (0, 1), 2),      # direct-store epilogue, stride 2
                                   ((4, 128, 7, 7), (256, 128, 1, 1), (0, 0), 1)],   # 1x1 layer as one row of pixels
                         ids=["3x3_c64", "odd_stride2", "1x1_flat"])
def test_outputs_stay_inside_their_buffers(ctx, dtype, shape):
    """Every direction writes a channels-last / OIHW output framed by canary bytes; the frame must
    be untouched afterwards and the payload right (what a memory checker would flag)."""
    xs, ws, pad, st = shape
    rs = np.random.RandomState(11)
    x = rs.standard_normal(xs).astype(dtype)
    w = (rs.standard_normal(ws) * 0.1).astype(dtype)
    kw = dict(border_mode=pad, subsample=(st, st))
    want_y = O.conv2d(x.astype(np.float32), w.astype(np.float32), **kw)
    dy = (rs.standard_normal(want_y.shape) * 0.1).astype(dtype)
    tol = 5e-3 if dtype == np.float32 else 2e-2
    T = shim.DeviceTensor
    X, W, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), T.from_host(ctx, dy, "nhwc")
    for name in ("fwd", "dgrad", "wgrad"):
        oshape = {"fwd": want_y.shape, "dgrad": xs, "wgrad": ws}[name]
        layout = "nchw" if name == "wgrad" else "nhwc"
        probe = T(ctx, oshape, dtype, layout)
        nbytes = probe.nbytes
        probe.free()
        base, ptr = _framed(ctx, nbytes)
        out = T(ctx, oshape, dtype, layout, _ptr=ptr)
        if name == "fwd":
            shim.device_conv2d(X, W, out=out, **kw)
            want = want_y
        elif name == "dgrad":
            shim.device_grad_inputs(W, DY, xs[2:], out=out, **kw)
            want = O.conv2d_grad_inputs(w.astype(np.float32), dy.astype(np.float32), xs[2:], **kw)
        else:
            shim.device_grad_weights(X, DY, ws[2:], out=out, **kw)
            want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), ws[2:], **kw)
        assert ctx.last_algo == "umma"
        assert _canaries_intact(ctx, base, nbytes), name
        assert O.rel_err(out.to_host().astype(np.float32), want) < tol, name
        ctx.free(base)
    for t in (X, W, DY):
        t.free()


def test_range_checked_build_passes_the_small_matrix():
    """The same parity tests on the library built with -DB200CONV_DEBUG, where every global store,
    tiled TMA store and gradient-slab index of the tensor-core kernels is compared with the
    extent the host passed (a violation fails the call).  Runs in a child process because a
    process binds one build of the library."""
    import os
    import subprocess
    import sys
    from theano_b200 import build as lib_build
    lib = lib_build.DEBUG_LIB
    if not os.path.exists(lib):
        pytest.skip("libb200conv_debug.so is not built (python -m theano_b200.build --debug)")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, B200CONV_LIB=lib)
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
                        os.path.join(root, "tests", "test_gpu_parity.py"), os.path.join(root, "tests", "test_gpu_prepack.py"),
                        "-k", "float32_against_reference or float16 or prepacked or medium or strided"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]


def test_large_host_arrays_travel_through_the_pinned_staging(ctx):
    """Host-pointer calls with arrays beyond 4 MB are cut into 16 MB chunks that copy threads move
    through pinned buffers while the DMA engine works on the previous chunk; sizes here are no
    multiple of the chunk, and every direction must still equal the oracle."""
    rs = np.random.RandomState(21)
    x = rs.standard_normal((37, 48, 50, 50)).astype(np.float32)            # 17.8 MB
    w = (rs.standard_normal((80, 48, 3, 3)) * 0.05).astype(np.float32)
    kw = dict(border_mode="half")
    y = shim.conv2d_forward(x, w, ctx=ctx, **kw)                            # 29.6 MB out
    want = O.conv2d(x, w, **kw)
    assert O.rel_err(y, want) < 5e-3
    dy = rs.standard_normal(y.shape).astype(np.float32)
    assert O.rel_err(shim.conv2d_grad_inputs(w, dy, (50, 50), ctx=ctx, **kw), O.conv2d_grad_inputs(w, dy, (50, 50), **kw)) < 5e-3
    assert O.rel_err(shim.conv2d_grad_weights(x, dy, (3, 3), ctx=ctx, **kw), O.conv2d_grad_weights(x, dy, (3, 3), **kw)) < 5e-3
    xh = x.astype(np.float16)
    yh = shim.conv2d_forward(xh, w.astype(np.float16), ctx=ctx, **kw)
    assert O.rel_err(yh.astype(np.float32), O.conv2d(xh.astype(np.float32), w.astype(np.float16).astype(np.float32), **kw)) < 2e-2
