"""Filters packed ahead of time (b200conv_prepack): same results as per-call packing, one launch
for many layers, stale forms are not used once the filters were reported changed."""
import numpy as np
import pytest

from oracle import corr_oracle as O
from theano_b200 import shim

pytestmark = pytest.mark.gpu

LAYERS = [((6, 32, 12, 12), (48, 32, 3, 3), dict(border_mode=(1, 1))),
          ((6, 64, 9, 9), (24, 64, 1, 1), dict(border_mode=(0, 0))),                      # 1x1: only gradInputs packs
          ((6, 16, 11, 11), (32, 16, 3, 3), dict(border_mode=(1, 1), subsample=(2, 2))),
          ((4, 32, 8, 8), (64, 8, 3, 3), dict(border_mode=(1, 1), num_groups=4))]


@pytest.fixture(scope="module")
def ctx():
    return shim.Context(0)          # its own context: the packed forms live in it


@pytest.mark.parametrize("dtype", [np.float16, np.float32], ids=["float16", "float32"])
def test_prepacked_filters_give_the_same_results_with_fewer_launches(ctx, dtype):
    tol = 2e-2 if dtype == np.float16 else 5e-3
    rs = np.random.RandomState(4)
    T = shim.DeviceTensor
    descs, ptrs, cases = [], [], []
    for xs, ws, kw in LAYERS:
        x = rs.standard_normal(xs).astype(dtype)
        w = (rs.standard_normal(ws) * 0.1).astype(dtype)
        X, W = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w)
        y = shim.device_conv2d(X, W, **kw)
        dy = (rs.standard_normal(y.shape) * 0.1).astype(dtype)
        DY = T.from_host(ctx, dy, "nhwc")
        descs.append(shim.layer_desc(xs, ws, dtype=dtype, **kw))
        ptrs.append(W.ptr)
        cases.append((x, w, dy, X, W, DY, kw))

    def run_all():
        n0 = ctx.launches
        outs = []
        for x, w, dy, X, W, DY, kw in cases:
            outs.append((shim.device_conv2d(X, W, **kw).to_host(), shim.device_grad_inputs(W, DY, x.shape[2:], **kw).to_host()))
        return outs, ctx.launches - n0

    plain, n_plain = run_all()
    n0 = ctx.launches
    ctx.prepack(descs, ptrs)
    assert ctx.launches - n0 == 1                       # one launch packs every bank of one data type
    packed, n_packed = run_all()
    assert n_packed < n_plain
    for (y0, dx0), (y1, dx1), (x, w, dy, X, W, DY, kw) in zip(plain, packed, cases):
        assert np.array_equal(y0, y1) and np.array_equal(dx0, dx1)
        xf, wf, dyf = (a.astype(np.float32) for a in (x, w, dy))
        assert O.rel_err(y1.astype(np.float32), O.conv2d(xf, wf, **kw)) < tol
        assert O.rel_err(dx1.astype(np.float32), O.conv2d_grad_inputs(wf, dyf, x.shape[2:], **kw)) < tol
    # new filters in the same buffer: reported -> packed per call again -> right; prepack -> right and cheap again
    x, w, dy, X, W, DY, kw = cases[0]
    w2 = (rs.standard_normal(w.shape) * 0.1).astype(dtype)
    ctx.h2d(W.ptr, w2)
    ctx.sync()
    ctx.filters_changed(W.ptr)
    want = O.conv2d(x.astype(np.float32), w2.astype(np.float32), **kw)
    assert O.rel_err(shim.device_conv2d(X, W, **kw).to_host().astype(np.float32), want) < tol
    ctx.prepack(descs[:1], ptrs[:1])
    n0 = ctx.launches
    got = shim.device_conv2d(X, W, **kw).to_host()
    assert O.rel_err(got.astype(np.float32), want) < tol
    ctx.filters_changed()
