"""Selection among kernel variants: every candidate the timing-based choice may pick gives the
oracle's result, the choice is remembered, and the remembered choices survive in a file.

Candidates per family: forward / gradInputs through the slab kernel or the per-tap kernel;
gradWeights with tap groups or one tap per item, each with the model's split-K slice count, half
and twice of it (and a few pinned counts).  The reference's GPU back end times its convolution
algorithms the same way (theano/gpuarray/opt.py:2144-2222)."""
import os
import tempfile

import numpy as np
import pytest

from oracle import corr_oracle as O
from theano_b200 import shim

pytestmark = pytest.mark.gpu

GEOMETRIES = [((8, 64, 14, 14), (96, 64, 3, 3), dict(border_mode=(1, 1))),                    # 3x3
              ((8, 128, 12, 12), (64, 128, 1, 1), dict(border_mode=(0, 0))),                  # 1x1 (one row of pixels)
              ((6, 32, 15, 15), (48, 32, 3, 3), dict(border_mode=(1, 1), subsample=(2, 2)))]  # stride 2


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["float32", "float16"])
@pytest.mark.parametrize("geo", GEOMETRIES, ids=["3x3", "1x1", "3x3s2"])
def test_every_candidate_equals_the_oracle(geo, dtype):
    xs, ws, kw = geo
    tol = 5e-3 if dtype == np.float32 else 2e-2
    ctx = shim.Context(0)
    ctx.set_autotune(False)
    rs = np.random.RandomState(9)
    x = rs.standard_normal(xs).astype(dtype)
    w = (rs.standard_normal(ws) * 0.1).astype(dtype)
    xf, wf = x.astype(np.float32), w.astype(np.float32)
    want_y = O.conv2d(xf, wf, **kw)
    dy = (rs.standard_normal(want_y.shape) * 0.1).astype(dtype)
    dyf = dy.astype(np.float32)
    want_dx = O.conv2d_grad_inputs(wf, dyf, xs[2:], **kw)
    want_dw = O.conv2d_grad_weights(xf, dyf, ws[2:], **kw)
    T = shim.DeviceTensor
    X, W, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), T.from_host(ctx, dy, "nhwc")
    for flags in (0, shim.NO_SLAB):
        y = shim.device_conv2d(X, W, flags=flags | shim.FORCE_UMMA, **kw).to_host().astype(np.float32)
        dx = shim.device_grad_inputs(W, DY, xs[2:], flags=flags | shim.FORCE_UMMA, **kw).to_host().astype(np.float32)
        assert O.rel_err(y, want_y) < tol and O.rel_err(dx, want_dx) < tol, flags
    for flags in (0, shim.NO_GROUP):
        for splits in (0, 1, 2, 3, 7, 1000):
            ctx.set_splits(splits)
            dw = shim.device_grad_weights(X, DY, ws[2:], flags=flags | shim.FORCE_UMMA, **kw).to_host().astype(np.float32)
            assert O.rel_err(dw, want_dw) < tol, (flags, splits)
    ctx.set_splits(0)
    with pytest.raises(ValueError):
        ctx.set_splits(-1)
    ctx.close()


def test_choices_are_remembered_and_persist():
    xs, ws, kw = GEOMETRIES[0]
    rs = np.random.RandomState(10)
    x = rs.standard_normal(xs).astype(np.float32)
    w = (rs.standard_normal(ws) * 0.1).astype(np.float32)
    dy = rs.standard_normal((xs[0], ws[0]) + xs[2:]).astype(np.float32)
    want = O.conv2d_grad_weights(x, dy, ws[2:], **kw)
    T = shim.DeviceTensor
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tuning.txt")
        a = shim.Context(0)                                  # timing-based selection is on by default
        X, W, DY = T.from_host(a, x, "nhwc"), T.from_host(a, w), T.from_host(a, dy, "nhwc")
        shim.device_conv2d(X, W, **kw)
        shim.device_grad_inputs(W, DY, xs[2:], **kw)
        first = shim.device_grad_weights(X, DY, ws[2:], **kw).to_host()
        n0 = a.launches
        again = shim.device_grad_weights(X, DY, ws[2:], **kw).to_host()
        assert a.launches - n0 <= 3                          # remembered: no candidate is timed again
        assert np.array_equal(first, again) and O.rel_err(first, want) < 5e-3
        a.tuning_save(path)
        text = open(path).read().splitlines()
        assert text[0].startswith("b200conv-tuning 1 ") and any(l.startswith("s ") for l in text) and any(l.startswith("a ") for l in text)
        b = shim.Context(0)
        assert b.tuning_load(path) == len(text) - 1
        X2, DY2 = T.from_host(b, x, "nhwc"), T.from_host(b, dy, "nhwc")
        n0 = b.launches
        got = shim.device_grad_weights(X2, DY2, ws[2:], **kw).to_host()
        assert b.launches - n0 <= 3                          # the loaded choice is used at once
        assert np.array_equal(got, first)
        open(path, "w").write("b200conv-tuning 1 some_other_device 1\n")
        with pytest.raises(ValueError):
            b.tuning_load(path)
        a.close()
        b.close()


@pytest.mark.parametrize("shape", [((8, 256, 14, 14), 512), ((3, 320, 7, 7), 256), ((5, 512, 9, 11), 320), ((1, 1024, 5, 3), 2048)],
                         ids=["256to512", "320to256", "512to320", "1024to2048"])
def test_cta_pair_kernel_equals_the_one_cta_kernel_and_the_oracle(shape):
    """1x1 float16 layers with 256+ channels run on CTA pairs (tcgen05 cta_group::2): forward with and
    without the fused bias + ReLU epilogue and gradInputs, against the one-CTA kernel (bit for bit: the
    accumulation order is the same) and the oracle; pixel counts that are no multiple of the 256-pixel
    pair tile and filter counts that are no multiple of 256 included."""
    xs, K = shape
    ctx = shim.Context(0)
    ctx.set_autotune(False)
    rs = np.random.RandomState(31)
    x = rs.standard_normal(xs).astype(np.float16)
    w = (rs.standard_normal((K, xs[1], 1, 1)) * 0.05).astype(np.float16)
    b = rs.standard_normal(K).astype(np.float16)
    xf, wf, bf = x.astype(np.float32), w.astype(np.float32), b.astype(np.float32)
    T = shim.DeviceTensor
    X, W, B = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), T.from_host(ctx, b.reshape(1, -1, 1, 1))
    want = O.conv2d(xf, wf)
    dy = (rs.standard_normal(want.shape) * 0.1).astype(np.float16)
    DY = T.from_host(ctx, dy, "nhwc")
    res = {}
    for pair in (True, False):
        ctx.set_pair_kernels(pair)
        n0 = ctx.launches
        res[pair] = (shim.device_conv2d(X, W).to_host(), shim.device_conv2d(X, W, bias=B, relu=True).to_host(),
                     shim.device_grad_inputs(W, DY, xs[2:]).to_host(),
                     shim.device_grad_weights(X, DY, (1, 1), flags=shim.NO_GROUP).to_host())
    for a, c in zip(res[True], res[False]):
        assert np.array_equal(a, c)
    assert O.rel_err(res[True][0].astype(np.float32), want) < 2e-2
    assert O.rel_err(res[True][1].astype(np.float32), O.bias_relu(want, bf, relu=True)) < 2e-2
    assert O.rel_err(res[True][2].astype(np.float32), O.conv2d_grad_inputs(wf, dy.astype(np.float32), xs[2:])) < 2e-2
    assert O.rel_err(res[True][3].astype(np.float32), O.conv2d_grad_weights(xf, dy.astype(np.float32), (1, 1))) < 2e-2
    ctx.close()


@pytest.mark.parametrize("geo", [((4, 256, 14, 14), 256, 3, 1), ((6, 512, 15, 15), 256, 3, 2), ((5, 320, 9, 9), 384, 1, 1)],
                         ids=["3x3", "3x3s2", "1x1_ragged"])
def test_cta_pair_gradweights_equals_the_one_cta_kernel_and_the_oracle(geo):
    """gradWeights of float16 layers with 256+ filters and channels on CTA pairs (256 x 256 tiles, each CTA
    loading its filters' dy rows and half of the x tile): equal to the one-CTA kernel bit for bit, with
    the ordered and the atomic split-K combination, and equal to the oracle."""
    xs, K, ks, st = geo
    ctx = shim.Context(0)
    ctx.set_autotune(False)
    rs = np.random.RandomState(32)
    pad = ks // 2
    kw = dict(border_mode=(pad, pad), subsample=(st, st))
    x = rs.standard_normal(xs).astype(np.float16)
    ho = (xs[2] + 2 * pad - ks) // st + 1
    dy = (rs.standard_normal((xs[0], K, ho, ho)) * 0.1).astype(np.float16)
    want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), (ks, ks), **kw)
    T = shim.DeviceTensor
    X, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, dy, "nhwc")
    got = {}
    for pair in (True, False):
        ctx.set_pair_kernels(pair)
        for splits in (0, 1, 3):
            ctx.set_splits(splits)
            got[pair, splits] = shim.device_grad_weights(X, DY, (ks, ks), flags=shim.NO_GROUP, **kw).to_host()
    for splits in (0, 1, 3):
        assert np.array_equal(got[True, splits], got[False, splits]), splits
        assert O.rel_err(got[True, splits].astype(np.float32), want) < 2e-2, splits
    ctx.set_pair_kernels(True)
    ctx.set_splits(2)
    a = shim.device_grad_weights(X, DY, (ks, ks), flags=shim.NO_GROUP | shim.ATOMIC_SPLITK, **kw).to_host()
    assert O.rel_err(a.astype(np.float32), want) < 2e-2
    ctx.close()


@pytest.mark.parametrize("geo", [((8, 64, 14, 14), 64, 3, 1, 1), ((5, 32, 17, 17), 96, 3, 1, 1), ((4, 64, 12, 12), 128, 5, 1, 1),
                                 ((4, 48, 16, 16), 64, 3, 1, 2), ((4, 64, 15, 15), 64, 3, 2, 1)],
                         ids=["64to64", "32to96", "5x5", "dilated", "stride2"])
def test_stacked_tap_gradweights_equals_one_mma_per_tap_and_the_oracle(geo):
    """gradWeights of float16 layers with at most 64 channels: the taps of a filter row as column groups of one
    MMA (leading-dimension offset = tap spacing) against one MMA per tap (bit for bit) and the oracle."""
    xs, K, ks, st, dil = geo
    ctx = shim.Context(0)
    ctx.set_autotune(False)
    rs = np.random.RandomState(33)
    pad = (ks // 2) * dil
    kw = dict(border_mode=(pad, pad), subsample=(st, st), filter_dilation=(dil, dil))
    x = rs.standard_normal(xs).astype(np.float16)
    ho = (xs[2] + 2 * pad - ((ks - 1) * dil + 1)) // st + 1
    dy = (rs.standard_normal((xs[0], K, ho, ho)) * 0.1).astype(np.float16)
    want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), (ks, ks), **kw)
    T = shim.DeviceTensor
    X, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, dy, "nhwc")
    got = {}
    for stacked in (True, False):
        ctx.set_stacked_taps(stacked)
        got[stacked] = shim.device_grad_weights(X, DY, (ks, ks), flags=shim.FORCE_UMMA, **kw).to_host()
    assert np.array_equal(got[True], got[False])
    assert O.rel_err(got[True].astype(np.float32), want) < 2e-2
    ctx.close()
