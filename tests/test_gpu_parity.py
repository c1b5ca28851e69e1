"""GPU parity tests: the CUDA path, called through the C ABI, against outputs of the
reference itself (golden fixtures) and against the CPU oracle on the same seeded inputs.

Error measure everywhere: max|a - b| / max|b|.  Tolerances: 5e-3 for float32 (the tensor
cores multiply in TF32), 2e-2 for float16, and 1e-4 / 2e-3 for the CUDA-core direct kernels
(float32 arithmetic, one rounding to the storage type).
"""
import numpy as np
import pytest

import cases as C
from oracle import corr_oracle as O
from theano_b200 import hostlogic, shim

pytestmark = pytest.mark.gpu

TOL_F32, TOL_F16 = 5e-3, 2e-2
CASES = C.all_cases()
NONEMPTY = [c for c in CASES if min(c["x"]) > 0 and min(c["w"]) > 0]


@pytest.fixture(scope="module")
def ctx():
    return shim.get_context(0)


def kwargs(c):
    return dict(border_mode=c["border"], subsample=c["sub"], filter_dilation=c["dil"],
                num_groups=c["groups"], filter_flip=c["flip"])


def tensor_core_expected(c):
    """float32: the tensor-core kernels take ungrouped layers, and grouped ones whose channel
    counts per group are multiples of 4 after neighbouring small groups have been merged."""
    g, cg, kg = c["groups"], c["w"][1], c["w"][0] // c["groups"]
    m = max([q for q in range(1, g + 1) if g % q == 0 and (q == 1 or (cg * q <= 32 and kg * q <= 256))])
    return g // m == 1 or ((cg * m) % 4 == 0 and (kg * m) % 4 == 0)


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_float32_against_reference_outputs(c, golden, ctx):
    x, w, dy = C.make_inputs(c)
    kw = kwargs(c)
    s = c["sample"]
    y = shim.conv2d_forward(x, w, ctx=ctx, **kw)
    if y.size and x.shape[1]:
        assert ctx.last_algo == ("umma" if tensor_core_expected(c) else "direct")
    dx = shim.conv2d_grad_inputs(w, dy, x.shape[2:], ctx=ctx, **kw)
    dw = shim.conv2d_grad_weights(x, dy, w.shape[2:], ctx=ctx, **kw)
    assert O.rel_err(C.sampled(y, s), golden[c["name"] + "/y"]) < TOL_F32
    assert O.rel_err(C.sampled(dx, s), golden[c["name"] + "/dx"]) < TOL_F32
    assert O.rel_err(dw, golden[c["name"] + "/dw"]) < TOL_F32


@pytest.mark.parametrize("c", NONEMPTY[::3], ids=[c["name"] for c in NONEMPTY[::3]])
def test_direct_kernels_against_reference_outputs(c, golden, ctx):
    x, w, dy = C.make_inputs(c)
    kw = kwargs(c)
    s = c["sample"]
    f = shim.FORCE_DIRECT
    assert O.rel_err(C.sampled(shim.conv2d_forward(x, w, ctx=ctx, flags=f, **kw), s), golden[c["name"] + "/y"]) < 1e-4
    assert ctx.last_algo == "direct"
    assert O.rel_err(C.sampled(shim.conv2d_grad_inputs(w, dy, x.shape[2:], ctx=ctx, flags=f, **kw), s),
                     golden[c["name"] + "/dx"]) < 1e-4
    assert O.rel_err(shim.conv2d_grad_weights(x, dy, w.shape[2:], ctx=ctx, flags=f, **kw), golden[c["name"] + "/dw"]) < 1e-4


@pytest.mark.parametrize("c", NONEMPTY[::2], ids=[c["name"] for c in NONEMPTY[::2]])
def test_float16_against_oracle(c, ctx):
    """float16 has no CPU path in the reference (nnet/opt.py:74); the oracle runs in float32 on
    the float16-rounded inputs, the convention of the reference's GPU tests
    (gpuarray/tests/config.py:36-40)."""
    x, w, dy = C.make_inputs(c, np.float16)
    kw = kwargs(c)
    xf, wf, dyf = x.astype(np.float32), w.astype(np.float32), dy.astype(np.float32)
    y = shim.conv2d_forward(x, w, ctx=ctx, **kw)
    assert y.dtype == np.float16
    assert O.rel_err(y, O.conv2d(xf, wf, **kw)) < TOL_F16
    assert O.rel_err(shim.conv2d_grad_inputs(w, dy, x.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_inputs(wf, dyf, x.shape[2:], **kw)) < TOL_F16
    assert O.rel_err(shim.conv2d_grad_weights(x, dy, w.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_weights(xf, dyf, w.shape[2:], **kw)) < TOL_F16


# Shapes that exercise tiling corners the small matrix cannot: several filter tiles, several
# channel blocks per tap, ragged channel counts, accumulators wider than one TMA box.
MEDIUM = [
    dict(x=(5, 160, 14, 14), w=(320, 160, 3, 3), border=(1, 1), sub=(1, 1), dil=(1, 1), groups=1),
    dict(x=(3, 72, 19, 17), w=(136, 72, 3, 3), border="half", sub=(2, 2), dil=(1, 1), groups=1),
    dict(x=(2, 192, 9, 9), w=(96, 192, 1, 1), border="valid", sub=(1, 1), dil=(1, 1), groups=1),
    dict(x=(2, 64, 12, 12), w=(64, 16, 3, 3), border=(2, 2), sub=(1, 1), dil=(2, 2), groups=4),
    dict(x=(2, 40, 21, 21), w=(24, 40, 5, 5), border="full", sub=(3, 2), dil=(1, 1), groups=1),
    dict(x=(130, 8, 7, 7), w=(8, 8, 3, 3), border="half", sub=(1, 1), dil=(1, 1), groups=1),
]


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("m", MEDIUM, ids=["k320", "ragged_s2", "1x1", "g4_dil2", "full_s32", "n130"])
def test_medium_shapes_against_oracle(m, dtype, ctx):
    rs = np.random.RandomState(11)
    x = rs.standard_normal(m["x"]).astype(dtype)
    fan = m["w"][1] * m["w"][2] * m["w"][3]
    w = (rs.standard_normal(m["w"]) * np.sqrt(2.0 / fan)).astype(dtype)
    kw = dict(border_mode=m["border"], subsample=m["sub"], filter_dilation=m["dil"], num_groups=m["groups"],
              filter_flip=True)
    xf, wf = x.astype(np.float32), w.astype(np.float32)
    yo = O.conv2d(xf, wf, **kw)
    dy = rs.standard_normal(yo.shape).astype(dtype)
    dyf = dy.astype(np.float32)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    assert O.rel_err(shim.conv2d_forward(x, w, ctx=ctx, **kw), yo) < tol
    assert ctx.last_algo == "umma"
    assert O.rel_err(shim.conv2d_grad_inputs(w, dy, x.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_inputs(wf, dyf, x.shape[2:], **kw)) < tol
    assert O.rel_err(shim.conv2d_grad_weights(x, dy, w.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_weights(xf, dyf, w.shape[2:], **kw)) < tol
    assert O.rel_err(shim.conv2d_grad_weights(x, dy, w.shape[2:], ctx=ctx, flags=shim.ATOMIC_SPLITK, **kw),
                     O.conv2d_grad_weights(xf, dyf, w.shape[2:], **kw)) < tol


def test_fused_bias_relu_and_pool(golden, ctx):
    c = [k for k in CASES if k["name"] == "cfg2_small"][0]
    x, w, _ = C.make_inputs(c)
    b = golden["epilogue/bias"]
    act = shim.conv2d_forward(x, w, border_mode=c["border"], bias=b, relu=True, ctx=ctx)
    assert O.rel_err(C.sampled(act, c["sample"]), golden["epilogue/act"]) < TOL_F32
    assert (act >= 0).all()
    pooled = shim.maxpool2x2(act, ctx=ctx)
    assert np.array_equal(pooled, O.maxpool2x2(act))           # max pooling is exact
    assert O.rel_err(pooled, golden["epilogue/pool"]) < TOL_F32


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("shape", [((3, 40, 14, 14), (64, 40, 3, 3), (1, 1), 1),       # slab kernel
                                   ((2, 32, 15, 13), (48, 32, 3, 3), "half", 2),       # per-tap kernel (stride 2)
                                   ((2, 3, 9, 9), (5, 3, 2, 2), "valid", 1)],          # direct kernel
                         ids=["slab", "pertap", "direct"])
def test_fused_scale_residual_leaky_relu(shape, dtype, ctx):
    """y = leaky(alpha * conv + bias + beta * residual) in the kernels' epilogues, host (NCHW) and
    device (channels-last) forms, against the restatement applied to the oracle's convolution."""
    xs, ws, border, stride = shape
    rs = np.random.RandomState(21)
    x = rs.standard_normal(xs).astype(dtype)
    w = (rs.standard_normal(ws) * 0.2).astype(dtype)
    b = rs.standard_normal(ws[0]).astype(dtype)
    kw = dict(border_mode=border, subsample=(stride, stride))
    conv = O.conv2d(x.astype(np.float32), w.astype(np.float32), **kw)
    res = rs.standard_normal(conv.shape).astype(dtype)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    for epi in (dict(alpha=0.5, beta=2.0, relu=True, slope=0.1, bias=b, residual=res),
                dict(alpha=1.0, beta=1.0, relu=False, slope=0.0, bias=None, residual=res),
                dict(alpha=-1.5, beta=1.0, relu=True, slope=0.25, bias=b, residual=None)):
        want = O.epilogue(conv, epi["bias"], None if epi["residual"] is None else epi["residual"].astype(np.float32),
                          epi["alpha"], epi["beta"], epi["relu"], epi["slope"])
        got = shim.conv2d_forward(x, w, ctx=ctx, **kw, **epi)
        assert O.rel_err(got, want) < tol
        if xs[1] * np.dtype(dtype).itemsize % 4 == 0 and ws[0] >= 8:    # tensor-core geometries: device form
            T = shim.DeviceTensor
            X, W = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w)
            B = T.from_host(ctx, epi["bias"].reshape(1, -1, 1, 1)) if epi["bias"] is not None else None
            R = T.from_host(ctx, epi["residual"], "nhwc") if epi["residual"] is not None else None
            Y = shim.device_conv2d(X, W, bias=B, residual=R, alpha=epi["alpha"], beta=epi["beta"],
                                   relu=epi["relu"], slope=epi["slope"], **kw)
            assert O.rel_err(Y.to_host(), want) < tol
    with pytest.raises(ValueError):
        shim.conv2d_forward(x, w, ctx=ctx, residual=res[:, :, :-1], **kw)


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("geom", [
    ((3, 3, 23, 20), (16, 3, 7, 7), (3, 3), (2, 2), (1, 1)),      # the stem shape, odd image
    ((2, 8, 17, 17), (24, 8, 3, 3), "half", (2, 2), (1, 1)),
    ((2, 4, 19, 22), (16, 4, 5, 4), (2, 1), (3, 2), (1, 1)),      # stride 3 x 2, even filter width
    ((2, 5, 16, 16), (8, 5, 3, 3), "full", (2, 2), (2, 1)),       # dilation beside the stride
    ((2, 16, 9, 9), (8, 16, 1, 1), "valid", (2, 2), (1, 1)),      # 1x1: three of four classes have no tap
], ids=["stem", "half", "s3x2", "dil", "1x1"])
def test_strided_grad_inputs_with_merged_parity_classes(geom, dtype, ctx):
    """Few channels and a stride: the parity classes run as one launch plus depth-to-space.  Same
    values as the oracle, as one launch per class, in NCHW and channels-last form."""
    xs, ws, border, sub, dil = geom
    rs = np.random.RandomState(33)
    kw = dict(border_mode=border, subsample=sub, filter_dilation=dil)
    w = (rs.standard_normal(ws) * 0.3).astype(dtype)
    yshape, _ = hostlogic.forward_shape(xs, ws, border, sub, dil, 1)
    dy = rs.standard_normal(yshape).astype(dtype)
    want = O.conv2d_grad_inputs(w.astype(np.float32), dy.astype(np.float32), xs[2:], **kw)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    got = shim.conv2d_grad_inputs(w, dy, xs[2:], ctx=ctx, flags=shim.FORCE_UMMA, **kw)
    assert got.shape == tuple(xs) and O.rel_err(got, want) < tol
    per_class = shim.conv2d_grad_inputs(w, dy, xs[2:], ctx=ctx, flags=shim.FORCE_UMMA | shim.NO_MERGE_PARITY, **kw)
    assert O.rel_err(got, per_class) < tol
    T = shim.DeviceTensor
    DX = shim.device_grad_inputs(T.from_host(ctx, w), T.from_host(ctx, dy, "nhwc"), xs[2:], **kw)
    assert DX.layout == "nhwc" and O.rel_err(DX.to_host(), want) < tol


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("geom", [
    ((3, 3, 46, 40), (64, 3, 7, 7), (3, 3)),          # the ResNet stem shape in small
    ((2, 3, 23, 21), (16, 3, 7, 7), (3, 3)),          # odd image: a half-filled last block row / column
    ((2, 3, 17, 18), (24, 3, 3, 3), (1, 1)),
    ((2, 4, 20, 20), (40, 4, 5, 5), "half"),
    ((2, 1, 19, 16), (8, 1, 7, 5), "valid"),
    ((2, 2, 16, 14), (8, 2, 4, 6), "full"),           # even filter sides: 6 columns from -5 span 4 blocks
    ((3, 3, 12, 12), (300, 3, 2, 2), "valid"),        # more filters than one accumulator holds
], ids=["stem", "odd", "3x3", "5x5", "c1", "full", "k300"])
def test_stride2_forward_with_pixel_blocks_as_channels(geom, dtype, ctx):
    """Stride 2 and at most 4 channels: 2 x 2 pixel blocks become channels and the layer runs as a
    stride-1 layer.  Same values as the oracle and as the path that keeps the pixels as they are,
    with and without the filter flip, for NCHW host arrays and channels-last device tensors, with
    the fused bias + ReLU."""
    xs, ws, border = geom
    rs = np.random.RandomState(51)
    x = rs.standard_normal(xs).astype(dtype)
    w = (rs.standard_normal(ws) * 0.2).astype(dtype)
    b = rs.standard_normal(ws[0]).astype(dtype)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    for flip in (True, False):
        kw = dict(border_mode=border, subsample=(2, 2), filter_flip=flip)
        want = O.conv2d(x.astype(np.float32), w.astype(np.float32), **kw)
        got = shim.conv2d_forward(x, w, ctx=ctx, flags=shim.FORCE_UMMA, **kw)
        assert got.shape == want.shape and O.rel_err(got, want) < tol
        plain = shim.conv2d_forward(x, w, ctx=ctx, flags=shim.FORCE_UMMA | shim.NO_S2D, **kw)
        assert O.rel_err(got, plain) < tol
        per_tap = shim.conv2d_forward(x, w, ctx=ctx, flags=shim.FORCE_UMMA | shim.NO_SLAB, **kw)
        assert O.rel_err(per_tap, want) < tol
    T = shim.DeviceTensor
    kw = dict(border_mode=border, subsample=(2, 2))
    want = O.bias_relu(O.conv2d(x.astype(np.float32), w.astype(np.float32), **kw), b.astype(np.float32), relu=True)
    Y = shim.device_conv2d(T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), bias=T.from_host(ctx, b.reshape(1, -1, 1, 1)),
                           relu=True, **kw)
    assert Y.layout == "nhwc" and O.rel_err(Y.to_host(), want) < tol


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
@pytest.mark.parametrize("geom", [
    ((3, 3, 46, 40), (64, 3, 7, 7), (3, 3)),
    ((2, 3, 23, 21), (16, 3, 7, 7), (3, 3)),
    ((2, 4, 20, 20), (40, 4, 5, 5), "half"),
    ((2, 2, 16, 14), (8, 2, 4, 6), "full"),
    ((3, 3, 12, 12), (300, 3, 2, 2), "valid"),
    ((40, 3, 30, 30), (16, 3, 3, 3), (1, 1)),         # enough pixels for several split-K slices
], ids=["stem", "odd", "5x5", "full", "k300", "splitk"])
def test_stride2_grad_weights_with_pixel_blocks_as_channels(geom, dtype, ctx):
    """gradWeights of the same layers: the image operand with 2 x 2 pixel blocks as channels, the
    result put back into filter order.  Same values as the oracle and as the path that keeps the
    pixels as they are; repeated calls are bit-identical."""
    xs, ws, border = geom
    rs = np.random.RandomState(52)
    x = rs.standard_normal(xs).astype(dtype)
    yshape, _ = hostlogic.forward_shape(xs, ws, border, (2, 2), (1, 1), 1)
    dy = (rs.standard_normal(yshape) * 0.25).astype(dtype)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    for flip in (True, False):
        kw = dict(border_mode=border, subsample=(2, 2), filter_flip=flip)
        want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), ws[2:], **kw)
        got = shim.conv2d_grad_weights(x, dy, ws[2:], ctx=ctx, flags=shim.FORCE_UMMA, **kw)
        assert got.shape == tuple(ws) and O.rel_err(got, want) < tol
        plain = shim.conv2d_grad_weights(x, dy, ws[2:], ctx=ctx, flags=shim.FORCE_UMMA | shim.NO_S2D, **kw)
        assert O.rel_err(got, plain) < tol
        again = shim.conv2d_grad_weights(x, dy, ws[2:], ctx=ctx, flags=shim.FORCE_UMMA, **kw)
        assert np.array_equal(got, again)
    T = shim.DeviceTensor
    kw = dict(border_mode=border, subsample=(2, 2))
    want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), ws[2:], **kw)
    DW = shim.device_grad_weights(T.from_host(ctx, x, "nhwc"), T.from_host(ctx, dy, "nhwc"), ws[2:], **kw)
    assert O.rel_err(DW.to_host(), want) < tol


def test_background_copies_and_image_views(ctx):
    """Uploads and downloads on the background streams, the batch in two halves through views of
    the device tensors (what the end-to-end leg of the benchmark does): same values as whole-batch
    calls and as the oracle."""
    rs = np.random.RandomState(41)
    N, C, K, H = 6, 32, 48, 12
    x = rs.standard_normal((N, C, H, H)).astype(np.float32)
    w = (rs.standard_normal((K, C, 3, 3)) * 0.1).astype(np.float32)
    kw = dict(border_mode=(1, 1))
    T = shim.DeviceTensor
    xh, yh = ctx.pinned_empty(x.shape, np.float32), ctx.pinned_empty((N, K, H, H), np.float32)
    xh[...] = x
    Xn, X = T(ctx, x.shape, np.float32, "nchw"), T(ctx, x.shape, np.float32, "nhwc")
    Wd, Yn = T.from_host(ctx, w), T(ctx, (N, K, H, H), np.float32, "nchw")
    parts = [(0, 4), (4, 6)]
    ctx.h2d_bg(Xn.images(*parts[0]).ptr, xh[0:4])
    for k, (a, b) in enumerate(parts):
        ctx.join_uploads()
        if k == 0:
            ctx.h2d_bg(Xn.images(*parts[1]).ptr, xh[4:6])
        ctx.nchw_to_nhwc(Xn.images(a, b).ptr, X.images(a, b).ptr, b - a, C, H, H, np.float32)
        shim.device_conv2d(X.images(a, b), Wd, out=Yn.images(a, b), **kw)
        ctx.d2h_bg(yh[a:b], Yn.images(a, b).ptr)
    ctx.sync()
    want = O.conv2d(x, w, **kw)
    assert O.rel_err(np.array(yh), want) < TOL_F32
    assert O.rel_err(X.to_host(), x) == 0.0
    with pytest.raises(ValueError):
        X.images(4, 9)


def test_causal_conv_known_answer_on_gpu(golden, ctx):
    """The literal triple of the reference's TestCausalConv (test_abstract_conv.py:2081-2102):
    left padding only, kernels one column wide, dilation along the sequence."""
    img, kern, top = golden["causal/img"], golden["causal/kern"], golden["causal/precomp_top"]
    d = int(golden["causal/dilation"])
    left = d * (kern.shape[2] - 1)
    kw = dict(border_mode=((left, 0), 0), filter_dilation=(d, 1), filter_flip=True)
    y = shim.conv2d_forward(img[:, :, :, None], kern[:, :, :, None], ctx=ctx, **kw)
    assert O.rel_err(y[:, :, :, 0], top) < TOL_F32
    dy = np.random.RandomState(3).standard_normal(y.shape).astype(np.float32)
    x4, k4 = np.ascontiguousarray(img[:, :, :, None]), np.ascontiguousarray(kern[:, :, :, None])
    assert O.rel_err(shim.conv2d_grad_inputs(k4, dy, x4.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_inputs(k4, dy, x4.shape[2:], **kw)) < TOL_F32
    assert O.rel_err(shim.conv2d_grad_weights(x4, dy, k4.shape[2:], ctx=ctx, **kw),
                     O.conv2d_grad_weights(x4, dy, k4.shape[2:], **kw)) < TOL_F32


@pytest.mark.parametrize("name", ["even", "odd", "ties", "wide"])
def test_pool_gradient_against_reference_outputs(pool_golden, name, ctx):
    x, y, gy, gx = (pool_golden["%s/%s" % (name, k)] for k in ("x", "y", "gy", "gx"))
    assert np.array_equal(shim.maxpool2x2(x, ctx=ctx), y)
    assert np.array_equal(shim.maxpool2x2_grad(x, y, gy, ctx=ctx), gx)        # exact, ties included
    # float16 and the channels-last device form give the same answer as the restatement
    xh, gyh = x.astype(np.float16), gy.astype(np.float16)
    yh = O.maxpool2x2(xh).astype(np.float16)          # exact: the maximum of float16 values
    assert np.array_equal(shim.maxpool2x2_grad(xh, yh, gyh, ctx=ctx), O.maxpool2x2_grad(xh, yh, gyh))
    T = shim.DeviceTensor
    X, GY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, gy, "nhwc")
    Y = shim.device_maxpool2x2(X)
    GX = shim.device_maxpool2x2_grad(X, Y, GY)
    assert np.array_equal(GX.to_host(), gx)
    with pytest.raises(ValueError):
        shim.maxpool2x2_grad(x, y[:, :, :-1], gy[:, :, :-1], ctx=ctx)


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
def test_device_resident_chain_channels_last(dtype, ctx):
    """conv+bias+ReLU -> pool -> conv with activations kept on the GPU in channels-last order."""
    rs = np.random.RandomState(5)
    x = rs.uniform(0, 1, (3, 3, 20, 20)).astype(dtype)
    w1 = (rs.standard_normal((24, 3, 3, 3)) * np.sqrt(2.0 / 27)).astype(dtype)
    b1 = (rs.standard_normal(24) * 0.1).astype(dtype)
    w2 = (rs.standard_normal((40, 24, 3, 3)) * np.sqrt(2.0 / 216)).astype(dtype)
    X = shim.DeviceTensor.from_host(ctx, x, "nhwc")
    W1 = shim.DeviceTensor.from_host(ctx, w1)
    B1 = shim.DeviceTensor.from_host(ctx, b1.reshape(1, -1, 1, 1))
    W2 = shim.DeviceTensor.from_host(ctx, w2)
    a1 = shim.device_conv2d(X, W1, border_mode="half", bias=B1, relu=True)
    p1 = shim.device_maxpool2x2(a1)
    a2 = shim.device_conv2d(p1, W2, border_mode="half", relu=True, out_layout="nchw")
    got = a2.to_host()
    f = np.float32
    r1 = O.bias_relu(O.conv2d(x.astype(f), w1.astype(f), border_mode="half"), b1.astype(f), relu=True)
    if dtype == np.float16:
        r1 = r1.astype(np.float16).astype(f)
    r2 = O.bias_relu(O.conv2d(O.maxpool2x2(r1), w2.astype(f), border_mode="half"), None, relu=True)
    assert O.rel_err(got, r2) < (TOL_F32 if dtype == np.float32 else TOL_F16)
    # gradients with channels-last operands
    dy = rs.standard_normal(a2.shape).astype(dtype)
    DY = shim.DeviceTensor.from_host(ctx, dy, "nhwc")
    dx = shim.device_grad_inputs(W2, DY, p1.shape[2:], border_mode="half").to_host()
    dw = shim.device_grad_weights(p1, DY, (3, 3), border_mode="half").to_host()
    p1h = p1.to_host().astype(f)
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    assert O.rel_err(dx, O.conv2d_grad_inputs(w2.astype(f), dy.astype(f), p1.shape[2:], border_mode="half")) < tol
    assert O.rel_err(dw, O.conv2d_grad_weights(p1h, dy.astype(f), (3, 3), border_mode="half")) < tol


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["f32", "f16"])
def test_channels_last_wide_outputs(dtype, ctx):
    """Channels-last outputs with 32 or more channels per group take the row-wise store path of
    the epilogue (whole pixel rows per store instruction); forward and gradInputs, with bias."""
    rs = np.random.RandomState(8)
    f = np.float32
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    for (N, Cc, K, H, W, g) in ((3, 64, 96, 13, 11, 1), (2, 64, 128, 9, 9, 2), (2, 40, 320, 7, 7, 1)):
        x = rs.standard_normal((N, Cc, H, W)).astype(dtype)
        w = (rs.standard_normal((K, Cc // g, 3, 3)) * np.sqrt(2.0 / (Cc // g * 9))).astype(dtype)
        b = rs.standard_normal(K).astype(dtype)
        kw = dict(border_mode="half", num_groups=g)
        X = shim.DeviceTensor.from_host(ctx, x, "nhwc")
        Wd = shim.DeviceTensor.from_host(ctx, w)
        B = shim.DeviceTensor.from_host(ctx, b.reshape(1, -1, 1, 1))
        y = shim.device_conv2d(X, Wd, bias=B, relu=True, out_layout="nhwc", **kw).to_host()
        ref = O.bias_relu(O.conv2d(x.astype(f), w.astype(f), **kw), b.astype(f), relu=True)
        assert O.rel_err(y, ref) < tol
        dy = rs.standard_normal(ref.shape).astype(dtype)
        DY = shim.DeviceTensor.from_host(ctx, dy, "nhwc")
        dx = shim.device_grad_inputs(Wd, DY, (H, W), out_layout="nhwc", **kw).to_host()
        assert O.rel_err(dx, O.conv2d_grad_inputs(w.astype(f), dy.astype(f), (H, W), **kw)) < tol
        # the per-tap kernel on the same channels-last tensors
        y2 = shim.device_conv2d(X, Wd, bias=B, relu=True, out_layout="nhwc", flags=shim.NO_SLAB, **kw).to_host()
        assert O.rel_err(y2, ref) < tol


def test_graph_replay_matches_eager_calls(ctx):
    """fwd + gradWeights + gradInputs recorded as one CUDA graph; replays follow the data."""
    rs = np.random.RandomState(12)
    x = rs.standard_normal((6, 32, 14, 14)).astype(np.float32)
    w = (rs.standard_normal((48, 32, 3, 3)) * 0.1).astype(np.float32)
    dy = rs.standard_normal((6, 48, 14, 14)).astype(np.float32)
    T = shim.DeviceTensor
    X, Wd, DY = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), T.from_host(ctx, dy, "nhwc")
    Y, DX, DW = T(ctx, dy.shape, np.float32, "nhwc"), T(ctx, x.shape, np.float32, "nhwc"), T(ctx, w.shape, np.float32)
    kw = dict(border_mode="half")

    def step():
        shim.device_conv2d(X, Wd, out=Y, **kw)
        shim.device_grad_weights(X, DY, (3, 3), out=DW, **kw)
        shim.device_grad_inputs(Wd, DY, (14, 14), out=DX, **kw)

    step()
    ctx.sync()
    eager = [t.to_host() for t in (Y, DX, DW)]
    n0 = ctx.launches
    g = ctx.capture(step)
    per_graph = ctx.launches - n0
    assert per_graph >= 5
    for t in (Y, DX, DW):
        ctx.memset(t.ptr, 0, t.nbytes)
    g.launch()
    assert ctx.launches - n0 == 2 * per_graph
    for a, b in zip(eager, (Y, DX, DW)):
        assert np.array_equal(a, b.to_host())
    # new data in the same buffers: the replay computes on it
    x2 = rs.standard_normal(x.shape).astype(np.float32)
    X2 = T.from_host(ctx, x2, "nhwc")
    ctx.check(ctx.lib.b200conv_memcpy_h2d(ctx.h, X.ptr, X2.to_layout("nhwc").ptr, 0))  # no-op copy keeps API use honest
    tmp = X2.to_host()
    ctx.h2d(X.ptr, np.ascontiguousarray(np.transpose(tmp, (0, 2, 3, 1))))
    g.launch()
    assert O.rel_err(Y.to_host(), O.conv2d(x2, w, **kw)) < TOL_F32
    with pytest.raises(ValueError):
        ctx.capture(lambda: shim.conv2d_forward(x, w, ctx=ctx))       # host-pointer calls are refused
    g.destroy()


def test_full_size_layer_properties(ctx):
    """The benchmark layer (N=128, 256->256, 14x14, 3x3 pad 1) at full size: tensor-core result
    equals the direct kernels' on the device, and the three directions satisfy the adjoint
    identity <conv(x,w), dy> = <x, gradInputs(w,dy)> = <w, gradWeights(x,dy)>."""
    rs = np.random.RandomState(1235)
    N, Cc, K, H = 128, 256, 256, 14
    x = rs.standard_normal((N, Cc, H, H)).astype(np.float32)
    w = (rs.standard_normal((K, Cc, 3, 3)) * np.sqrt(2.0 / (Cc * 9))).astype(np.float32)
    dy = rs.standard_normal((N, K, H, H)).astype(np.float32)
    kw = dict(border_mode=(1, 1), filter_flip=True)
    y = shim.conv2d_forward(x, w, ctx=ctx, **kw)
    assert ctx.last_algo == "umma"
    dx = shim.conv2d_grad_inputs(w, dy, (H, H), ctx=ctx, **kw)
    dw = shim.conv2d_grad_weights(x, dy, (3, 3), ctx=ctx, **kw)
    f = shim.FORCE_DIRECT
    assert O.rel_err(y, shim.conv2d_forward(x, w, ctx=ctx, flags=f, **kw)) < TOL_F32
    assert O.rel_err(dx, shim.conv2d_grad_inputs(w, dy, (H, H), ctx=ctx, flags=f, **kw)) < TOL_F32
    assert O.rel_err(dw, shim.conv2d_grad_weights(x, dy, (3, 3), ctx=ctx, flags=f, **kw)) < TOL_F32
    a = float(np.vdot(y.astype(np.float64), dy))
    b = float(np.vdot(dx.astype(np.float64), x))
    c = float(np.vdot(dw.astype(np.float64), w))
    scale = np.sqrt(float(np.vdot(y, y)) * float(np.vdot(dy, dy)))
    assert abs(a - b) / scale < 1e-3 and abs(a - c) / scale < 1e-3
    # two runs give bit-identical filter gradients (ordered split-K reduction)
    assert np.array_equal(dw, shim.conv2d_grad_weights(x, dy, (3, 3), ctx=ctx, **kw))
    # and the oracle agrees on a slice of the batch
    assert O.rel_err(y[:4], O.conv2d(x[:4], w, **kw)) < TOL_F32


def test_linearity_large(ctx):
    """conv(a*x1 + x2, w) = a*conv(x1, w) + conv(x2, w) on a VGG-sized layer slice."""
    rs = np.random.RandomState(3)
    x1 = rs.standard_normal((4, 64, 112, 112)).astype(np.float32)
    x2 = rs.standard_normal((4, 64, 112, 112)).astype(np.float32)
    w = (rs.standard_normal((64, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(np.float32)
    y1 = shim.conv2d_forward(x1, w, border_mode="half", ctx=ctx)
    y2 = shim.conv2d_forward(x2, w, border_mode="half", ctx=ctx)
    y3 = shim.conv2d_forward(2 * x1 + x2, w, border_mode="half", ctx=ctx)
    assert O.rel_err(y3, 2 * y1 + y2) < TOL_F32


def test_noncontiguous_and_mixed_dtype_inputs(ctx):
    rs = np.random.RandomState(9)
    x = rs.standard_normal((2, 6, 9, 9)).astype(np.float32)
    w = rs.standard_normal((4, 6, 3, 3)).astype(np.float32)
    wv = w[:, :, ::-1, ::-1]                                     # the view the lowering inserts
    assert not wv.flags.c_contiguous
    a = shim.conv2d_forward(x, wv, filter_flip=False, ctx=ctx)
    b = shim.conv2d_forward(x, w, filter_flip=True, ctx=ctx)
    assert O.rel_err(a, b) < 1e-6
    y = shim.conv2d_forward(x.astype(np.float16), w, ctx=ctx)    # upcast to the common dtype
    assert y.dtype == np.float32
    with pytest.raises(TypeError):
        shim.conv2d_forward(x.astype(np.float64), w, ctx=ctx)    # float64 is not taken over


def test_errors_and_empty_tensors(ctx):
    x = np.zeros((2, 3, 5, 5), np.float32)
    with pytest.raises(ValueError):
        shim.conv2d_forward(x, np.zeros((4, 2, 3, 3), np.float32), ctx=ctx)
    with pytest.raises(ValueError):
        shim.conv2d_forward(x, np.zeros((4, 3, 7, 7), np.float32), ctx=ctx)
    with pytest.raises(ValueError):
        shim.conv2d_grad_inputs(np.zeros((4, 3, 3, 3), np.float32), np.zeros((2, 4, 3, 3), np.float32), (9, 9), ctx=ctx)
    with pytest.raises(ValueError):
        shim.conv2d_grad_weights(x, np.zeros((2, 4, 3, 3), np.float32), None, subsample=(2, 2), ctx=ctx)
    # the C ABI itself rejects an inconsistent descriptor
    d = shim.make_desc((2, 3, 5, 5), (4, 3, 3, 3), (2, 4, 4, 4), ((0, 0), (0, 0)), (1, 1), (1, 1), 1, 1, np.float32)
    y = np.zeros((2, 4, 4, 4), np.float32)
    with pytest.raises(ValueError):
        ctx.fwd(d, x.ctypes.data, x.ctypes.data, None, y.ctypes.data, shim.HOST_PTRS)
    # zero-sized batch / channels / filters give zeros (corr_gemm.c:281-296)
    assert shim.conv2d_forward(np.zeros((0, 1, 6, 6), np.float32), np.ones((1, 1, 2, 2), np.float32), ctx=ctx).shape == (0, 1, 5, 5)
    y = shim.conv2d_forward(np.ones((1, 0, 6, 6), np.float32), np.ones((1, 0, 2, 2), np.float32), ctx=ctx)
    assert y.shape == (1, 1, 5, 5) and not y.any()
    dw = shim.conv2d_grad_weights(np.zeros((0, 1, 6, 6), np.float32), np.zeros((0, 1, 5, 5), np.float32), (2, 2), ctx=ctx)
    assert dw.shape == (1, 1, 2, 2) and not dw.any()


@pytest.mark.parametrize("dtype", [np.float32, np.float16], ids=["float32", "float16"])
@pytest.mark.parametrize("geo", [((6, 64, 28, 28), 64), ((3, 32, 20, 24), 128), ((5, 128, 14, 14), 256), ((2, 3, 32, 32), 64)],
                         ids=["64to64", "32to128", "128to256", "stem3"])
def test_pooling_fused_into_the_convolution_epilogue(ctx, geo, dtype):
    """conv + bias + ReLU + 2x2 max pooling in one kernel against the oracle's conv, bias + ReLU and
    Pool(ignore_border=True, mode='max') and against the library's own two-call form (which may run another
    kernel variant: equal up to the rounding of a different accumulation order)."""
    xs, K = geo
    tol = TOL_F32 if dtype == np.float32 else TOL_F16
    rs = np.random.RandomState(41)
    x = rs.standard_normal(xs).astype(dtype)
    w = (rs.standard_normal((K, xs[1], 3, 3)) * 0.1).astype(dtype)
    b = rs.standard_normal(K).astype(dtype)
    kw = dict(border_mode=(1, 1))
    T = shim.DeviceTensor
    X, W, B = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w), T.from_host(ctx, b.reshape(1, -1, 1, 1))
    two = shim.device_maxpool2x2(shim.device_conv2d(X, W, bias=B, relu=True, **kw)).to_host()
    try:
        fused = shim.device_conv2d(X, W, bias=B, relu=True, pool=True, **kw).to_host()
    except shim.B200Error as e:
        assert "cannot pool" in str(e) or "pooling epilogue" in str(e)
        pytest.skip("this geometry's epilogue cannot pool: %s" % e)
    want = O.maxpool2x2(O.bias_relu(O.conv2d(x.astype(np.float32), w.astype(np.float32), **kw), b.astype(np.float32), relu=True))
    assert fused.shape == want.shape
    assert O.rel_err(fused.astype(np.float32), two.astype(np.float32)) < tol / 4
    assert O.rel_err(fused.astype(np.float32), want) < tol
