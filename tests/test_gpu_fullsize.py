"""GPU parity at benchmark size: every distinct layer of the benchmark configurations, at the
batch size the benchmark uses, through the same device calls the benchmark times.

Checked against the CPU oracle (the restatement of corr_gemm.c, itself pinned to outputs of the
reference) on the same seeded tensors: forward and gradInputs on a slice of the batch (they are
independent per image, corr_gemm.c:304,496), gradWeights on the whole batch (it is a reduction
over all of it, corr_gemm.c:397-455).  float16 layers: the oracle runs in float32 on the
float16-rounded inputs (the reference has no float16 CPU path; its own GPU tests compare that
way, theano/gpuarray/tests/config.py:36-40).

Error measure: max|a - b| / max|b|; tolerances 5e-3 (float32 data, TF32 multiply) and 2e-2
(float16).
"""
import numpy as np
import pytest

from oracle import corr_oracle as O
from theano_b200 import shim
from theano_b200 import workloads as WL

pytestmark = pytest.mark.gpu

TOL = {np.dtype(np.float32): 5e-3, np.dtype(np.float16): 2e-2}


@pytest.fixture(scope="module")
def ctx():
    return shim.get_context(0)


def _slice_images(n):
    """Images whose forward / gradInputs results are compared: both ends and the middle."""
    return sorted(set([0, n // 2, n - 1]))


def check_layer(ctx, lay, batch, dtype, dirs, seed, relu=False, x_dist="normal"):
    dtype = np.dtype(dtype)
    tol = TOL[dtype]
    kw = WL.conv_kwargs(lay)
    x, w, dy = WL.layer_tensors(lay, batch, dtype, seed, x_dist=x_dist)
    T = shim.DeviceTensor
    X, W = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w)
    H, ks = lay["H"], lay["k"]
    errs = {}
    imgs = _slice_images(batch)
    if "fwd" in dirs:
        bias = None
        B = None
        if relu:
            bias = WL.random_tensor(seed + 7, (lay["K"],), dtype, 0.1)
            B = T.from_host(ctx, bias.reshape(1, -1, 1, 1))
        pool = bool(lay.get("pool"))
        Y = shim.device_conv2d(X, W, bias=B, relu=relu, pool=pool, **kw)
        assert ctx.last_algo == "umma"
        for i in imgs:
            got = Y.images(i, i + 1).to_host()
            want = O.bias_relu(O.conv2d(x[i:i + 1].astype(np.float32), w.astype(np.float32), **kw),
                               None if bias is None else bias.astype(np.float32), relu=relu)
            if pool:
                want = O.maxpool2x2(want)
            errs["fwd[%d]" % i] = O.rel_err(got.astype(np.float32), want)
        Y.free()
    if "dgrad" in dirs or "wgrad" in dirs:
        DY = T.from_host(ctx, dy, "nhwc")
        if "dgrad" in dirs:
            DX = shim.device_grad_inputs(W, DY, (H, H), **kw)
            assert ctx.last_algo == "umma"
            for i in imgs:
                got = DX.images(i, i + 1).to_host()
                want = O.conv2d_grad_inputs(w.astype(np.float32), dy[i:i + 1].astype(np.float32), (H, H), **kw)
                errs["dgrad[%d]" % i] = O.rel_err(got.astype(np.float32), want)
            DX.free()
        if "wgrad" in dirs:
            DW = shim.device_grad_weights(X, DY, (ks, ks), **kw)
            assert ctx.last_algo == "umma"
            got = DW.to_host()
            want = O.conv2d_grad_weights(x.astype(np.float32), dy.astype(np.float32), (ks, ks), **kw)
            errs["wgrad"] = O.rel_err(got.astype(np.float32), want)
            DW.free()
        DY.free()
    X.free()
    W.free()
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, "%s batch %d %s: %s (tolerance %g; all: %s)" % (WL.layer_name(lay), batch, dtype.name, bad, tol, errs)
    return errs


def _ids(layers):
    return [WL.layer_name(l).replace(" ", "_") for l in layers]


@pytest.mark.parametrize("lay", WL.RESNET50, ids=_ids(WL.RESNET50))
def test_resnet50_float16_batch256(lay, ctx):
    """BASELINE config 5: the 23 distinct shapes of the 53 ResNet-50 convolutions, float16, N = 256."""
    check_layer(ctx, lay, 256, np.float16, ("fwd", "dgrad", "wgrad"), seed=5000 + WL.RESNET50.index(lay))


@pytest.mark.parametrize("lay", WL.SWEEP, ids=_ids(WL.SWEEP))
def test_sweep_float32_batch256(lay, ctx):
    """BASELINE config 4 a-d: 1x1, stride 2, dilation 2 and 32 groups, float32, N = 256."""
    check_layer(ctx, lay, 256, np.float32, ("fwd", "dgrad", "wgrad"), seed=4000 + WL.SWEEP.index(lay))


@pytest.mark.parametrize("lay", WL.VGG16, ids=_ids(WL.VGG16))
def test_vgg16_float32_batch64(lay, ctx):
    """BASELINE config 3: the 9 distinct shapes of the 13 VGG-16 convolutions with fused
    bias + ReLU, float32, N = 64."""
    check_layer(ctx, lay, 64, np.float32, ("fwd",), seed=3000 + WL.VGG16.index(lay), relu=True,
                x_dist="uniform" if lay["C"] == 3 else "normal")


def test_resnet3x3_float32_batch128_all_directions(ctx):
    """BASELINE config 2 at full size, the three directions against the oracle."""
    lay = WL.CONFIGS["cfg2"]["layers"][0]
    check_layer(ctx, lay, 128, np.float32, ("fwd", "dgrad", "wgrad"), seed=2000)


def test_vgg_block_device_resident_chain(ctx):
    """conv -> bias -> ReLU -> conv -> bias -> ReLU -> 2x2 max-pool, channels-last tensors that never
    leave the GPU between the layers (the first VGG-16 block at N = 64, 224 x 224), against the
    oracle on three images."""
    n, dtype = 64, np.float32
    l1, l2 = WL.VGG16[0], WL.VGG16[1]
    x, w1, _ = WL.layer_tensors(l1, n, dtype, 3100, x_dist="uniform")
    _, w2, _ = WL.layer_tensors(l2, 1, dtype, 3101)
    b1 = WL.random_tensor(3102, (64,), dtype, 0.1)
    b2 = WL.random_tensor(3103, (64,), dtype, 0.1)
    T = shim.DeviceTensor
    X, W1, W2 = T.from_host(ctx, x, "nhwc"), T.from_host(ctx, w1), T.from_host(ctx, w2)
    B1, B2 = T.from_host(ctx, b1.reshape(1, -1, 1, 1)), T.from_host(ctx, b2.reshape(1, -1, 1, 1))
    Y1 = shim.device_conv2d(X, W1, bias=B1, relu=True, **WL.conv_kwargs(l1))
    Y2 = shim.device_conv2d(Y1, W2, bias=B2, relu=True, **WL.conv_kwargs(l2))
    P = shim.device_maxpool2x2(Y2)
    for i in _slice_images(n):
        got = P.images(i, i + 1).to_host()
        a = O.bias_relu(O.conv2d(x[i:i + 1], w1, **WL.conv_kwargs(l1)), b1, relu=True)
        a = O.bias_relu(O.conv2d(a, w2, **WL.conv_kwargs(l2)), b2, relu=True)
        want = O.maxpool2x2(a)
        assert O.rel_err(got, want) < 5e-3, i
    for t in (X, W1, W2, B1, B2, Y1, Y2, P):
        t.free()
