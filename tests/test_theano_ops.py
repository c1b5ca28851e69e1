"""The Theano-facing layer on CPU: graph rewriting, op contracts and perform() plumbing.

These tests import the reference from its source tree (skipped when it is absent).  No GPU is
present here, so ``perform`` is exercised with the three ``theano_b200.shim`` calls replaced by
the CPU oracle: what is under test is everything above the C ABI (argument order, flip, shape
inputs, gradients built from the ops, fusion), against the reference's own CorrMM results.
"""
import pickle

import numpy as np
import pytest

import ref_theano

pytestmark = pytest.mark.skipif(not ref_theano.available(), reason="reference source tree not present")


@pytest.fixture(scope="module")
def th():
    theano = ref_theano.import_theano()
    import theano_b200.opt  # noqa: F401  (registers the optimizers)
    return theano


@pytest.fixture()
def oracle_device(monkeypatch):
    """Stand-in for the GPU: the shim's numpy-level calls answered by the CPU oracle."""
    from oracle import corr_oracle as O
    from theano_b200 import shim
    calls = {"fwd": 0, "gw": 0, "gi": 0, "pool": 0}

    def fwd(x, w, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
            filter_flip=True, bias=None, relu=False, slope=0.0, out=None, **_):
        calls["fwd"] += 1
        y = O.conv2d(x, w, border_mode, subsample, filter_dilation, num_groups, filter_flip)
        if slope:
            return O.epilogue(y, bias, None, 1.0, 1.0, relu, slope).astype(np.asarray(x).dtype)
        return O.bias_relu(y, bias, relu).astype(np.asarray(x).dtype)

    def gw(x, dy, kshape=None, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
           filter_flip=True, out=None, **_):
        calls["gw"] += 1
        return O.conv2d_grad_weights(x, dy, kshape, border_mode, subsample, filter_dilation, num_groups, filter_flip)

    def gi(w, dy, imshape=None, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
           filter_flip=True, out=None, **_):
        calls["gi"] += 1
        return O.conv2d_grad_inputs(w, dy, imshape, border_mode, subsample, filter_dilation, num_groups, filter_flip)

    def pool(x, **_):
        calls["pool"] += 1
        return O.maxpool2x2(x)

    monkeypatch.setattr(shim, "conv2d_forward", fwd)
    monkeypatch.setattr(shim, "conv2d_grad_weights", gw)
    monkeypatch.setattr(shim, "conv2d_grad_inputs", gi)
    def pool_grad(x, y, gy, **_):
        calls["pool_grad"] = calls.get("pool_grad", 0) + 1
        return O.maxpool2x2_grad(x, y, gy)

    monkeypatch.setattr(shim, "maxpool2x2", pool)
    monkeypatch.setattr(shim, "maxpool2x2_grad", pool_grad)
    return calls


def op_classes(f):
    return [type(n.op).__name__ for n in f.maker.fgraph.toposort()]


def test_optimizer_swaps_ops_in_and_tag_restores_corrmm(th):
    T = th.tensor
    x, w = T.ftensor4(), T.ftensor4()
    y = T.nnet.conv2d(x, w, border_mode="half", subsample=(2, 1), filter_dilation=(1, 2))
    gx, gw = th.grad(y.sum(), [x, w])
    f = th.function([x, w], [y, gx, gw])
    names = op_classes(f)
    assert "B200Conv2d" in names and "B200Conv2d_gradInputs" in names and "B200Conv2d_gradWeights" in names
    assert not any(n.startswith("CorrMM") or n.startswith("AbstractConv") for n in names)
    # the flip is inside the kernels: no Subtensor view of a 4-D tensor is left in the graph
    assert not [n for n in f.maker.fgraph.toposort()
                if type(n.op).__name__ == "Subtensor" and n.inputs[0].ndim == 4]
    conv = [n.op for n in f.maker.fgraph.toposort() if type(n.op).__name__ == "B200Conv2d"][0]
    assert (conv.border_mode, conv.subsample, conv.filter_dilation, conv.filter_flip) == ("half", (2, 1), (1, 2), True)
    f0 = th.function([x, w], [y, gx, gw], mode=th.compile.get_default_mode().excluding("conv_b200"))
    names0 = op_classes(f0)
    assert "CorrMM" in names0 and "CorrMM_gradInputs" in names0 and "CorrMM_gradWeights" in names0
    assert not any(n.startswith("B200") for n in names0)


def test_optimizer_declines_what_it_does_not_cover(th):
    T = th.tensor
    xd, wd = T.dtensor4(), T.dtensor4()
    f = th.function([xd, wd], T.nnet.conv2d(xd, wd))
    assert "CorrMM" in op_classes(f) and "B200Conv2d" not in op_classes(f)
    x, w6 = T.ftensor4(), T.TensorType("float32", (False,) * 6)()
    f = th.function([x, w6], T.nnet.conv2d(x, w6, unshared=True))
    assert "CorrMM" in op_classes(f) and "B200Conv2d" not in op_classes(f)


CASES = [
    dict(x=(3, 4, 9, 8), w=(6, 4, 3, 3), border="valid", sub=(1, 1), dil=(1, 1), groups=1, flip=True),
    dict(x=(2, 4, 9, 8), w=(6, 4, 3, 2), border="half", sub=(2, 1), dil=(1, 2), groups=1, flip=False),
    dict(x=(2, 6, 7, 7), w=(4, 3, 3, 3), border="full", sub=(1, 1), dil=(1, 1), groups=2, flip=True),
    dict(x=(2, 3, 8, 6), w=(5, 3, 2, 3), border=((1, 2), (2, 0)), sub=(2, 2), dil=(1, 1), groups=1, flip=True),
    dict(x=(1, 2, 6, 6), w=(2, 2, 3, 3), border=(2, 1), sub=(1, 1), dil=(2, 1), groups=1, flip=True),
]


@pytest.mark.parametrize("c", CASES, ids=[str(i) for i in range(len(CASES))])
def test_compiled_graph_matches_corrmm(th, oracle_device, c):
    """The abstract graph compiled twice: with the B200 ops and with the tag excluded (CorrMM)."""
    T = th.tensor
    rs = np.random.RandomState(4)
    x, w, g = T.ftensor4(), T.ftensor4(), T.ftensor4()
    y = T.nnet.conv2d(x, w, border_mode=c["border"], subsample=c["sub"], filter_dilation=c["dil"],
                      num_groups=c["groups"], filter_flip=c["flip"])
    outs = [y] + th.grad((y * g).sum(), [x, w])
    f = th.function([x, w, g], outs)
    f0 = th.function([x, w, g], outs, mode=th.compile.get_default_mode().excluding("conv_b200"))
    xv = rs.random_sample(c["x"]).astype("float32")
    wv = rs.random_sample(c["w"]).astype("float32")
    y0 = th.function([x, w], y, mode=th.compile.get_default_mode().excluding("conv_b200"))(xv, wv)
    gv = rs.random_sample(y0.shape).astype("float32")
    got, ref = f(xv, wv, gv), f0(xv, wv, gv)
    assert oracle_device["fwd"] >= 1 and oracle_device["gi"] == 1 and oracle_device["gw"] == 1
    for a, b in zip(got, ref):
        assert a.shape == b.shape and a.dtype == b.dtype
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-5)


def test_second_order_and_verify_grad(th, oracle_device):
    from theano_b200.ops import B200Conv2d, B200Conv2d_gradInputs, B200Conv2d_gradWeights
    rs = np.random.RandomState(2)
    xv = rs.random_sample((2, 2, 6, 6)).astype("float32")
    wv = rs.random_sample((3, 2, 3, 3)).astype("float32")
    gv = rs.random_sample((2, 3, 4, 4)).astype("float32")
    mode = th.compile.Mode(optimizer=None)
    th.gradient.verify_grad(lambda a, b: B200Conv2d("valid")(a, b), [xv, wv], rng=rs, mode=mode, eps=1e-2,
                            abs_tol=5e-2, rel_tol=5e-2)
    th.gradient.verify_grad(lambda a, b: B200Conv2d_gradWeights("valid")(a, b, (3, 3)), [xv, gv], rng=rs,
                            mode=mode, eps=1, abs_tol=5e-2, rel_tol=5e-2)
    th.gradient.verify_grad(lambda a, b: B200Conv2d_gradInputs("valid")(a, b, (6, 6)), [wv, gv], rng=rs,
                            mode=mode, eps=1, abs_tol=5e-2, rel_tol=5e-2)


def test_bias_relu_fusion_and_pool(th, oracle_device, golden):
    import cases as C
    from theano.tensor.signal.pool import pool_2d
    T = th.tensor
    x, w, b = T.ftensor4(), T.ftensor4(), T.fvector()
    act = T.nnet.relu(T.nnet.conv2d(x, w, border_mode=(1, 1)) + b.dimshuffle("x", 0, "x", "x"))
    f = th.function([x, w, b], [act, pool_2d(act, (2, 2), ignore_border=True)])
    names = op_classes(f)
    assert names.count("B200Conv2d") == 1 and "B200MaxPool2x2" in names
    assert "Elemwise" not in names and "Pool" not in names
    conv = [n for n in f.maker.fgraph.toposort() if type(n.op).__name__ == "B200Conv2d"][0]
    assert conv.op.relu and len(conv.inputs) == 3
    c = [k for k in C.all_cases() if k["name"] == "cfg2_small"][0]
    xv, wv, _ = C.make_inputs(c)
    a, p = f(xv, wv, golden["epilogue/bias"])
    np.testing.assert_allclose(C.sampled(a, c["sample"]), golden["epilogue/act"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(p, golden["epilogue/pool"], rtol=1e-4, atol=1e-5)
    # maximum(z, 0) form, no bias
    f2 = th.function([x, w], T.maximum(T.nnet.conv2d(x, w), 0))
    assert op_classes(f2) == ["B200Conv2d"]
    # in a training graph the pre-activation is needed by the backward pass: no fusion
    g = th.function([x, w, b], th.grad(act.sum(), [w]))
    convs = [n.op for n in g.maker.fgraph.toposort() if type(n.op).__name__ == "B200Conv2d"]
    assert convs and not any(o.relu for o in convs)


def test_leaky_relu_fusion(th, oracle_device):
    """relu(conv + b, alpha) in the reference's form f1 * z + f2 * |z| (nnet.py:2244-2250) becomes
    one B200Conv2d with relu and slope; values equal the unfused reference graph."""
    T = th.tensor
    x, w, b = T.ftensor4(), T.ftensor4(), T.fvector()
    act = T.nnet.relu(T.nnet.conv2d(x, w, border_mode="half") + b.dimshuffle("x", 0, "x", "x"), 0.125)
    f = th.function([x, w, b], act)
    names = op_classes(f)
    assert names == ["B200Conv2d"], names
    op = f.maker.fgraph.toposort()[0].op
    assert op.relu and abs(op.slope - 0.125) < 1e-6
    f0 = th.function([x, w, b], act, mode=th.compile.get_default_mode().excluding("conv_b200"))
    rs = np.random.RandomState(4)
    vals = [rs.standard_normal((2, 3, 7, 6)).astype(np.float32), rs.standard_normal((5, 3, 3, 3)).astype(np.float32),
            rs.standard_normal(5).astype(np.float32)]
    np.testing.assert_allclose(f(*vals), f0(*vals), rtol=1e-4, atol=1e-5)
    # ops with different slopes are different ops; pickling keeps the slope
    from theano_b200.ops import B200Conv2d
    assert B200Conv2d(relu=True, slope=0.1) != B200Conv2d(relu=True, slope=0.2)
    assert pickle.loads(pickle.dumps(B200Conv2d(relu=True, slope=0.1))).slope == 0.1
    # gradient through the fused op (built by hand: the optimizer never fuses in training graphs)
    y = B200Conv2d(border_mode="half", relu=True, slope=0.125)(x, w, b)
    g = th.function([x, w, b], th.grad(y.sum(), [x, w]))
    g0 = th.function([x, w, b], th.grad(act.sum(), [x, w]),
                     mode=th.compile.get_default_mode().excluding("conv_b200"))
    for a_, b_ in zip(g(*vals), g0(*vals)):
        np.testing.assert_allclose(a_, b_, rtol=1e-4, atol=1e-4)


def test_pool_gradient_op_in_training_graph(th, oracle_device):
    """conv -> 2x2 max pool, differentiated: the optimizer puts the device pooling and its
    gradient op in; values equal the reference graph compiled without the B200 ops."""
    from theano.tensor.signal.pool import pool_2d
    T = th.tensor
    x, w = T.ftensor4(), T.ftensor4()
    y = pool_2d(T.nnet.conv2d(x, w, border_mode=(1, 1)), (2, 2), ignore_border=True)
    cost = (y * y).sum()
    gw, gx = th.grad(cost, [w, x])
    f = th.function([x, w], [y, gw, gx])
    names = op_classes(f)
    assert "B200MaxPool2x2" in names and "B200MaxPool2x2Grad" in names
    assert "Pool" not in names and "MaxPoolGrad" not in names
    f0 = th.function([x, w], [y, gw, gx], mode=th.compile.get_default_mode().excluding("conv_b200"))
    assert "MaxPoolGrad" in op_classes(f0)
    rs = np.random.RandomState(5)
    xv = rs.standard_normal((2, 3, 9, 8)).astype(np.float32)
    wv = rs.standard_normal((4, 3, 3, 3)).astype(np.float32)
    for a, b in zip(f(xv, wv), f0(xv, wv)):
        np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-4)
    assert oracle_device["pool_grad"] >= 1
    # op contract of the gradient op
    from theano_b200.ops import B200MaxPool2x2Grad
    op = B200MaxPool2x2Grad()
    assert op == B200MaxPool2x2Grad() and hash(op) == hash(B200MaxPool2x2Grad())
    with pytest.raises(TypeError):
        op(T.fmatrix(), T.ftensor4(), T.ftensor4())


def _same_as_corrmm(th, inputs, outputs, values, oracle_device):
    f = th.function(inputs, outputs)
    names = op_classes(f)
    assert any(n.startswith("B200Conv2d") for n in names)
    assert not any(n.startswith("CorrMM") or n.startswith("AbstractConv") for n in names)
    f0 = th.function(inputs, outputs, mode=th.compile.get_default_mode().excluding("conv_b200"))
    assert any(n.startswith("CorrMM") for n in op_classes(f0))
    for a, b in zip(f(*values), f0(*values)):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-4)
    return names


def test_other_entry_points_that_build_the_abstract_ops(th, oracle_device):
    """conv2d_transpose, separable_conv2d (depthwise = one group per channel, then 1x1) and
    causal_conv1d (theano/tensor/nnet/nnet/__init__.py:172, abstract_conv.py:650, 1603) only construct the three
    abstract ops: the same optimizers take them, values equal the CorrMM graphs."""
    T = th.tensor
    from theano.tensor.nnet import conv2d_transpose
    from theano.tensor.nnet.abstract_conv import causal_conv1d, separable_conv2d
    rs = np.random.RandomState(9)
    # transposed convolution = gradInputs of a strided convolution
    x, w = T.ftensor4(), T.ftensor4()
    up = conv2d_transpose(x, w, output_shape=(2, 3, 11, 9), border_mode=(1, 1), input_dilation=(2, 2))
    names = _same_as_corrmm(th, [x, w], [up, th.grad(up.sum(), w)],
                            [rs.standard_normal((2, 5, 6, 5)).astype(np.float32),
                             rs.standard_normal((5, 3, 3, 3)).astype(np.float32)], oracle_device)
    assert "B200Conv2d_gradInputs" in names
    # depthwise (C groups, one input channel each) followed by a 1x1 convolution
    d, p = T.ftensor4(), T.ftensor4()
    sep = separable_conv2d(x, d, p, num_channels=4, border_mode="half")
    names = _same_as_corrmm(th, [x, d, p], [sep] + th.grad(sep.sum(), [x, d, p]),
                            [rs.standard_normal((2, 4, 7, 6)).astype(np.float32),
                             rs.standard_normal((8, 1, 3, 3)).astype(np.float32),
                             rs.standard_normal((5, 8, 1, 1)).astype(np.float32)], oracle_device)
    convs = [n for n in names if n == "B200Conv2d"]
    assert len(convs) == 2
    # causal 1-D convolution: left padding only, kernels one column wide
    s, k = T.ftensor3(), T.ftensor3()
    c1 = causal_conv1d(s, k, filter_shape=(3, 2, 4), filter_dilation=2)
    _same_as_corrmm(th, [s, k], [c1] + th.grad((c1 * c1).sum(), [s, k]),
                    [rs.standard_normal((2, 2, 13)).astype(np.float32),
                     rs.standard_normal((3, 2, 4)).astype(np.float32)], oracle_device)


def test_infer_shape_and_op_contract(th):
    from theano_b200.ops import B200Conv2d, B200Conv2d_gradInputs, B200Conv2d_gradWeights
    T = th.tensor
    x, w, g = T.ftensor4(), T.ftensor4(), T.ftensor4()
    for bm, sub, dil in (("valid", (1, 1), (1, 1)), ("half", (2, 2), (1, 1)), ("full", (1, 2), (2, 1)), ((1, 2), (1, 1), (1, 1))):
        y = B200Conv2d(bm, sub, dil)(x, w)
        dw = B200Conv2d_gradWeights(bm, sub, dil)(x, g, w.shape[-2:])
        dx = B200Conv2d_gradInputs(bm, sub, dil)(w, g, x.shape[-2:])
        f = th.function([x, w, g], [y.shape, dw.shape, dx.shape], on_unused_input="ignore")
        assert not any(n.startswith("B200") for n in op_classes(f))      # shapes need no convolution
        xs, ws = (2, 3, 11, 9), (4, 3, 3, 2)
        from theano_b200 import hostlogic
        ys = hostlogic.forward_shape(xs, ws, bm, sub, dil)[0]
        s = f(np.zeros(xs, "float32"), np.zeros(ws, "float32"), np.zeros(ys, "float32"))
        assert tuple(s[0]) == ys and tuple(s[1]) == ws and tuple(s[2]) == xs
    a, b = B200Conv2d("half", (1, 1)), B200Conv2d("half", (1, 1))
    assert a == b and hash(a) == hash(b) and a != B200Conv2d("half", (1, 1), relu=True)
    assert pickle.loads(pickle.dumps(a)) == a
    assert B200Conv2d(1).border_mode == ((1, 1), (1, 1))
    with pytest.raises(ValueError):
        B200Conv2d("same")
    with pytest.raises(TypeError):
        B200Conv2d()(T.ftensor3(), w)
    with pytest.raises(ValueError):
        B200Conv2d_gradWeights("half")(x, g)                 # shape required for 'half'
    with pytest.raises(ValueError):
        B200Conv2d_gradInputs("valid", (2, 2))(w, g)         # shape required for stride 2
    assert B200Conv2d().flops([(2, 3, 8, 8), (4, 3, 3, 3)], [(2, 4, 6, 6)]) == 2 * 2 * 4 * 3 * 9 * 36
    node = B200Conv2d_gradWeights("valid")(x, g, (3, 3)).owner
    assert node.op.connection_pattern(node) == [[1], [1], [0], [0]]


def test_perform_fails_loudly_without_gpu(th):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from theano_b200 import shim
    T = th.tensor
    x, w = T.ftensor4(), T.ftensor4()
    f = th.function([x, w], T.nnet.conv2d(x, w))
    with pytest.raises(shim.B200Error):
        f(np.zeros((1, 1, 5, 5), "float32"), np.zeros((1, 1, 3, 3), "float32"))


class _FakeDeviceTensor(object):
    """numpy-backed stand-in for shim.DeviceTensor (what the device ops need of it)."""
    uploads = 0
    downloads = 0

    def __init__(self, arr, layout="nhwc"):
        self.arr, self.layout, self.ctx, self.ptr = np.ascontiguousarray(arr), layout, "fake-ctx", id(self)
        self.shape, self.dtype = self.arr.shape, self.arr.dtype

    @classmethod
    def from_host(cls, ctx, arr, layout="nchw"):
        if np.asarray(arr).ndim == 4 and layout == "nhwc":
            cls.uploads += 1                 # activations; filters and biases are uploaded as 'nchw'
        return cls(np.array(arr), layout)

    def to_host(self, out=None):
        type(self).downloads += 1
        return self.arr.copy()


def test_device_resident_chain_in_a_theano_graph(th, monkeypatch):
    """With the 'b200_device' pass a conv -> pool -> conv inference graph uploads its input once,
    keeps the activations in device tensors between the ops and downloads once; values equal the
    reference graph.  (Device calls answered by the CPU oracle.)"""
    from oracle import corr_oracle as O
    from theano_b200 import devtype, shim
    from theano.tensor.signal.pool import pool_2d
    F = _FakeDeviceTensor
    F.uploads = F.downloads = 0

    def dev_conv(x, w, bias=None, relu=False, slope=0.0, out_layout=None, border_mode="valid", subsample=(1, 1),
                 filter_dilation=(1, 1), num_groups=1, filter_flip=True, **_):
        y = O.conv2d(x.arr, w.arr, border_mode, subsample, filter_dilation, num_groups, filter_flip)
        b = bias.arr.reshape(-1) if bias is not None else None
        return F(O.epilogue(y, b, None, 1.0, 1.0, relu, slope).astype(x.arr.dtype))

    monkeypatch.setattr(shim, "DeviceTensor", F)
    monkeypatch.setattr(shim, "get_context", lambda *a: "fake-ctx")
    monkeypatch.setattr(shim, "device_conv2d", dev_conv)
    monkeypatch.setattr(shim, "device_maxpool2x2", lambda x: F(O.maxpool2x2(x.arr)))
    T = th.tensor
    x, w1, b1, w2, b2 = T.ftensor4(), T.ftensor4(), T.fvector(), T.ftensor4(), T.fvector()
    a1 = T.nnet.relu(T.nnet.conv2d(x, w1, border_mode=(1, 1)) + b1.dimshuffle("x", 0, "x", "x"))
    a2 = T.nnet.relu(T.nnet.conv2d(pool_2d(a1, (2, 2), ignore_border=True), w2, border_mode=(1, 1)) +
                     b2.dimshuffle("x", 0, "x", "x"), 0.1)
    mode = th.compile.get_default_mode()
    f = th.function([x, w1, b1, w2, b2], [a2, a2.shape], mode=mode.including(devtype.TAG))
    names = op_classes(f)
    assert names[:5] == ["B200FromHost", "B200DevConv2d", "B200DevMaxPool2x2", "B200DevConv2d", "HostFromB200"], names
    assert not any(n in ("B200Conv2d", "B200MaxPool2x2", "Pool") for n in names)
    # without the tag the host ops stay
    assert "B200DevConv2d" not in op_classes(th.function([x, w1, b1, w2, b2], a2))
    rs = np.random.RandomState(8)
    vals = [rs.standard_normal((2, 3, 10, 8)).astype(np.float32), rs.standard_normal((6, 3, 3, 3)).astype(np.float32),
            rs.standard_normal(6).astype(np.float32), rs.standard_normal((4, 6, 3, 3)).astype(np.float32),
            rs.standard_normal(4).astype(np.float32)]
    got, shp = f(*vals)
    want = th.function([x, w1, b1, w2, b2], a2, mode=mode.excluding("conv_b200"))(*vals)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
    assert tuple(shp) == want.shape
    assert (F.uploads, F.downloads) == (1, 1)
    # the Type: equality, filtering, pickling of a compiled function's ops
    t = devtype.B200TensorType("float32", (False,) * 4)
    assert t == devtype.B200TensorType("float32", (False,) * 4) and t != devtype.B200TensorType("float16", (False,) * 4)
    assert isinstance(t.filter(vals[0]), F)
    with pytest.raises(TypeError):
        t.filter(vals[0], strict=True)
    with pytest.raises(TypeError):
        t.filter(vals[0].astype(np.float64))
    assert pickle.loads(pickle.dumps(devtype.B200DevConv2d(relu=True, slope=0.1))) == devtype.B200DevConv2d(relu=True, slope=0.1)


def test_device_resident_training_graph(th, monkeypatch):
    """With the 'b200_device' pass the gradient ops of a conv -> pool -> conv graph run on device
    tensors too: gradWeights reads the activations the forward pass left on the device, gradInputs and
    the pooling gradient pass their results on without a download; the input is uploaded once and
    only the three results come back.  Values equal the reference graph.  (Device calls answered by
    the CPU oracle.)"""
    from oracle import corr_oracle as O
    from theano_b200 import devtype, shim
    from theano.tensor.signal.pool import pool_2d
    F = _FakeDeviceTensor
    F.uploads = F.downloads = 0

    def dev_conv(x, w, bias=None, relu=False, slope=0.0, out_layout=None, **kw):
        assert bias is None and not relu
        return F(O.conv2d(x.arr, w.arr, **kw))

    def dev_dgrad(w, dy, imshape, out_layout=None, **kw):
        return F(O.conv2d_grad_inputs(w.arr, dy.arr, imshape, **kw))

    def dev_wgrad(x, dy, kshape, **kw):
        return F(O.conv2d_grad_weights(x.arr, dy.arr, kshape, **kw), "nchw")

    monkeypatch.setattr(shim, "DeviceTensor", F)
    monkeypatch.setattr(shim, "get_context", lambda *a: "fake-ctx")
    monkeypatch.setattr(shim, "device_conv2d", dev_conv)
    monkeypatch.setattr(shim, "device_grad_inputs", dev_dgrad)
    monkeypatch.setattr(shim, "device_grad_weights", dev_wgrad)
    monkeypatch.setattr(shim, "device_maxpool2x2", lambda x: F(O.maxpool2x2(x.arr)))
    monkeypatch.setattr(shim, "device_maxpool2x2_grad", lambda x, y, g: F(O.maxpool2x2_grad(x.arr, y.arr, g.arr)))
    T = th.tensor
    x, w1, w2, r = T.ftensor4(), T.ftensor4(), T.ftensor4(), T.ftensor4()
    a1 = T.nnet.conv2d(x, w1, border_mode=(1, 1))
    a2 = T.nnet.conv2d(pool_2d(a1, (2, 2), ignore_border=True), w2, border_mode=(1, 1), subsample=(2, 2))
    loss = (a2 * r).sum()
    grads = th.grad(loss, [w1, w2, x])
    mode = th.compile.get_default_mode()
    f = th.function([x, w1, w2, r], grads, mode=mode.including(devtype.TAG))
    names = op_classes(f)
    for want in ("B200DevConv2d", "B200DevMaxPool2x2", "B200DevConv2d_gradInputs", "B200DevConv2d_gradWeights",
                 "B200DevMaxPool2x2Grad"):
        assert want in names, (want, names)
    assert names.count("B200DevConv2d_gradWeights") == 2 and names.count("B200DevConv2d_gradInputs") == 2
    for gone in ("B200Conv2d", "B200Conv2d_gradInputs", "B200Conv2d_gradWeights", "B200MaxPool2x2",
                 "B200MaxPool2x2Grad", "Pool", "MaxPoolGrad"):
        assert gone not in names, (gone, names)
    rs = np.random.RandomState(12)
    vals = [rs.standard_normal((2, 3, 12, 8)).astype(np.float32), rs.standard_normal((5, 3, 3, 3)).astype(np.float32),
            rs.standard_normal((4, 5, 3, 3)).astype(np.float32), rs.standard_normal((2, 4, 3, 2)).astype(np.float32)]
    got = f(*vals)
    want = th.function([x, w1, w2, r], grads, mode=mode.excluding("conv_b200"))(*vals)
    for g, w in zip(got, want):
        assert g.shape == w.shape
        np.testing.assert_allclose(g, w, rtol=1e-4, atol=1e-4)
    # x and the loss weights go up once each; dW1, dW2 and dx come down (the fake counts 4-D
    # 'nhwc' uploads and every download)
    assert (F.uploads, F.downloads) == (2, 3), (F.uploads, F.downloads)
    # the constructors refuse what the host ops refuse
    dx = devtype.B200TensorType("float32")()
    with pytest.raises(ValueError):
        devtype.B200DevConv2d_gradInputs(subsample=(2, 2))(w1, dx)
    with pytest.raises(ValueError):
        devtype.B200DevConv2d_gradWeights(border_mode="half")(dx, dx)
    with pytest.raises(TypeError):
        devtype.B200DevConv2d_gradWeights()(x, dx)
    op = devtype.B200DevConv2d_gradWeights(border_mode=(1, 1), subsample=(2, 2))
    assert pickle.loads(pickle.dumps(op)) == op


def test_elementwise_nodes_between_device_ops_stay_on_the_device(th):
    """conv + bias -> relu -> conv, differentiated with a given output gradient, compiled with the
    'b200_device' pass: the bias add, the rectifier, its gradient and the bias-gradient sum become
    device ops, so the graph uploads each 4-D input once (x and the output gradient) and downloads
    only what the function returns (y and dx; the filter and bias gradients are small host results)."""
    from theano_b200 import devtype
    T = th.tensor
    x, w1, w2, gy, b1 = T.ftensor4(), T.ftensor4(), T.ftensor4(), T.ftensor4(), T.fvector()
    pre = T.nnet.conv2d(x, w1, border_mode="half") + b1.dimshuffle("x", 0, "x", "x")
    y = T.nnet.conv2d(T.nnet.relu(pre), w2, border_mode="half")
    grads = th.grad(None, [w1, w2, b1, x], known_grads={y: gy})
    f = th.function([x, w1, w2, b1, gy], [y] + grads, mode=th.compile.get_default_mode().including(devtype.TAG))
    nodes = f.maker.fgraph.toposort()
    ops = [type(n.op).__name__ for n in nodes]
    assert ops.count("B200FromHost") == 2 and ops.count("HostFromB200") == 2, ops
    assert "B200DevChannelSum" in ops and ops.count("B200DevElemwise") >= 5, ops
    from theano.tensor.elemwise import Elemwise
    assert not [n for n in nodes if isinstance(n.op, Elemwise) and n.outputs[0].ndim == 4], ops
    # without the pass the same graph keeps its host Elemwise nodes
    g = th.function([x, w1, w2, b1, gy], [y] + grads)
    assert "B200DevElemwise" not in [type(n.op).__name__ for n in g.maker.fgraph.toposort()]
