"""The Theano plug-in path on a real GPU: graphs compiled by the reference's own compiler run the
B200 ops' ``perform`` through the C ABI.  Needs an importable reference (its source tree, or the
copy installed under baseline/_ref); skipped otherwise."""
import numpy as np
import pytest

import ref_theano
from oracle import corr_oracle as O

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_theano.available(), reason="reference Theano not importable here")]


@pytest.fixture(scope="module")
def th():
    try:                                        # the reference's own tool chain (g++, headers) must work here
        theano = ref_theano.import_theano()
        a = theano.tensor.fvector()
        assert theano.function([a], a + 1)(np.zeros(2, np.float32))[0] == 1
    except Exception as e:                      # noqa: BLE001
        pytest.skip("the reference cannot compile graphs on this machine: %r" % (e,))
    import theano_b200.devtype  # noqa: F401  (registers every pass)
    return theano


def names(f):
    return [type(n.op).__name__ for n in f.maker.fgraph.toposort()]


def test_training_graph_on_gpu(th):
    """conv -> pool, differentiated: forward, both gradients and the pool gradient run on the GPU
    and equal the CPU restatement."""
    from theano.tensor.signal.pool import pool_2d
    T = th.tensor
    x, w = T.ftensor4(), T.ftensor4()
    c = T.nnet.conv2d(x, w, border_mode="half", subsample=(1, 1))
    y = pool_2d(c, (2, 2), ignore_border=True)
    gw, gx = th.grad((y * y).sum() * 0.5, [w, x])
    f = th.function([x, w], [c, y, gw, gx])
    ops = names(f)
    for n in ("B200Conv2d", "B200Conv2d_gradWeights", "B200Conv2d_gradInputs", "B200MaxPool2x2", "B200MaxPool2x2Grad"):
        assert n in ops, ops
    rs = np.random.RandomState(12)
    xv = rs.standard_normal((4, 32, 14, 14)).astype(np.float32)
    wv = (rs.standard_normal((48, 32, 3, 3)) * 0.1).astype(np.float32)
    cv, yv, gwv, gxv = f(xv, wv)
    assert O.rel_err(cv, O.conv2d(xv, wv, border_mode="half")) < 5e-3
    assert np.array_equal(yv, O.maxpool2x2(cv))
    # which element of a window is the maximum depends on the last bits of the convolution: route
    # the gradient with the values the GPU produced, then check the two convolution gradients
    gconv = O.maxpool2x2_grad(cv, yv, yv)                   # d(0.5 * sum y^2)/dy = y
    assert O.rel_err(gwv, O.conv2d_grad_weights(xv, gconv, (3, 3), border_mode="half")) < 5e-3
    assert O.rel_err(gxv, O.conv2d_grad_inputs(wv, gconv, (14, 14), border_mode="half")) < 5e-3


def test_device_resident_inference_chain_on_gpu(th):
    """Two conv+bias+(leaky) ReLU layers with a pool between them, activations kept in HBM by the
    'b200_device' pass; same values as the graph of host ops and as the CPU restatement."""
    from theano.tensor.signal.pool import pool_2d
    from theano_b200 import devtype
    T = th.tensor
    x, w1, b1, w2, b2 = T.ftensor4(), T.ftensor4(), T.fvector(), T.ftensor4(), T.fvector()
    a1 = T.nnet.relu(T.nnet.conv2d(x, w1, border_mode=(1, 1)) + b1.dimshuffle("x", 0, "x", "x"))
    a2 = T.nnet.relu(T.nnet.conv2d(pool_2d(a1, (2, 2), ignore_border=True), w2, border_mode=(1, 1)) +
                     b2.dimshuffle("x", 0, "x", "x"), 0.1)
    mode = th.compile.get_default_mode()
    f_dev = th.function([x, w1, b1, w2, b2], a2, mode=mode.including(devtype.TAG))
    f_host = th.function([x, w1, b1, w2, b2], a2)
    assert names(f_dev) == ["B200FromHost", "B200DevConv2d", "B200DevMaxPool2x2", "B200DevConv2d", "HostFromB200"]
    assert names(f_host) == ["B200Conv2d", "B200MaxPool2x2", "B200Conv2d"]
    rs = np.random.RandomState(13)
    vals = [rs.standard_normal((8, 16, 28, 28)).astype(np.float32),
            (rs.standard_normal((64, 16, 3, 3)) * 0.1).astype(np.float32), rs.standard_normal(64).astype(np.float32),
            (rs.standard_normal((32, 64, 3, 3)) * 0.05).astype(np.float32), rs.standard_normal(32).astype(np.float32)]
    got_dev, got_host = f_dev(*vals), f_host(*vals)
    r1 = O.maxpool2x2(O.bias_relu(O.conv2d(vals[0], vals[1], border_mode=(1, 1)), vals[2], relu=True))
    want = O.epilogue(O.conv2d(r1, vals[3], border_mode=(1, 1)), vals[4], None, 1.0, 1.0, True, 0.1)
    assert O.rel_err(got_dev, want) < 5e-3 and O.rel_err(got_host, want) < 5e-3
    assert O.rel_err(got_dev, got_host) < 1e-6 or np.allclose(got_dev, got_host, rtol=1e-5, atol=1e-5)


def test_device_resident_training_graph_on_gpu(th):
    """conv -> pool -> strided conv, differentiated, with the 'b200_device' pass: every convolution,
    pooling and gradient op runs on device tensors; the three gradients equal the CPU restatement
    (the pooling gradient routed with the activations the GPU produced)."""
    from theano.tensor.signal.pool import pool_2d
    from theano_b200 import devtype
    T = th.tensor
    x, w1, w2, r = T.ftensor4(), T.ftensor4(), T.ftensor4(), T.ftensor4()
    a1 = T.nnet.conv2d(x, w1, border_mode=(1, 1))
    p1 = pool_2d(a1, (2, 2), ignore_border=True)
    a2 = T.nnet.conv2d(p1, w2, border_mode=(1, 1), subsample=(2, 2))
    grads = th.grad((a2 * r).sum(), [w1, w2, x])
    mode = th.compile.get_default_mode()
    f = th.function([x, w1, w2, r], [a1] + grads, mode=mode.including(devtype.TAG))
    ops = names(f)
    # the loss is linear in the second convolution, so only the first forward is in the graph
    assert ops.count("B200DevConv2d") == 1 and ops.count("B200DevConv2d_gradWeights") == 2, ops
    assert ops.count("B200DevConv2d_gradInputs") == 2 and "B200DevMaxPool2x2Grad" in ops, ops
    assert not [n for n in ops if n.startswith("B200Conv2d") or n.startswith("B200MaxPool")], ops
    assert ops.count("B200FromHost") == 2, ops              # x and r
    rs = np.random.RandomState(14)
    xv = rs.standard_normal((8, 16, 28, 28)).astype(np.float32)
    w1v = (rs.standard_normal((64, 16, 3, 3)) * 0.1).astype(np.float32)
    w2v = (rs.standard_normal((32, 64, 3, 3)) * 0.05).astype(np.float32)
    rv = rs.standard_normal((8, 32, 7, 7)).astype(np.float32)
    a1v, gw1, gw2, gx = f(xv, w1v, w2v, rv)
    assert O.rel_err(a1v, O.conv2d(xv, w1v, border_mode=(1, 1))) < 5e-3
    p1v = O.maxpool2x2(a1v)
    k2 = dict(border_mode=(1, 1), subsample=(2, 2))
    g_p1 = O.conv2d_grad_inputs(w2v, rv, (14, 14), **k2)
    g_a1 = O.maxpool2x2_grad(a1v, p1v, g_p1)
    assert O.rel_err(gw2, O.conv2d_grad_weights(p1v, rv, (3, 3), **k2)) < 5e-3
    assert O.rel_err(gw1, O.conv2d_grad_weights(xv, g_a1, (3, 3), border_mode=(1, 1))) < 5e-3
    assert O.rel_err(gx, O.conv2d_grad_inputs(w1v, g_a1, (28, 28), border_mode=(1, 1))) < 5e-3


def test_elementwise_device_kernels_against_numpy():
    """b200conv_elementwise and b200conv_channel_sum on channels-last tensors (24 channels: the
    float32 layout has no pad channels, the float16 layout none either; 6 channels: padded)."""
    from theano_b200 import shim
    ctx = shim.get_context(0)
    rs = np.random.RandomState(3)
    for dtype, tol in ((np.float32, 1e-6), (np.float16, 2e-3)):
        for c in (24, 6):
            a = rs.standard_normal((3, c, 9, 7)).astype(dtype)
            b = (rs.standard_normal((3, c, 9, 7)) + 3.0).astype(dtype)
            v = rs.standard_normal(c).astype(dtype)
            A, B = shim.DeviceTensor.from_host(ctx, a, "nhwc"), shim.DeviceTensor.from_host(ctx, b, "nhwc")
            af, bf, vf = a.astype(np.float32), b.astype(np.float32), v.astype(np.float32).reshape(1, -1, 1, 1)
            cases = [("add", B, af + bf), ("mul", B, af * bf), ("sub", B, af - bf), ("rsub", B, bf - af),
                     ("div", B, af / bf), ("max", B, np.maximum(af, bf)), ("add", v, af + vf), ("mul", v, af * vf),
                     ("mul", 0.5, af * 0.5), ("rsub", 2.0, 2.0 - af), ("abs", None, np.abs(af)),
                     ("sgn", None, np.sign(af)), ("neg", None, -af)]
            for op, operand, want in cases:
                got = shim.device_elementwise(op, A, operand).to_host().astype(np.float32)
                assert np.allclose(got, want, rtol=tol, atol=tol), (np.dtype(dtype).name, c, op)
            s = shim.device_channel_sum(A).astype(np.float32)
            assert np.allclose(s, af.sum(axis=(0, 2, 3)), rtol=5e-3, atol=5e-3), (np.dtype(dtype).name, c)


def test_device_resident_relu_training_graph_against_corrmm(th):
    """conv + bias -> relu -> conv with both passes on (B200 ops, device residency with the
    element-wise ops on the device) against the SAME graph compiled without the B200 optimizers,
    i.e. the reference's CorrMM ops and its own Elemwise: forward result and all four gradients."""
    from theano_b200 import devtype
    T = th.tensor
    x, w1, w2, gy, b1 = T.ftensor4(), T.ftensor4(), T.ftensor4(), T.ftensor4(), T.fvector()
    pre = T.nnet.conv2d(x, w1, border_mode="half") + b1.dimshuffle("x", 0, "x", "x")
    y = T.nnet.conv2d(T.nnet.relu(pre), w2, border_mode="half")
    grads = th.grad(None, [w1, w2, b1, x], known_grads={y: gy})
    mode = th.compile.get_default_mode()
    f = th.function([x, w1, w2, b1, gy], [y] + grads, mode=mode.including(devtype.TAG))
    ref = th.function([x, w1, w2, b1, gy], [y] + grads, mode=mode.excluding("conv_b200"))
    ops, ref_ops = names(f), names(ref)
    assert ops.count("B200FromHost") == 2 and ops.count("HostFromB200") == 2, ops
    assert "CorrMM" in ref_ops and not [n for n in ref_ops if n.startswith("B200")], ref_ops
    rs = np.random.RandomState(15)
    # The rectifier's gradient is a step at zero: where the first convolution lands within TF32
    # rounding of zero the two implementations would pick different sides, and the comparison
    # would measure that, not the kernels.  x, w1 and b1 are therefore multiples of 1/8 in a small
    # range: their products and sums are exact in TF32 / float32, so both graphs see the same
    # pre-activation and the same mask; everything behind it is ordinary random data.
    vals = [(rs.randint(-8, 9, (6, 16, 20, 20)) / 8.0).astype(np.float32),
            (rs.randint(-4, 5, (32, 16, 3, 3)) / 8.0).astype(np.float32),
            (rs.standard_normal((24, 32, 3, 3)) * 0.1).astype(np.float32),
            (rs.randint(-4, 5, 32) / 8.0).astype(np.float32),
            rs.standard_normal((6, 24, 20, 20)).astype(np.float32)]
    got, want = f(*vals), ref(*vals)
    for name, a, b in zip(("y", "dw1", "dw2", "db1", "dx"), got, want):
        assert O.rel_err(np.asarray(a), np.asarray(b)) < 5e-3, name
