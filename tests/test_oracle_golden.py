"""The CPU oracle against outputs of the reference itself (golden fixtures) and
against the known answers held by the reference's own tests."""
import numpy as np
import pytest

import cases as C
from oracle import corr_oracle as O

CASES = C.all_cases()
TOL = 2e-5   # float32 gemm vs float32 gemm with another summation order


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_outputs(c, golden):
    x, w, dy = C.make_inputs(c)
    kw = dict(border_mode=c["border"], subsample=c["sub"], filter_dilation=c["dil"],
              num_groups=c["groups"], filter_flip=c["flip"])
    y = O.conv2d(x, w, **kw)
    dx = O.conv2d_grad_inputs(w, dy, x.shape[2:], **kw)
    dw = O.conv2d_grad_weights(x, dy, w.shape[2:], **kw)
    s = c["sample"]
    assert O.rel_err(C.sampled(y, s), golden[c["name"] + "/y"]) < TOL
    assert O.rel_err(C.sampled(dx, s), golden[c["name"] + "/dx"]) < TOL
    assert O.rel_err(dw, golden[c["name"] + "/dw"]) < TOL


def test_plain_c_gemm_equals_blas_gemm():
    c = [k for k in CASES if k["name"] == "cfg2_small"][0]
    x, w, dy = C.make_inputs(c)
    a = O.corr_fwd(x, w, c["border"])
    had = O.use_blas(False)
    try:
        b = O.corr_fwd(x, w, c["border"])
    finally:
        O.use_blas(True)
    assert not had
    assert O.rel_err(a, b) < TOL


def test_float64_oracle_close_to_float32():
    c = [k for k in CASES if k["name"] == "cfg4c_small"][0]
    x, w, dy = C.make_inputs(c)
    kw = dict(border_mode=c["border"], subsample=c["sub"], filter_dilation=c["dil"])
    assert O.rel_err(O.conv2d(x, w, **kw), O.conv2d(x, w, real="double", **kw)) < 1e-5


def test_causal_conv_known_answer(golden):
    """TestCausalConv (reference test_abstract_conv.py:2081-2102): causal_conv1d is the 2-D op
    with border_mode ((left_pad, 0), 0), kW = 1 and dilation (d, 1) (abstract_conv.py:1676-1703)."""
    img, kern, top = golden["causal/img"], golden["causal/kern"], golden["causal/precomp_top"]
    d = int(golden["causal/dilation"])
    left = d * (kern.shape[2] - 1)
    y = O.conv2d(img[:, :, :, None], kern[:, :, :, None], border_mode=((left, 0), 0),
                 filter_dilation=(d, 1), filter_flip=True)
    np.testing.assert_allclose(y[:, :, :, 0], top, rtol=1e-6)


def test_epilogue_and_pool(golden):
    c = [k for k in CASES if k["name"] == "cfg2_small"][0]
    x, w, _ = C.make_inputs(c)
    act = O.bias_relu(O.conv2d(x, w, border_mode=c["border"]), golden["epilogue/bias"], relu=True)
    assert O.rel_err(C.sampled(act, c["sample"]), golden["epilogue/act"]) < TOL
    assert O.rel_err(O.maxpool2x2(act), golden["epilogue/pool"]) < TOL


def test_shape_known_answers():
    """TestGetConvOutShape.test_basic (reference test_abstract_conv.py:102-118)."""
    L = O.lib()
    img, ker, sub, dil = (12, 9), (5, 6), (1, 2), (2, 1)

    def shp(pads):
        return tuple(L.oracle_out_size(img[a], ker[a], dil[a], pads[a][0], pads[a][1], sub[a]) for a in range(2))
    assert shp(O._pads("valid", ker, dil)) == (4, 2)
    assert shp(O._pads("half", ker, dil)) == (12, 5)
    assert shp(O._pads("full", ker, dil)) == (20, 7)
    assert shp(O._pads((1, 2), ker, dil)) == (6, 4)


def test_errors():
    x = np.zeros((2, 3, 5, 5), np.float32)
    with pytest.raises(ValueError):
        O.corr_fwd(x, np.zeros((4, 2, 3, 3), np.float32))            # stack size mismatch
    with pytest.raises(ValueError):
        O.corr_fwd(x, np.zeros((4, 3, 7, 7), np.float32))            # impossible output
    with pytest.raises(ValueError):
        O.corr_grad_inputs(np.zeros((4, 3, 3, 3), np.float32), np.zeros((2, 4, 3, 3), np.float32),
                           (9, 9))                                    # shape the forward cannot make
    with pytest.raises(ValueError):
        O.corr_grad_weights(x, np.zeros((2, 4, 3, 3), np.float32), None, subsample=(2, 2))


@pytest.mark.parametrize("name", ["even", "odd", "ties", "wide"])
def test_pool_and_pool_gradient_against_reference_outputs(pool_golden, name):
    """Pool / MaxPoolGrad of the reference (compiled C code), ws = stride = 2: exact."""
    x, y, gy, gx = (pool_golden["%s/%s" % (name, k)] for k in ("x", "y", "gy", "gx"))
    assert np.array_equal(O.maxpool2x2(x), y)
    assert np.array_equal(O.maxpool2x2_grad(x, y, gy), gx)
    if name == "ties":                       # several maxima in a window all receive the gradient
        assert (gx != 0).sum() > gy.size
