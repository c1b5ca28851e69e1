"""Host-side shape logic against the reference's known answers."""
import pytest

from theano_b200 import hostlogic as H


def test_output_shape_known_answers():
    # TestGetConvOutShape.test_basic, reference test_abstract_conv.py:102-118
    x, w, sub, dil = (3, 2, 12, 9), (4, 2, 5, 6), (1, 2), (2, 1)
    assert H.forward_shape(x, w, "valid", sub, dil)[0] == (3, 4, 4, 2)
    assert H.forward_shape(x, w, "half", sub, dil)[0] == (3, 4, 12, 5)
    assert H.forward_shape(x, w, "full", sub, dil)[0] == (3, 4, 20, 7)
    assert H.forward_shape(x, w, (1, 2), sub, dil)[0] == (3, 4, 6, 4)


def test_border_mode_normalisation():
    assert H.normalize_border_mode(2) == ((2, 2), (2, 2))
    assert H.normalize_border_mode((1, (2, 3))) == ((1, 1), (2, 3))
    assert H.normalize_border_mode("half") == "half"
    for bad in (-1, (1,), (1, -2), "same", ((1, 2, 3), 1)):
        with pytest.raises(ValueError):
            H.normalize_border_mode(bad)


def test_gradient_shape_inference():
    # stride 1: both sizes can be inferred; stride 2 / half: they must be given (corr.py:286-294)
    assert H.gradweights_kshape((2, 3, 9, 9), (2, 4, 7, 7), "valid", (1, 1), (1, 1)) == (3, 3)
    assert H.gradweights_kshape((2, 3, 9, 9), (2, 4, 11, 11), "full", (1, 1), (1, 1)) == (3, 3)
    assert H.gradweights_kshape((2, 3, 9, 9), (2, 4, 5, 5), (0, 0), (1, 1), (2, 2)) == (3, 3)
    with pytest.raises(ValueError):
        H.gradweights_kshape((2, 3, 9, 9), (2, 4, 4, 4), "valid", (2, 2), (1, 1))
    with pytest.raises(ValueError):
        H.gradweights_kshape((2, 3, 9, 9), (2, 4, 9, 9), "half", (1, 1), (1, 1))
    assert H.gradinputs_imshape((4, 3, 3, 3), (2, 4, 7, 7), "valid", (1, 1), (1, 1))[0] == (9, 9)
    with pytest.raises(ValueError):
        H.gradinputs_imshape((4, 3, 3, 3), (2, 4, 4, 4), "valid", (2, 2), (1, 1))


def test_inconsistent_shapes_raise_value_error():
    # reference test_abstract_conv.py:602-656: output shapes the forward cannot produce
    for o in (-3, -1, 1, 2):
        pads = H.resolve_pads("valid", (3, 3), (1, 1))
        with pytest.raises(ValueError):
            H.check_consistent((1, 1, 7, 7), (1, 1, 3, 3), (1, 1, 5 + o, 5 + o), pads, (1, 1), (1, 1), 1)
    with pytest.raises(ValueError):
        H.forward_shape((1, 3, 5, 5), (2, 2, 3, 3), "valid", (1, 1), (1, 1))
    with pytest.raises(ValueError):
        H.forward_shape((1, 3, 5, 5), (2, 3, 7, 7), "valid", (1, 1), (1, 1))
    with pytest.raises(TypeError):
        H.forward_shape((1, 3, 5), (2, 3, 3, 3), "valid", (1, 1), (1, 1))
