"""Graph optimizers that swap the B200 ops into existing Theano graphs.

Importing this module registers

* three local optimizers in ``theano.tensor.nnet.opt.conv_groupopt`` (tag ``conv_b200``)
  that lower ``AbstractConv2d``, ``AbstractConv2d_gradWeights`` and
  ``AbstractConv2d_gradInputs`` to the B200 ops.  They are registered with the keyword
  ``position=-1`` so that they are tried before the reference's GEMM lowerings
  (theano/tensor/nnet/opt.py:445-476; ``LocalGroupDB.register`` takes the position only as a
  keyword, theano/gof/optdb.py:417-427).  ``mode.excluding('conv_b200')`` gives the reference
  path back.
* one pass at optdb position 48.8 (after the abstract-conv check at 48.7, before elemwise
  fusion at 49) that folds ``relu(conv + bias)`` into the convolution's epilogue, and turns
  the 2x2 max pooling that follows into the device op when its input already comes from one.

Declined (left to CorrMM): ``unshared=True``, float64, non-TensorType inputs.
"""
import numpy as np
import theano
from theano import gof, tensor
from theano.compile import optdb
from theano.gof import local_optimizer
from theano.gof.opt import copy_stack_trace
from theano.tensor import TensorType
from theano.tensor.elemwise import DimShuffle, Elemwise
from theano.tensor.nnet import opt as nnet_opt
from theano.tensor.nnet.abstract_conv import (AbstractConv2d, AbstractConv2d_gradInputs,
                                              AbstractConv2d_gradWeights)
from theano.tensor.opt import in2out

from .ops import (B200Conv2d, B200Conv2d_gradInputs, B200Conv2d_gradWeights, B200MaxPool2x2,
                  B200MaxPool2x2Grad)

TAG = "conv_b200"


def _eligible(node, *vars_):
    if getattr(node.op, "unshared", False):
        return False
    for v in vars_:
        if not isinstance(v.type, TensorType) or v.dtype not in ("float16", "float32"):
            return False
    return True


def _props(op):
    return dict(border_mode=op.border_mode, subsample=op.subsample, filter_dilation=op.filter_dilation,
                num_groups=op.num_groups, filter_flip=op.filter_flip)


def _finish(node, rval):
    copy_stack_trace(node.outputs[0], rval)
    if rval.type != node.outputs[0].type:
        rval = tensor.patternbroadcast(rval, node.outputs[0].broadcastable)
        copy_stack_trace(node.outputs[0], rval)
    return [rval]


@local_optimizer([AbstractConv2d])
def local_abstractconv_b200(node):
    if not isinstance(node.op, AbstractConv2d):
        return None
    img, kern = node.inputs
    if not _eligible(node, img, kern):
        return None
    return _finish(node, B200Conv2d(**_props(node.op))(img, kern))


@local_optimizer([AbstractConv2d_gradWeights])
def local_abstractconv_gradweights_b200(node):
    if not isinstance(node.op, AbstractConv2d_gradWeights):
        return None
    img, topgrad, shape = node.inputs
    if not _eligible(node, img, topgrad):
        return None
    return _finish(node, B200Conv2d_gradWeights(**_props(node.op))(img, topgrad, shape))


@local_optimizer([AbstractConv2d_gradInputs])
def local_abstractconv_gradinputs_b200(node):
    if not isinstance(node.op, AbstractConv2d_gradInputs):
        return None
    kern, topgrad, shape = node.inputs
    if not _eligible(node, kern, topgrad):
        return None
    return _finish(node, B200Conv2d_gradInputs(**_props(node.op))(kern, topgrad, shape))


# ---- epilogue fusion ---------------------------------------------------------------------
def _is_elemwise(var, scalar_cls):
    return (var.owner is not None and isinstance(var.owner.op, Elemwise) and
            isinstance(var.owner.op.scalar_op, scalar_cls))


def _const_value(var):
    try:
        v = tensor.get_scalar_constant_value(var)
    except tensor.NotScalarConstantError:
        return None
    return float(v)


def _relu_argument(node):
    """If ``node`` computes relu(z) return z, else None.  Forms: 0.5 * (z + abs(z))
    (theano/tensor/nnet/nnet.py:2242-2243) and maximum(z, 0)."""
    sc = theano.scalar
    if not isinstance(node.op, Elemwise):
        return None
    if isinstance(node.op.scalar_op, sc.Maximum) and len(node.inputs) == 2:
        for a, b in (node.inputs, node.inputs[::-1]):
            if _const_value(b) == 0.0:
                return a
        return None
    if isinstance(node.op.scalar_op, sc.Mul) and len(node.inputs) == 2:
        for c, s in (node.inputs, node.inputs[::-1]):
            if _const_value(c) != 0.5 or not _is_elemwise(s, sc.Add) or len(s.owner.inputs) != 2:
                continue
            for z, az in (s.owner.inputs, s.owner.inputs[::-1]):
                if _is_elemwise(az, sc.Abs) and az.owner.inputs[0] is z:
                    return z
    return None


def _leaky_relu_argument(node):
    """If ``node`` computes the reference's leaky rectifier f1 * z + f2 * abs(z) with constants
    f1 = 0.5 * (1 + slope), f2 = 0.5 * (1 - slope) (theano/tensor/nnet/nnet.py:2244-2250) return
    (z, slope, [the nodes of the pattern]), else None."""
    sc = theano.scalar
    if not _is_elemwise(node.outputs[0], sc.Add) or len(node.inputs) != 2:
        return None
    for lin, ab in (node.inputs, node.inputs[::-1]):
        if not (_is_elemwise(lin, sc.Mul) and _is_elemwise(ab, sc.Mul)):
            continue
        if len(lin.owner.inputs) != 2 or len(ab.owner.inputs) != 2:
            continue
        for f1v, z in (lin.owner.inputs, lin.owner.inputs[::-1]):
            f1 = _const_value(f1v)
            if f1 is None:
                continue
            for f2v, az in (ab.owner.inputs, ab.owner.inputs[::-1]):
                f2 = _const_value(f2v)
                if f2 is None or not _is_elemwise(az, sc.Abs) or az.owner.inputs[0] is not z:
                    continue
                slope = f1 - f2
                if abs(f1 + f2 - 1.0) > 1e-6 or not (0.0 < slope < 1.0):
                    continue
                if not (_only_used_by(lin, [node]) and _only_used_by(ab, [node]) and
                        _only_used_by(az, [ab.owner])):
                    continue
                return z, slope, [node, lin.owner, ab.owner, az.owner]
    return None


def _only_used_by(var, nodes):
    return all(client in nodes for client, _ in var.clients)


@local_optimizer([Elemwise])
def local_b200_conv_bias_relu(node):
    """relu(B200Conv2d(x, w) [+ bias.dimshuffle('x', 0, 'x', 'x')]) -> one B200Conv2d with the
    epilogue fused; only when the intermediate values have no other use (in a training graph
    the backward pass reads conv + bias, and the pattern is left alone)."""
    sc = theano.scalar
    slope = 0.0
    leaky = _leaky_relu_argument(node)
    if leaky is not None:
        z, slope, inner = leaky
    else:
        z = _relu_argument(node)
        inner = [node]
    if z is None or z.owner is None:
        return None
    if leaky is None and isinstance(node.op.scalar_op, sc.Mul):
        add = [i for i in node.inputs if _is_elemwise(i, sc.Add)][0]
        ab = [i for i in add.owner.inputs if _is_elemwise(i, sc.Abs)][0]
        inner += [add.owner, ab.owner]
        if not _only_used_by(add, [node]) or not _only_used_by(ab, [add.owner]):
            return None
    conv, bias = z, None
    if _is_elemwise(z, sc.Add) and len(z.owner.inputs) == 2:
        for a, b in (z.owner.inputs, z.owner.inputs[::-1]):
            if (b.owner is not None and isinstance(b.owner.op, DimShuffle) and
                    b.owner.op.new_order == ("x", 0, "x", "x") and a.owner is not None and
                    isinstance(a.owner.op, B200Conv2d)):
                conv, bias = a, b.owner.inputs[0]
        if bias is None:
            return None
        if not _only_used_by(z, inner) or not _only_used_by(conv, [z.owner]):
            return None
    elif not _only_used_by(z, inner):
        return None
    if conv.owner is None or not isinstance(conv.owner.op, B200Conv2d):
        return None
    op = conv.owner.op
    if op.relu or len(conv.owner.inputs) != 2:
        return None
    if bias is not None and bias.dtype != conv.dtype:
        return None
    if bias is not None and (bias.ndim != 1 or bias.broadcastable[0]):
        # a length-1 bias broadcasts over the filters in the unfused graph; the fused epilogue
        # reads one value per filter
        return None
    fused = B200Conv2d(relu=True, slope=slope, **_props(op))
    args = list(conv.owner.inputs) + ([bias] if bias is not None else [])
    return _finish(node, fused(*args))


@local_optimizer(None)
def local_b200_maxpool(node):
    """Pool{ignore_border=True, mode='max'}(y, [2 2], [2 2], [0 0]) on the output of a B200 conv."""
    from theano.tensor.signal.pool import Pool
    if not isinstance(node.op, Pool) or node.op.mode != "max" or not node.op.ignore_border or node.op.ndim != 2:
        return None
    x = node.inputs[0]
    if x.owner is None or not isinstance(x.owner.op, B200Conv2d) or x.ndim != 4:
        return None
    try:
        ws, st, pad = (tuple(int(v) for v in tensor.get_constant_value(i) if True) for i in node.inputs[1:4])
    except Exception:
        try:
            ws, st, pad = (tuple(int(v) for v in i.data) for i in node.inputs[1:4])
        except Exception:
            return None
    if ws != (2, 2) or st != (2, 2) or pad != (0, 0):
        return None
    return _finish(node, B200MaxPool2x2()(x))


def _const_pairs(inputs):
    try:
        return tuple(tuple(int(v) for v in tensor.get_constant_value(i)) for i in inputs)
    except Exception:
        try:
            return tuple(tuple(int(v) for v in i.data) for i in inputs)
        except Exception:
            return None


@local_optimizer(None)
def local_b200_maxpool_grad(node):
    """MaxPoolGrad{ignore_border=True}(x, maxout, gz, [2 2], [2 2], [0 0]) whose x comes from a
    B200 conv (theano/tensor/signal/pool.py:1091): the gradient of the pooling swapped above."""
    from theano.tensor.signal.pool import MaxPoolGrad
    if not isinstance(node.op, MaxPoolGrad) or not node.op.ignore_border or node.op.ndim != 2:
        return None
    x, maxout, gz = node.inputs[:3]
    if x.owner is None or not isinstance(x.owner.op, B200Conv2d) or x.ndim != 4:
        return None
    if not (x.dtype == maxout.dtype == gz.dtype) or x.dtype not in ("float16", "float32"):
        return None
    consts = _const_pairs(node.inputs[3:6])
    if consts != ((2, 2), (2, 2), (0, 0)):
        return None
    return _finish(node, B200MaxPool2x2Grad()(x, maxout, gz))


_registered = False


def register():
    """Idempotent registration in the reference's optimizer databases."""
    global _registered
    if _registered:
        return
    g = nnet_opt.conv_groupopt
    g.register("local_abstractconv_b200", local_abstractconv_b200, TAG, "fast_compile", "fast_run",
               position=-1)
    g.register("local_abstractconv_gradweights_b200", local_abstractconv_gradweights_b200, TAG,
               "fast_compile", "fast_run", position=-1)
    g.register("local_abstractconv_gradinputs_b200", local_abstractconv_gradinputs_b200, TAG,
               "fast_compile", "fast_run", position=-1)
    optdb.register("b200_conv_epilogue", in2out(local_b200_conv_bias_relu, local_b200_maxpool, local_b200_maxpool_grad,
                                               name="b200_conv_epilogue"),
                   48.8, "fast_run", TAG)
    _registered = True


register()
