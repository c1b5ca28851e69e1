"""Device-resident values in Theano graphs: a Type, the two transfer ops, device versions of
the three convolution ops, of the 2x2 pooling and of its gradient, and the graph pass that
chains them.

With the pass enabled (``mode.including('b200_device')``) a graph like

    pool(relu(conv(relu(conv(x, w1) + b1), w2) + b2))

runs as ``HostFromB200(pool(conv(conv(B200FromHost(x), w1, b1), w2, b2)))``: one upload, one
download, activations stay in HBM in channels-last order between the ops.  In a training graph
the gradient ops follow: gradWeights reads the image that the forward pass left in HBM,
gradInputs and the pooling gradient hand their results on in HBM.  Without the pass every
B200 op takes and returns host arrays, like the reference's CPU ops.

The pattern is the reference's own GPU back end: a ``Type`` whose values wrap device memory
(theano/gpuarray/type.py:140-400), ``GpuFromHost`` / ``HostFromGpu``
(theano/gpuarray/basic_ops.py:565-806), and a local optimizer that cancels a transfer pair.
Filters and biases stay ordinary host tensors (shared variables of the user's model); they are
small and are uploaded by the op that uses them.

Importing this module needs an importable ``theano``.
"""
import numpy as np
import theano
from theano import Apply, gof
from theano.gof import local_optimizer
from theano.tensor import TensorType, as_tensor_variable

from . import hostlogic, shim
from .ops import (B200Conv2d, B200Conv2d_gradInputs, B200Conv2d_gradWeights, B200MaxPool2x2,
                  B200MaxPool2x2Grad)

TAG = "b200_device"


class B200TensorType(gof.Type):
    """4-D activation tensor living in HBM (a ``shim.DeviceTensor``, channels-last).

    ``dtype`` and ``broadcastable`` have the meaning they have in ``TensorType``; two types
    are equal when both are."""

    def __init__(self, dtype, broadcastable=(False, False, False, False)):
        self.dtype = str(dtype)
        if self.dtype not in ("float16", "float32"):
            raise TypeError("B200TensorType holds float16 or float32, not %s" % dtype)
        self.broadcastable = tuple(bool(b) for b in broadcastable)
        if len(self.broadcastable) != 4:
            raise TypeError("B200TensorType is 4-dimensional")
        self.ndim = 4

    def __eq__(self, other):
        return type(self) == type(other) and self.dtype == other.dtype and self.broadcastable == other.broadcastable

    def __hash__(self):
        return hash((type(self), self.dtype, self.broadcastable))

    def __str__(self):
        return "B200TensorType{%s, %s}" % (self.dtype, self.broadcastable)

    def filter(self, data, strict=False, allow_downcast=None):
        if isinstance(data, shim.DeviceTensor):
            if str(data.dtype) != self.dtype or len(data.shape) != 4:
                raise TypeError("device tensor of %s / %d dims for %s" % (data.dtype, len(data.shape), self))
        elif strict:
            raise TypeError("%s expects a device tensor, got %s" % (self, type(data)))
        else:
            arr = np.asarray(data)
            if arr.ndim != 4:
                raise TypeError("%s expects 4 dimensions" % self)
            if str(arr.dtype) != self.dtype and not allow_downcast:
                raise TypeError("%s cannot hold %s without a cast" % (self, arr.dtype))
            data = shim.DeviceTensor.from_host(shim.get_context(), arr.astype(self.dtype), "nhwc")
        for dim, b in zip(data.shape, self.broadcastable):
            if b and dim != 1:
                raise TypeError("non-unit size on a broadcastable dimension of %s" % self)
        return data

    @staticmethod
    def values_eq(a, b):
        return a.shape == b.shape and np.array_equal(a.to_host(), b.to_host())

    @staticmethod
    def values_eq_approx(a, b, rtol=1e-3, atol=1e-4):
        return a.shape == b.shape and np.allclose(a.to_host(), b.to_host(), rtol=rtol, atol=atol)

    @staticmethod
    def may_share_memory(a, b):
        return isinstance(a, shim.DeviceTensor) and isinstance(b, shim.DeviceTensor) and a.ptr == b.ptr

    def value_zeros(self, shape):
        t = shim.DeviceTensor(shim.get_context(), shape, self.dtype, "nhwc")
        t.ctx.memset(t.ptr, 0, t.nbytes)
        return t

    def get_shape_info(self, obj):
        return obj.shape

    def get_size(self, shape_info):
        return int(np.prod(shape_info)) * np.dtype(self.dtype).itemsize


class B200Variable(gof.Variable):
    """Variable of a B200TensorType: the attributes the shape machinery of the reference reads
    from tensor variables (theano/tensor/opt.py ShapeFeature)."""
    ndim = property(lambda self: self.type.ndim)
    dtype = property(lambda self: self.type.dtype)
    broadcastable = property(lambda self: self.type.broadcastable)


class B200Constant(gof.Constant):
    ndim = property(lambda self: self.type.ndim)
    dtype = property(lambda self: self.type.dtype)
    broadcastable = property(lambda self: self.type.broadcastable)


B200TensorType.Variable = B200Variable
B200TensorType.Constant = B200Constant


def _host_type(dev_type):
    return TensorType(dev_type.dtype, dev_type.broadcastable)


class B200FromHost(gof.Op):
    """Host array (NCHW) -> device tensor (channels-last); GpuFromHost of the reference
    (theano/gpuarray/basic_ops.py:652)."""
    __props__ = ()

    def make_node(self, x):
        x = as_tensor_variable(x)
        if x.type.ndim != 4 or x.dtype not in ("float16", "float32"):
            raise TypeError("B200FromHost takes a 4-D float16 / float32 tensor")
        return Apply(self, [x], [B200TensorType(x.dtype, x.broadcastable)()])

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = shim.DeviceTensor.from_host(shim.get_context(), inputs[0], "nhwc")

    def infer_shape(self, node, shapes):
        return shapes

    def grad(self, inputs, grads):
        return [HostFromB200()(grads[0])]


class HostFromB200(gof.Op):
    """Device tensor -> host array (NCHW); HostFromGpu of the reference
    (theano/gpuarray/basic_ops.py:565)."""
    __props__ = ()

    def make_node(self, x):
        if not isinstance(x.type, B200TensorType):
            raise TypeError("HostFromB200 takes a device tensor")
        return Apply(self, [x], [_host_type(x.type)()])

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = inputs[0].to_host()

    def infer_shape(self, node, shapes):
        return shapes

    def grad(self, inputs, grads):
        return [B200FromHost()(grads[0])]


class B200DevConv2d(gof.Op):
    """``B200Conv2d`` on a device-resident image: inputs (img: device, kern: host[, bias: host]),
    output a device tensor.  Same properties as ``B200Conv2d`` (ops.py), same epilogue."""
    __props__ = B200Conv2d.__props__
    check_broadcast = False

    def __init__(self, **props):
        self.host_op = B200Conv2d(**props)
        for name in self.__props__:
            setattr(self, name, getattr(self.host_op, name))

    def make_node(self, img, kern, bias=None):
        if not isinstance(img.type, B200TensorType):
            raise TypeError("img must be a device tensor")
        kern = as_tensor_variable(kern)
        if kern.type.ndim != 4:
            raise TypeError("kern must be 4D tensor")
        if kern.dtype != img.type.dtype:
            raise TypeError("img and kern must share one dtype")
        inputs = [img, kern]
        if bias is not None:
            bias = as_tensor_variable(bias)
            if bias.type.ndim != 1 or bias.dtype != img.type.dtype:
                raise TypeError("bias must be a vector of the image's dtype")
            inputs.append(bias)
        bcast = (img.type.broadcastable[0], kern.type.broadcastable[0], False, False)
        return Apply(self, inputs, [B200TensorType(img.type.dtype, bcast)()])

    def infer_shape(self, node, shapes):
        return self.host_op.infer_shape(node, shapes)

    def perform(self, node, inputs, output_storage):
        img, kern = inputs[0], inputs[1]
        ctx = img.ctx
        w = shim.DeviceTensor.from_host(ctx, kern)
        b = None
        if len(inputs) == 3:
            b = shim.DeviceTensor.from_host(ctx, np.asarray(inputs[2]).reshape(1, -1, 1, 1))
        output_storage[0][0] = shim.device_conv2d(img, w, bias=b, relu=self.relu, slope=self.slope,
                                                  out_layout="nhwc", **self.host_op._kwargs())


class B200DevMaxPool2x2(gof.Op):
    """``B200MaxPool2x2`` on a device tensor."""
    __props__ = ()

    def make_node(self, x):
        if not isinstance(x.type, B200TensorType):
            raise TypeError("x must be a device tensor")
        bcast = (x.type.broadcastable[0], x.type.broadcastable[1], False, False)
        return Apply(self, [x], [B200TensorType(x.type.dtype, bcast)()])

    def infer_shape(self, node, shapes):
        n, c, h, w = shapes[0]
        return [(n, c, h // 2, w // 2)]

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = shim.device_maxpool2x2(inputs[0])


class _DevGradBase(gof.Op):
    """Shared parts of the two device gradient ops: the properties of the host op they replace and
    its shape inference (the input positions are the same)."""
    __props__ = B200Conv2d_gradInputs.__props__
    check_broadcast = False
    host_class = None

    def __init__(self, **props):
        self.host_op = self.host_class(**props)
        for name in self.__props__:
            setattr(self, name, getattr(self.host_op, name))

    def infer_shape(self, node, shapes):
        return self.host_op.infer_shape(node, shapes)

    def do_constant_folding(self, node):
        return False


class B200DevConv2d_gradInputs(_DevGradBase):
    """``B200Conv2d_gradInputs`` with the output gradient and the result in HBM:
    inputs (kern: host, topgrad: device[, height, width]), output a device tensor."""
    host_class = B200Conv2d_gradInputs

    def make_node(self, kern, topgrad, *hw):
        if not isinstance(topgrad.type, B200TensorType):
            raise TypeError("topgrad must be a device tensor")
        kern = as_tensor_variable(kern)
        if kern.type.ndim != 4 or kern.dtype != topgrad.type.dtype:
            raise TypeError("kern must be a 4D tensor of the gradient's dtype")
        if len(hw) not in (0, 2):
            raise TypeError("give both height and width, or neither")
        if not hw and self.subsample != (1, 1):
            raise ValueError("shape must be given if subsample != (1, 1)")
        hw = [as_tensor_variable(v).astype("int64") for v in hw]
        chan = False if self.num_groups > 1 else kern.type.broadcastable[-3]
        bcast = (topgrad.type.broadcastable[0], chan, False, False)
        return Apply(self, [kern, topgrad] + hw, [B200TensorType(kern.dtype, bcast)()])

    def perform(self, node, inputs, output_storage):
        kern, topgrad = inputs[:2]
        imshape = tuple(int(v) for v in inputs[2:]) if len(inputs) == 4 else None
        w = shim.DeviceTensor.from_host(topgrad.ctx, kern)
        output_storage[0][0] = shim.device_grad_inputs(w, topgrad, imshape, out_layout="nhwc",
                                                       **self.host_op._kwargs())


class B200DevConv2d_gradWeights(_DevGradBase):
    """``B200Conv2d_gradWeights`` on device-resident activations: inputs (img: device,
    topgrad: device[, height, width]); the filter gradient is small and is returned as a host
    array, where the update rule of the model reads it."""
    host_class = B200Conv2d_gradWeights

    def make_node(self, img, topgrad, *hw):
        for v in (img, topgrad):
            if not isinstance(v.type, B200TensorType):
                raise TypeError("img and topgrad must be device tensors")
        if img.type.dtype != topgrad.type.dtype:
            raise TypeError("img and topgrad must share one dtype")
        if len(hw) not in (0, 2):
            raise TypeError("give both height and width, or neither")
        if not hw and (self.subsample != (1, 1) or self.border_mode == "half"):
            raise ValueError('shape must be given if subsample != (1, 1) or border_mode == "half"')
        hw = [as_tensor_variable(v).astype("int64") for v in hw]
        chan = False if self.num_groups > 1 else img.type.broadcastable[1]
        bcast = (topgrad.type.broadcastable[1], chan, False, False)
        return Apply(self, [img, topgrad] + hw, [TensorType(img.type.dtype, bcast)()])

    def perform(self, node, inputs, output_storage):
        img, topgrad = inputs[:2]
        kshape = tuple(int(v) for v in inputs[2:]) if len(inputs) == 4 else None
        dw = shim.device_grad_weights(img, topgrad, kshape, **self.host_op._kwargs())
        output_storage[0][0] = dw.to_host()


class B200DevMaxPool2x2Grad(gof.Op):
    """``B200MaxPool2x2Grad`` on device tensors (x, maxout, gz) -> gx."""
    __props__ = ()

    def make_node(self, x, maxout, gz):
        for v in (x, maxout, gz):
            if not isinstance(v.type, B200TensorType):
                raise TypeError("x, maxout and gz must be device tensors")
        if not (x.type.dtype == maxout.type.dtype == gz.type.dtype):
            raise TypeError("one dtype for all inputs")
        return Apply(self, [x, maxout, gz], [x.type()])

    def infer_shape(self, node, shapes):
        return [shapes[0]]

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = shim.device_maxpool2x2_grad(*inputs)


class B200DevElemwise(gof.Op):
    """One binary or unary element-wise operation on a device tensor (``shim.device_elementwise``):
    the Elemwise nodes between convolution ops (bias add, rectifier pieces, gradient masks,
    residual add, scale) without a trip to the host, as the reference's GPU back end keeps them
    (theano/gpuarray/elemwise.py:86).  ``kind`` says what the second operand is: 'tensor' (a
    device tensor of the same shape), 'scalar' (a host scalar), 'channel' (a host vector
    broadcast as b.dimshuffle('x', 0, 'x', 'x')) or 'none' (unary)."""
    __props__ = ("op", "kind")

    def __init__(self, op, kind):
        if op not in shim.EW_OPS or kind not in ("tensor", "scalar", "channel", "none"):
            raise ValueError("unknown element-wise device op %r / %r" % (op, kind))
        self.op, self.kind = op, kind

    def make_node(self, a, b=None):
        if not isinstance(a.type, B200TensorType):
            raise TypeError("the first operand must be a device tensor")
        inputs = [a]
        if self.kind == "tensor":
            if not isinstance(b.type, B200TensorType) or b.type.dtype != a.type.dtype:
                raise TypeError("the second operand must be a device tensor of the same dtype")
            inputs.append(b)
        elif self.kind in ("scalar", "channel"):
            b = as_tensor_variable(b)
            if b.type.ndim != (0 if self.kind == "scalar" else 1):
                raise TypeError("second operand has the wrong number of dimensions")
            inputs.append(b)
        elif b is not None:
            raise TypeError("unary op with two operands")
        return Apply(self, inputs, [a.type()])

    def infer_shape(self, node, shapes):
        return [shapes[0]]

    def perform(self, node, inputs, output_storage):
        b = inputs[1] if len(inputs) == 2 else None
        if self.kind == "scalar":
            b = float(np.asarray(b))
        output_storage[0][0] = shim.device_elementwise(self.op, inputs[0], b)


class B200DevChannelSum(gof.Op):
    """Sum{axis=[0, 2, 3]} of a device tensor (the bias gradient): a host vector."""
    __props__ = ()

    def make_node(self, x):
        if not isinstance(x.type, B200TensorType):
            raise TypeError("x must be a device tensor")
        return Apply(self, [x], [TensorType(x.type.dtype, (x.type.broadcastable[1],))()])

    def infer_shape(self, node, shapes):
        return [(shapes[0][1],)]

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = shim.device_channel_sum(inputs[0])


# ---- the graph pass ---------------------------------------------------------------------
def _on_device(var):
    """The device variable behind a host variable produced by HostFromB200, else a fresh upload."""
    if var.owner is not None and isinstance(var.owner.op, HostFromB200):
        return var.owner.inputs[0]
    return B200FromHost()(var)


def _back(node, dev_out):
    from theano.gof.opt import copy_stack_trace
    host = HostFromB200()(dev_out)
    if host.type != node.outputs[0].type:
        host = theano.tensor.patternbroadcast(host, node.outputs[0].broadcastable)
    copy_stack_trace(node.outputs[0], host)
    return [host]


@local_optimizer([B200Conv2d])
def local_b200_conv_to_device(node):
    """B200Conv2d(img, kern[, bias]) -> HostFromB200(B200DevConv2d(device(img), kern[, bias]));
    device(img) reuses the producer's device tensor when img itself came from a device op."""
    if not isinstance(node.op, B200Conv2d):
        return None
    op = node.op
    dev = B200DevConv2d(**{name: getattr(op, name) for name in B200Conv2d.__props__})
    img = node.inputs[0]
    if img.dtype != node.inputs[1].dtype:
        return None
    return _back(node, dev(_on_device(img), *node.inputs[1:]))


@local_optimizer([B200MaxPool2x2])
def local_b200_pool_to_device(node):
    if not isinstance(node.op, B200MaxPool2x2):
        return None
    return _back(node, B200DevMaxPool2x2()(_on_device(node.inputs[0])))


def _props(op):
    return {name: getattr(op, name) for name in B200Conv2d_gradInputs.__props__}


@local_optimizer([B200Conv2d_gradInputs])
def local_b200_gradinputs_to_device(node):
    """gradInputs takes its output gradient from HBM when it is there already and leaves its
    result there for the next device op (a transfer pair around it costs what the host op's own
    copies cost, so the rewrite never loses)."""
    if not isinstance(node.op, B200Conv2d_gradInputs):
        return None
    if node.inputs[0].dtype != node.inputs[1].dtype:
        return None
    dev = B200DevConv2d_gradInputs(**_props(node.op))
    return _back(node, dev(node.inputs[0], _on_device(node.inputs[1]), *node.inputs[2:]))


@local_optimizer([B200Conv2d_gradWeights])
def local_b200_gradweights_to_device(node):
    """gradWeights reads whichever of its two activations are in HBM already in place (the image
    that the forward pass produced there, above all) and uploads the other."""
    if not isinstance(node.op, B200Conv2d_gradWeights):
        return None
    img, top = node.inputs[:2]
    if img.dtype != top.dtype:
        return None
    dev = B200DevConv2d_gradWeights(**_props(node.op))
    out = dev(_on_device(img), _on_device(top), *node.inputs[2:])
    if out.type != node.outputs[0].type:
        out = theano.tensor.patternbroadcast(out, node.outputs[0].broadcastable)
    from theano.gof.opt import copy_stack_trace
    copy_stack_trace(node.outputs[0], out)
    return [out]


@local_optimizer([B200MaxPool2x2Grad])
def local_b200_poolgrad_to_device(node):
    if not isinstance(node.op, B200MaxPool2x2Grad):
        return None
    return _back(node, B200DevMaxPool2x2Grad()(*[_on_device(v) for v in node.inputs]))


def _device_backed(var):
    return var.owner is not None and isinstance(var.owner.op, HostFromB200)


def _scalar_operand(var):
    """The 0-d variable behind an operand that broadcasts one value over the whole tensor."""
    if all(var.broadcastable):
        return var.dimshuffle() if var.ndim else var
    return None


def _channel_operand(var):
    """The vector behind b.dimshuffle('x', 0, 'x', 'x')."""
    from theano.tensor.elemwise import DimShuffle
    if (var.owner is not None and isinstance(var.owner.op, DimShuffle) and
            var.owner.op.new_order == ("x", 0, "x", "x") and not var.owner.inputs[0].broadcastable[0]):
        return var.owner.inputs[0]
    return None


_BINARY = {"Add": ("add", "add"), "Mul": ("mul", "mul"), "Sub": ("sub", "rsub"), "TrueDiv": ("div", "rdiv"),
           "Maximum": ("max", "max")}
_UNARY = {"Abs": "abs", "Sgn": "sgn", "Neg": "neg"}


@local_optimizer(None)
def local_b200_elemwise_to_device(node):
    """Elemwise{add, mul, sub, true_div, maximum, abs_, sgn, neg} whose result is a full 4-D
    float16 / float32 tensor and one of whose operands already lives in HBM -> a chain of
    B200DevElemwise ops on that device tensor.  The other operands may be tensors of the same
    shape (uploaded if they are host values), values broadcast over everything, or per-channel
    vectors.  The pass runs before the reference's Elemwise fusion, so the nodes are the plain
    scalar operations."""
    from theano.tensor.elemwise import Elemwise
    if not isinstance(node.op, Elemwise) or len(node.outputs) != 1:
        return None
    out = node.outputs[0]
    if out.ndim != 4 or out.dtype not in ("float16", "float32") or any(out.broadcastable):
        return None
    name = type(node.op.scalar_op).__name__
    ins = list(node.inputs)
    if any(v.dtype != out.dtype for v in ins):
        return None
    full = [v for v in ins if v.ndim == 4 and not any(v.broadcastable)]
    if not any(_device_backed(v) for v in full):
        return None
    if name in _UNARY:
        return _back(node, B200DevElemwise(_UNARY[name], "none")(_on_device(ins[0])))
    if name not in _BINARY or len(ins) < 2:
        return None
    if name in ("Sub", "TrueDiv", "Maximum") and len(ins) != 2:
        return None
    fwd, rev = _BINARY[name]

    def classify(v):
        if v.ndim == 4 and not any(v.broadcastable):
            return "tensor", v
        s = _scalar_operand(v)
        if s is not None:
            return "scalar", s
        c = _channel_operand(v)
        if c is not None:
            return "channel", c
        return None, None

    kinds = [classify(v) for v in ins]
    if any(k is None for k, _ in kinds):
        return None
    # start from a device-backed tensor operand; for the ordered ops it must be the first or the second
    first = next(i for i, v in enumerate(ins) if kinds[i][0] == "tensor" and _device_backed(v))
    acc = _on_device(ins[first])
    if name in ("Sub", "TrueDiv"):
        other = 1 - first
        kind, val = kinds[other]
        opname = fwd if first == 0 else rev
        acc = B200DevElemwise(opname, kind)(acc, _on_device(val) if kind == "tensor" else val)
        return _back(node, acc)
    for i, (kind, val) in enumerate(kinds):
        if i == first:
            continue
        acc = B200DevElemwise(fwd, kind)(acc, _on_device(val) if kind == "tensor" else val)
    return _back(node, acc)


@local_optimizer(None)
def local_b200_channel_sum_to_device(node):
    """Sum{axis=[0, 2, 3]} of a tensor that lives in HBM (the bias gradient of a convolution
    layer) -> B200DevChannelSum."""
    from theano.tensor.elemwise import Sum
    if not isinstance(node.op, Sum) or node.op.axis is None or tuple(sorted(node.op.axis)) != (0, 2, 3):
        return None
    x = node.inputs[0]
    if x.ndim != 4 or x.dtype not in ("float16", "float32") or not _device_backed(x):
        return None
    if node.outputs[0].dtype != x.dtype:
        return None
    out = B200DevChannelSum()(_on_device(x))
    if out.type != node.outputs[0].type:
        return None
    from theano.gof.opt import copy_stack_trace
    copy_stack_trace(node.outputs[0], out)
    return [out]


@local_optimizer([B200FromHost])
def local_cut_b200_transfers(node):
    """B200FromHost(HostFromB200(x)) -> x (the cut of the reference's local_cut_gpu_transfers,
    theano/gpuarray/opt.py)."""
    if not isinstance(node.op, B200FromHost):
        return None
    x = node.inputs[0]
    if x.owner is not None and isinstance(x.owner.op, HostFromB200):
        src = x.owner.inputs[0]
        if src.type == node.outputs[0].type:
            return [src]
    return None


_registered = False


def register():
    """Registers the pass in optdb after the epilogue fusion (48.8) under the tag ``b200_device``
    only: it is switched on with ``mode.including('b200_device')``."""
    global _registered
    if _registered:
        return
    from theano.compile import optdb
    from theano.gof.opt import in2out
    from . import opt as _opt  # noqa: F401  (the lowering and fusion passes must be registered first)
    optdb.register("b200_device_residency",
                   in2out(local_b200_conv_to_device, local_b200_pool_to_device,
                          local_b200_gradinputs_to_device, local_b200_gradweights_to_device,
                          local_b200_poolgrad_to_device, local_b200_elemwise_to_device,
                          local_b200_channel_sum_to_device, local_cut_b200_transfers,
                          name="b200_device_residency"),
                   48.9, TAG)
    _registered = True


register()
