"""Theano Ops that run the 2-D convolution on a B200 through ``libb200conv``.

``B200Conv2d``, ``B200Conv2d_gradWeights`` and ``B200Conv2d_gradInputs`` keep the
``make_node`` / ``infer_shape`` / ``grad`` / ``connection_pattern`` contracts of the
reference's ``CorrMM``, ``CorrMM_gradWeights`` and ``CorrMM_gradInputs``
(theano/tensor/nnet/corr.py:592,685,801) and take the same parameters
(``border_mode, subsample, filter_dilation, num_groups``) plus ``filter_flip`` of
the abstract ops (theano/tensor/nnet/abstract_conv.py:2063-2156): the flip is done
inside the kernels, so no ``Subtensor`` node is inserted around them.

Execution is ``perform`` -> ``theano_b200.shim`` (ctypes) -> CUDA; there is no C code
for Theano to generate and no CPU implementation: without the library or a B200 the
thunk raises.  Instances hold only their ``__props__`` (no library handles), so
compiled functions stay picklable.

Importing this module needs an importable ``theano``.
"""
import numpy as np
import theano
from theano import Apply, gof
from theano.tensor import TensorType, as_tensor_variable
from theano.tensor.nnet.abstract_conv import get_conv_output_shape

from . import hostlogic, shim

_FLOAT_DTYPES = ("float16", "float32")


class BaseB200Conv(gof.Op):
    """Parameter handling shared by the three ops (mirrors BaseCorrMM, corr.py:20-167)."""
    check_broadcast = False
    __props__ = ("border_mode", "subsample", "filter_dilation", "num_groups", "filter_flip")

    def __init__(self, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
                 filter_flip=True):
        self.border_mode = hostlogic.normalize_border_mode(border_mode)
        if len(subsample) != 2:
            raise ValueError("subsample must have two elements")
        if len(filter_dilation) != 2:
            raise ValueError("filter_dilation must have two elements")
        self.subsample = tuple(int(s) for s in subsample)
        self.filter_dilation = tuple(int(d) for d in filter_dilation)
        if num_groups < 1:
            raise ValueError("Number of groups should be greater than 0")
        self.num_groups = int(num_groups)
        self.filter_flip = bool(filter_flip)

    def __str__(self):
        return "%s{%s, %s, %s, %s, flip=%s}" % (self.__class__.__name__, self.border_mode, self.subsample,
                                                self.filter_dilation, self.num_groups, self.filter_flip)

    def _kwargs(self):
        return dict(border_mode=self.border_mode, subsample=self.subsample,
                    filter_dilation=self.filter_dilation, num_groups=self.num_groups,
                    filter_flip=self.filter_flip)

    @staticmethod
    def as_common_dtype(in1, in2):
        dtype = theano.scalar.upcast(in1.dtype, in2.dtype)
        if dtype not in _FLOAT_DTYPES:
            raise TypeError("B200 convolution handles float16 and float32, got %s" % dtype)
        return in1.astype(dtype), in2.astype(dtype)

    def do_constant_folding(self, node):
        return False

    def flops(self, inp, outp):
        """Same count as the abstract ops report to the profiler (abstract_conv.py:2163-2177)."""
        if isinstance(self, B200Conv2d):
            xs, ws, ys = inp[0], inp[1], outp[0]
        elif isinstance(self, B200Conv2d_gradWeights):
            xs, ws, ys = inp[0], outp[0], inp[1]
        else:
            xs, ws, ys = outp[0], inp[0], inp[1]
        return hostlogic.conv_flops(xs, ws, ys)

    def _pads_symbolic(self):
        """Pads for infer_shape: sentinels -1 (half) / -2 (full) like BaseCorrMM.pad."""
        if self.border_mode == "half":
            return (-1, -1), (-1, -1)
        if self.border_mode == "full":
            return (-2, -2), (-2, -2)
        if self.border_mode == "valid":
            return (0, 0), (0, 0)
        return self.border_mode


class B200Conv2d(BaseB200Conv):
    """Forward convolution, optionally with the bias add and ReLU that follow it fused in.

    ``op(img, kern)`` or ``op(img, kern, bias)``; ``relu=True`` applies the reference's rectifier
    ``0.5 * ((1 + slope) * v + (1 - slope) * abs(v))`` (theano/tensor/nnet/nnet.py:2242-2250;
    ``slope`` 0 is the plain ReLU) to ``conv + bias``.
    """
    __props__ = BaseB200Conv.__props__ + ("relu", "slope")

    def __init__(self, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
                 filter_flip=True, relu=False, slope=0.0):
        super(B200Conv2d, self).__init__(border_mode, subsample, filter_dilation, num_groups, filter_flip)
        self.relu = bool(relu)
        self.slope = float(slope) if self.relu else 0.0

    def __setstate__(self, state):
        self.__dict__.update(state)
        self.__dict__.setdefault("slope", 0.0)

    def make_node(self, img, kern, bias=None):
        img = as_tensor_variable(img)
        kern = as_tensor_variable(kern)
        img, kern = self.as_common_dtype(img, kern)
        if img.type.ndim != 4:
            raise TypeError("img must be 4D tensor")
        if kern.type.ndim != 4:
            raise TypeError("kern must be 4D tensor")
        inputs = [img, kern]
        if bias is not None:
            bias = as_tensor_variable(bias).astype(img.dtype)
            if bias.type.ndim != 1:
                raise TypeError("bias must be a vector")
            inputs.append(bias)
        broadcastable = [img.type.broadcastable[0], kern.type.broadcastable[0], False, False]
        return Apply(self, inputs, [TensorType(img.type.dtype, broadcastable)()])

    def infer_shape(self, node, input_shape):
        return [get_conv_output_shape(input_shape[0], input_shape[1], self.border_mode, self.subsample,
                                      self.filter_dilation)]

    def perform(self, node, inputs, output_storage):
        img, kern = inputs[0], inputs[1]
        bias = inputs[2] if len(inputs) == 3 else None
        out = output_storage[0][0]
        output_storage[0][0] = shim.conv2d_forward(img, kern, bias=bias, relu=self.relu, slope=self.slope,
                                                   out=out, **self._kwargs())

    def grad(self, inp, grads):
        bottom, weights = inp[0], inp[1]
        top, = grads
        if self.relu:
            pos = theano.tensor.gt(self(*inp), 0)      # act(v) > 0 exactly where v > 0 (slope >= 0)
            top = top * (pos + self.slope * (1 - pos)) if self.slope else top * pos
        k = self._kwargs()
        d_bottom = B200Conv2d_gradInputs(**k)(weights, top, bottom.shape[-2:])
        d_weights = B200Conv2d_gradWeights(**k)(bottom, top, weights.shape[-2:])
        res = (d_bottom, d_weights)
        if len(inp) == 3:
            res += (top.sum(axis=(0, 2, 3)),)
        return res


class B200Conv2d_gradWeights(BaseB200Conv):
    """Gradient wrt the filters: ``op(img, topgrad, shape)`` -> [K, C/groups, kH, kW]."""

    def make_node(self, img, topgrad, shape=None):
        img = as_tensor_variable(img)
        topgrad = as_tensor_variable(topgrad)
        img, topgrad = self.as_common_dtype(img, topgrad)
        if img.type.ndim != 4:
            raise TypeError("img must be 4D tensor")
        if topgrad.type.ndim != 4:
            raise TypeError("topgrad must be 4D tensor")
        if shape is None:
            if self.subsample != (1, 1) or self.border_mode == "half":
                raise ValueError('shape must be given if subsample != (1, 1) or border_mode == "half"')
            height_width = []
        else:
            height_width = [as_tensor_variable(shape[0]).astype("int64"),
                            as_tensor_variable(shape[1]).astype("int64")]
        broadcastable = [topgrad.type.broadcastable[1], img.type.broadcastable[1], False, False]
        if self.num_groups > 1:
            broadcastable[1] = False
        return Apply(self, [img, topgrad] + height_width, [TensorType(img.type.dtype, broadcastable)()])

    def infer_shape(self, node, input_shape):
        (ph_l, ph_r), (pw_l, pw_r) = self._pads_symbolic()
        dH, dW = self.subsample
        dilH, dilW = self.filter_dilation
        imshp, topshp = input_shape[0], input_shape[1]
        ssize = imshp[1] // self.num_groups
        nkern = topshp[1]
        hw = node.inputs[2:]

        def ksize(a, p_l, p_r, stride, dil):
            if stride != 1 or p_l == -1 or p_r == -1:
                return hw[a]
            if p_l == -2 or p_r == -2:
                return (2 - imshp[2 + a] + (topshp[2 + a] - 1) * stride - 1) // dil + 1
            return (imshp[2 + a] + p_l + p_r - (topshp[2 + a] - 1) * stride - 1) // dil + 1

        return [(nkern, ssize, ksize(0, ph_l, ph_r, dH, dilH), ksize(1, pw_l, pw_r, dW, dilW))]

    def perform(self, node, inputs, output_storage):
        img, topgrad = inputs[:2]
        kshape = tuple(int(v) for v in inputs[2:]) if len(inputs) == 4 else None
        out = output_storage[0][0]
        output_storage[0][0] = shim.conv2d_grad_weights(img, topgrad, kshape, out=out, **self._kwargs())

    def grad(self, inp, grads):
        bottom, top = inp[:2]
        weights, = grads
        k = self._kwargs()
        d_bottom = B200Conv2d_gradInputs(**k)(weights, top, bottom.shape[-2:])
        d_top = B200Conv2d(**k)(bottom, weights)
        d_hw = (theano.gradient.DisconnectedType()(),) * 2 if len(inp) == 4 else ()
        return (d_bottom, d_top) + d_hw

    def connection_pattern(self, node):
        return [[1], [1]] if node.nin == 2 else [[1], [1], [0], [0]]


class B200Conv2d_gradInputs(BaseB200Conv):
    """Gradient wrt the image: ``op(kern, topgrad, shape)`` -> [N, C, H, W]."""

    def make_node(self, kern, topgrad, shape=None):
        kern = as_tensor_variable(kern)
        topgrad = as_tensor_variable(topgrad)
        kern, topgrad = self.as_common_dtype(kern, topgrad)
        if kern.type.ndim != 4:
            raise TypeError("kern must be 4D tensor")
        if topgrad.type.ndim != 4:
            raise TypeError("topgrad must be 4D tensor")
        if shape is None:
            if self.subsample != (1, 1):
                raise ValueError("shape must be given if subsample != (1, 1)")
            height_width = []
        else:
            height_width = [as_tensor_variable(shape[0]).astype("int64"),
                            as_tensor_variable(shape[1]).astype("int64")]
        if self.num_groups > 1:
            broadcastable = [topgrad.type.broadcastable[0], False, False, False]
        else:
            broadcastable = [topgrad.type.broadcastable[0], kern.type.broadcastable[-3], False, False]
        return Apply(self, [kern, topgrad] + height_width, [TensorType(kern.type.dtype, broadcastable)()])

    def infer_shape(self, node, input_shape):
        (ph_l, ph_r), (pw_l, pw_r) = self._pads_symbolic()
        dH, dW = self.subsample
        dilH, dilW = self.filter_dilation
        kshp, topshp = input_shape[0], input_shape[1]
        ssize = kshp[1] * self.num_groups
        hw = node.inputs[2:]

        def size(a, p_l, p_r, stride, dil):
            if len(hw) == 2:      # a given size always wins (corr.py:492-493)
                return hw[a]
            dil_k = (kshp[2 + a] - 1) * dil + 1
            if p_l == -1 or p_r == -1:
                p_l = p_r = dil_k // 2
            elif p_l == -2 or p_r == -2:
                p_l = p_r = dil_k - 1
            if stride != 1:
                raise ValueError("shape must be given if subsample != (1, 1)")
            return (topshp[2 + a] - 1) * stride + dil_k - p_l - p_r

        return [(topshp[0], ssize, size(0, ph_l, ph_r, dH, dilH), size(1, pw_l, pw_r, dW, dilW))]

    def perform(self, node, inputs, output_storage):
        kern, topgrad = inputs[:2]
        imshape = tuple(int(v) for v in inputs[2:]) if len(inputs) == 4 else None
        out = output_storage[0][0]
        output_storage[0][0] = shim.conv2d_grad_inputs(kern, topgrad, imshape, out=out, **self._kwargs())

    def grad(self, inp, grads):
        weights, top = inp[:2]
        bottom, = grads
        k = self._kwargs()
        d_weights = B200Conv2d_gradWeights(**k)(bottom, top, weights.shape[-2:])
        d_top = B200Conv2d(**k)(bottom, weights)
        d_hw = (theano.gradient.DisconnectedType()(),) * 2 if len(inp) == 4 else ()
        return (d_weights, d_top) + d_hw

    def connection_pattern(self, node):
        return [[1], [1]] if node.nin == 2 else [[1], [1], [0], [0]]


class B200MaxPool2x2(gof.Op):
    """``Pool(ignore_border=True, mode='max')`` with ws = stride = (2, 2) and no padding
    (theano/tensor/signal/pool.py:271), the pooling between VGG blocks."""
    __props__ = ()

    def make_node(self, x):
        x = as_tensor_variable(x)
        if x.type.ndim != 4:
            raise TypeError("x must be 4D tensor")
        if x.dtype not in _FLOAT_DTYPES:
            raise TypeError("B200 pooling handles float16 and float32")
        return Apply(self, [x], [TensorType(x.dtype, (x.broadcastable[0], x.broadcastable[1], False, False))()])

    def infer_shape(self, node, input_shape):
        n, c, h, w = input_shape[0]
        return [(n, c, h // 2, w // 2)]

    def perform(self, node, inputs, output_storage):
        output_storage[0][0] = shim.maxpool2x2(inputs[0])

    def grad(self, inp, grads):
        # ties get the gradient at every maximal position, like the reference's MaxPoolGrad
        # (pool.py:1139-1186)
        x, = inp
        gz, = grads
        return [B200MaxPool2x2Grad()(x, self(x), gz)]


class B200MaxPool2x2Grad(gof.Op):
    """``MaxPoolGrad(ignore_border=True)`` for ws = stride = (2, 2), pad 0
    (theano/tensor/signal/pool.py:1091-1186): inputs (x, maxout, gz), output gx like x."""
    __props__ = ()

    def make_node(self, x, maxout, gz):
        x, maxout, gz = (as_tensor_variable(v) for v in (x, maxout, gz))
        for v in (x, maxout, gz):
            if v.type.ndim != 4:
                raise TypeError("x, maxout and gz must be 4D tensors")
        if x.dtype not in _FLOAT_DTYPES or not (x.dtype == maxout.dtype == gz.dtype):
            raise TypeError("B200 pooling gradient handles float16 and float32, one dtype for all inputs")
        return Apply(self, [x, maxout, gz], [x.type()])

    def infer_shape(self, node, input_shapes):
        return [input_shapes[0]]

    def perform(self, node, inputs, output_storage):
        x, maxout, gz = inputs
        output_storage[0][0] = shim.maxpool2x2_grad(x, maxout, gz)

    def grad(self, inp, grads):
        # second derivative: leave it to the reference's op (pool.py:1177-1186)
        from theano.tensor.signal.pool import DownsampleFactorMaxGradGrad
        import theano.tensor as T
        x, maxout, gz = inp
        ggx, = grads
        return [T.zeros_like(x), T.zeros_like(maxout),
                DownsampleFactorMaxGradGrad(ndim=2, ignore_border=True)(x, maxout, ggx, (2, 2), (2, 2), (0, 0))]
