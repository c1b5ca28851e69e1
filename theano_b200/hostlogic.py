"""Host-side shape logic of the convolution ops (pure Python, no device code).

Mirrors what the reference does around ``corrMM``: border-mode normalisation
(theano/tensor/nnet/corr.py:62-93), resolution of ``'half'``/``'full'`` into
pad widths (corr.py:375-395), kernel-size inference for the weight gradient
(corr.py:340-369), image-size inference for the input gradient
(corr.py:492-493) and the output size with Python floor division
(theano/tensor/nnet/abstract_conv.py:131-155, c_code/corr_gemm.c:175-185).
Errors are raised as the reference raises them (``ValueError`` for geometry).
"""
import numbers


def normalize_border_mode(border_mode):
    """-> 'valid' | 'half' | 'full' | ((pad_top, pad_bottom), (pad_left, pad_right))."""
    if isinstance(border_mode, numbers.Integral):
        if border_mode < 0:
            raise ValueError("invalid border_mode {}, which must be a non-negative integer".format(border_mode))
        return ((int(border_mode),) * 2,) * 2
    if isinstance(border_mode, (tuple, list)):
        border_mode = tuple(border_mode)
        if len(border_mode) != 2:
            raise ValueError("invalid border_mode {} which must be a tuple of length 2".format(border_mode))
        border = ()
        for mode in border_mode:
            if isinstance(mode, (tuple, list)) and len(mode) == 2 and min(mode) >= 0:
                border += ((int(mode[0]), int(mode[1])),)
            elif isinstance(mode, numbers.Integral) and mode >= 0:
                border += ((int(mode), int(mode)),)
            else:
                raise ValueError("invalid border mode {}. The tuple can only contain integers or "
                                 "tuples of length 2".format(border_mode))
        return border
    if border_mode not in ("valid", "full", "half"):
        raise ValueError('invalid border_mode {}, which must be either "valid", "full", "half", an '
                         "integer or a tuple of two integers or a pair of integers".format(border_mode))
    return border_mode


def resolve_pads(border_mode, kshape, dilation):
    """Pad widths ((top, bottom), (left, right)) once the kernel size is known."""
    bm = normalize_border_mode(border_mode)
    dil_k = [(int(kshape[a]) - 1) * int(dilation[a]) + 1 for a in range(2)]
    if bm == "valid":
        return ((0, 0), (0, 0))
    if bm == "half":
        return ((dil_k[0] // 2,) * 2, (dil_k[1] // 2,) * 2)
    if bm == "full":
        return ((dil_k[0] - 1,) * 2, (dil_k[1] - 1,) * 2)
    return bm


def out_size(size, k, dilation, pad, stride):
    """One axis of the forward output shape (floor division also for negative numerators)."""
    return (size + pad[0] + pad[1] - ((k - 1) * dilation + 1)) // stride + 1


def forward_shape(xshape, wshape, border_mode, subsample, dilation, num_groups=1):
    """Output shape of CorrMM(x, w); raises ValueError like corr_gemm.c:164-172, corr.py:408."""
    if len(xshape) != 4:
        raise TypeError("img must be 4D tensor")
    if len(wshape) != 4:
        raise TypeError("kern must be 4D tensor")
    if xshape[1] != wshape[1] * num_groups:
        raise ValueError("CorrMM images and kernel must have the same stack size")
    if wshape[0] % num_groups:
        raise ValueError("CorrMM the number of filters must be divisible by the number of groups")
    pads = resolve_pads(border_mode, wshape[2:], dilation)
    ho = out_size(xshape[2], wshape[2], dilation[0], pads[0], subsample[0])
    wo = out_size(xshape[3], wshape[3], dilation[1], pads[1], subsample[1])
    if ho <= 0 or wo <= 0:
        raise ValueError("CorrMM: impossible output shape\n  bottom shape: %s\n  weights shape: %s\n"
                         "  top shape: %s" % (tuple(xshape), tuple(wshape), (xshape[0], wshape[0], ho, wo)))
    return (xshape[0], wshape[0], ho, wo), pads


def gradweights_kshape(xshape, dyshape, border_mode, subsample, dilation, kshape=None):
    """Kernel height/width for the weight gradient (corr.py:340-369)."""
    bm = normalize_border_mode(border_mode)
    res = []
    for a in range(2):
        if kshape is not None and kshape[a] is not None:
            res.append(int(kshape[a]))
            continue
        if subsample[a] != 1 or bm == "half":
            raise ValueError("shape must be given if subsample != (1, 1) or border_mode == \"half\"")
        if bm == "full":
            k = (2 - xshape[2 + a] + (dyshape[2 + a] - 1) * subsample[a] - 1) // dilation[a] + 1
        else:
            p = (0, 0) if bm == "valid" else bm[a]
            k = (xshape[2 + a] + p[0] + p[1] - (dyshape[2 + a] - 1) * subsample[a] - 1) // dilation[a] + 1
        res.append(int(k))
    if res[0] <= 0 or res[1] <= 0:
        raise ValueError("CorrMM backprop wrt. weights: impossible output shape")
    return tuple(res)


def gradinputs_imshape(wshape, dyshape, border_mode, subsample, dilation, imshape=None):
    """Image height/width for the input gradient (corr.py:492-493)."""
    pads = resolve_pads(border_mode, wshape[2:], dilation)
    res = []
    for a in range(2):
        if imshape is not None and imshape[a] is not None:
            res.append(int(imshape[a]))
        elif subsample[a] != 1:
            raise ValueError("shape must be given if subsample != (1, 1)")
        else:
            res.append((dyshape[2 + a] - 1) * subsample[a] + (wshape[2 + a] - 1) * dilation[a] + 1
                       - pads[a][0] - pads[a][1])
    if res[0] <= 0 or res[1] <= 0:
        raise ValueError("CorrMM backprop wrt. inputs: impossible output shape")
    return tuple(res), pads


def check_consistent(xshape, wshape, dyshape, pads, subsample, dilation, num_groups):
    """The shape test of corr_gemm.c:164-237 (raises ValueError)."""
    if xshape[1] != wshape[1] * num_groups:
        raise ValueError("CorrMM images and kernel must have the same stack size")
    if wshape[0] % num_groups:
        raise ValueError("CorrMM the number of filters must be divisible by the number of groups")
    ho = out_size(xshape[2], wshape[2], dilation[0], pads[0], subsample[0])
    wo = out_size(xshape[3], wshape[3], dilation[1], pads[1], subsample[1])
    exp = (xshape[0], wshape[0], ho, wo)
    if tuple(dyshape) != exp:
        raise ValueError("CorrMM shape inconsistency:\n  bottom shape: %s\n  weight shape: %s\n"
                         "  top shape: %s (expected %s)" % (tuple(xshape), tuple(wshape), tuple(dyshape), exp))


def conv_flops(xshape, wshape, yshape):
    """2*N*K*(C/g)*kH*kW*Ho*Wo, the count the reference profiler uses (abstract_conv.py:2163-2177)."""
    n, k, ho, wo = yshape
    return 2 * n * k * wshape[1] * wshape[2] * wshape[3] * ho * wo
