"""ctypes front end of the CPU oracle (test infrastructure, not product code).

Restates, on top of ``corr_oracle.c``, what the reference ops
``CorrMM`` / ``CorrMM_gradWeights`` / ``CorrMM_gradInputs``
(theano/tensor/nnet/corr.py:592,685,801) compute, including the host logic of
``c_code_helper`` (corr.py:340-533): kernel-size inference for the weight
gradient, ``half``/``full`` padding and the output shape of each direction.

The ``conv2d*`` helpers add the kernel flip that the lowering optimizers
insert around the CorrMM ops (theano/tensor/nnet/opt.py:84-92,136-147,196-204),
so they match ``AbstractConv2d(filter_flip=...)`` and its two gradients.

Parity pin: ``tests/golden/make_golden.py`` runs the reference itself (imported
from its source tree) on seeded inputs and stores its outputs; the non-GPU tests
check this oracle against those files and against the known answers in the
reference's own tests.
"""
import ctypes
import glob
import os
import sys

import numpy as np

from . import build_oracle

_LIBS = {}
_BLAS_KEEPALIVE = []


def _find_blas(real):
    """Look for a Fortran-interface LP64 gemm in the wheels' bundled OpenBLAS."""
    sym = "sgemm_" if real == "float" else "dgemm_"
    cands = []
    for sp in sys.path:
        cands += glob.glob(os.path.join(sp, "scipy.libs", "libscipy_openblas-*.so"))
        cands += glob.glob(os.path.join(sp, "opencv_python_headless.libs", "libopenblasp-*.so"))
    for path in cands:
        try:
            lib = ctypes.CDLL(path)
        except OSError:
            continue
        for prefix in ("scipy_", ""):
            try:
                fn = getattr(lib, prefix + sym)
            except AttributeError:
                continue
            setter = None
            for sname in (prefix + "openblas_set_num_threads", "openblas_set_num_threads"):
                try:
                    setter = getattr(lib, sname)
                    break
                except AttributeError:
                    pass
            _BLAS_KEEPALIVE.append(lib)
            return fn, setter, path
    return None, None, None


def lib(real="float"):
    """Load (building if needed) the oracle for ``real`` and hand it a BLAS gemm if one is found."""
    if real in _LIBS:
        return _LIBS[real]
    build_oracle.build()
    L = ctypes.CDLL(build_oracle.lib_path(real))
    L.oracle_corr.restype = ctypes.c_int
    L.oracle_corr.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 3 + [ctypes.c_int] * 18
    L.oracle_out_size.restype = ctypes.c_int
    L.oracle_out_size.argtypes = [ctypes.c_int] * 6
    L.oracle_maxpool2x2.restype = None
    L.oracle_maxpool2x2.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 4
    L.oracle_set_gemm.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    L.blas_fn, L.blas_setter, L.blas_path = _find_blas(real)
    _LIBS[real] = L
    use_blas(True, real)
    return L


def use_blas(on, real="float"):
    """Switch between the bundled OpenBLAS gemm and the portable C loops."""
    L = lib(real)
    if on and L.blas_fn is not None:
        L.oracle_set_gemm(ctypes.cast(L.blas_fn, ctypes.c_void_p),
                          ctypes.cast(L.blas_setter, ctypes.c_void_p) if L.blas_setter else None)
    else:
        L.oracle_set_gemm(None, None)
    return bool(L.oracle_has_ext_gemm())


def threads():
    return lib().oracle_max_threads()


def set_threads(n, real="float"):
    """Number of OpenMP threads the oracle uses (launchers often export OMP_NUM_THREADS=1)."""
    lib(real).oracle_set_threads(int(n))
    return threads()


def _np_real(real):
    return np.float32 if real == "float" else np.float64


def _norm_border(border_mode):
    """border_mode -> 'valid' | 'half' | 'full' | ((pt, pb), (pl, pr)), as corr.py:62-93."""
    if isinstance(border_mode, (int, np.integer)):
        if border_mode < 0:
            raise ValueError("invalid border_mode %r" % (border_mode,))
        return ((int(border_mode),) * 2,) * 2
    if isinstance(border_mode, tuple):
        if len(border_mode) != 2:
            raise ValueError("invalid border_mode %r" % (border_mode,))
        out = ()
        for m in border_mode:
            if isinstance(m, tuple) and len(m) == 2 and min(m) >= 0:
                out += ((int(m[0]), int(m[1])),)
            elif not isinstance(m, tuple) and m >= 0:
                out += ((int(m), int(m)),)
            else:
                raise ValueError("invalid border_mode %r" % (border_mode,))
        return out
    if border_mode not in ("valid", "half", "full"):
        raise ValueError("invalid border_mode %r" % (border_mode,))
    return border_mode


def _pads(border_mode, kshape, dilation):
    """Resolved ((pt, pb), (pl, pr)) for a known kernel size (corr.py:375-395)."""
    bm = _norm_border(border_mode)
    dk = [(kshape[i] - 1) * dilation[i] + 1 for i in range(2)]
    if bm == "valid":
        return ((0, 0), (0, 0))
    if bm == "half":
        return ((dk[0] // 2,) * 2, (dk[1] // 2,) * 2)
    if bm == "full":
        return ((dk[0] - 1,) * 2, (dk[1] - 1,) * 2)
    return bm


def _call(direction, bottom, weight, top, sub, dil, pads, groups, real):
    N, C, H, W = bottom.shape
    K, _, kH, kW = weight.shape
    _, _, Ho, Wo = top.shape
    for a in (bottom, weight, top):
        assert a.flags.c_contiguous and a.dtype == _np_real(real)
    rc = lib(real).oracle_corr(direction, bottom.ctypes.data, weight.ctypes.data, top.ctypes.data,
                               N, C, H, W, K, kH, kW, Ho, Wo, sub[0], sub[1], dil[0], dil[1],
                               pads[0][0], pads[0][1], pads[1][0], pads[1][1], groups)
    if rc == -1:
        raise ValueError("CorrMM shape inconsistency")
    if rc != 0:
        raise RuntimeError("oracle failed with code %d" % rc)


def corr_fwd(x, w, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
             real="float"):
    """CorrMM (corr.py:592): cross-correlation, no kernel flip."""
    dt = _np_real(real)
    x = np.ascontiguousarray(x, dtype=dt)
    w = np.ascontiguousarray(w, dtype=dt)
    if x.ndim != 4 or w.ndim != 4:
        raise TypeError("img and kern must be 4D")
    if x.shape[1] != w.shape[1] * num_groups:
        raise ValueError("CorrMM images and kernel must have the same stack size")
    if w.shape[0] % num_groups:
        raise ValueError("CorrMM the number of filters must be divisible by the number of groups")
    pads = _pads(border_mode, w.shape[2:], filter_dilation)
    L = lib(real)
    Ho = L.oracle_out_size(x.shape[2], w.shape[2], filter_dilation[0], pads[0][0], pads[0][1], subsample[0])
    Wo = L.oracle_out_size(x.shape[3], w.shape[3], filter_dilation[1], pads[1][0], pads[1][1], subsample[1])
    if Ho <= 0 or Wo <= 0:
        raise ValueError("CorrMM: impossible output shape")
    y = np.empty((x.shape[0], w.shape[0], Ho, Wo), dt)
    _call(0, x, w, y, subsample, filter_dilation, pads, num_groups, real)
    return y


def corr_grad_weights(x, dy, kshape=None, border_mode="valid", subsample=(1, 1),
                      filter_dilation=(1, 1), num_groups=1, real="float"):
    """CorrMM_gradWeights (corr.py:685); kernel size inferred as corr.py:340-369."""
    dt = _np_real(real)
    x = np.ascontiguousarray(x, dtype=dt)
    dy = np.ascontiguousarray(dy, dtype=dt)
    bm = _norm_border(border_mode)
    ksz = []
    for a in range(2):
        if kshape is not None:        # a given size always wins (corr.py:346-349)
            ksz.append(int(kshape[a]))
            continue
        if subsample[a] != 1 or bm == "half":
            raise ValueError("shape must be given if subsample != (1, 1) or border_mode == 'half'")
        if bm == "full":
            k = (2 - x.shape[2 + a] + (dy.shape[2 + a] - 1) * subsample[a] - 1) // filter_dilation[a] + 1
        else:
            p = (0, 0) if bm == "valid" else bm[a]
            k = (x.shape[2 + a] + p[0] + p[1] - (dy.shape[2 + a] - 1) * subsample[a] - 1) // filter_dilation[a] + 1
        ksz.append(int(k))
    if ksz[0] <= 0 or ksz[1] <= 0:
        raise ValueError("CorrMM backprop wrt. weights: impossible output shape")
    pads = _pads(bm, ksz, filter_dilation)
    dw = np.empty((dy.shape[1], x.shape[1] // num_groups, ksz[0], ksz[1]), dt)
    if x.shape[0] != dy.shape[0]:
        raise ValueError("CorrMM shape inconsistency")
    _call(1, x, dw, dy, subsample, filter_dilation, pads, num_groups, real)
    return dw


def corr_grad_inputs(w, dy, imshape=None, border_mode="valid", subsample=(1, 1),
                     filter_dilation=(1, 1), num_groups=1, real="float"):
    """CorrMM_gradInputs (corr.py:801); image size as corr.py:492-493."""
    dt = _np_real(real)
    w = np.ascontiguousarray(w, dtype=dt)
    dy = np.ascontiguousarray(dy, dtype=dt)
    pads = _pads(border_mode, w.shape[2:], filter_dilation)
    hw = []
    for a in range(2):
        if imshape is not None:       # a given size always wins (corr.py:492-493)
            hw.append(int(imshape[a]))
        elif subsample[a] != 1:
            raise ValueError("shape must be given if subsample != (1, 1)")
        else:
            hw.append((dy.shape[2 + a] - 1) * subsample[a] + (w.shape[2 + a] - 1) * filter_dilation[a]
                      + 1 - pads[a][0] - pads[a][1])
    if hw[0] <= 0 or hw[1] <= 0:
        raise ValueError("CorrMM backprop wrt. inputs: impossible output shape")
    if w.shape[0] != dy.shape[1]:
        raise ValueError("CorrMM shape inconsistency")
    dx = np.empty((dy.shape[0], w.shape[1] * num_groups, hw[0], hw[1]), dt)
    _call(2, dx, w, dy, subsample, filter_dilation, pads, num_groups, real)
    return dx


def _flip(w):
    return w[:, :, ::-1, ::-1]


def conv2d(x, w, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
           filter_flip=True, real="float"):
    """AbstractConv2d as lowered by local_abstractconv_gemm (nnet/opt.py:70-95)."""
    return corr_fwd(x, _flip(w) if filter_flip else w, border_mode, subsample, filter_dilation,
                    num_groups, real)


def conv2d_grad_weights(x, dy, kshape, border_mode="valid", subsample=(1, 1),
                        filter_dilation=(1, 1), num_groups=1, filter_flip=True, real="float"):
    """AbstractConv2d_gradWeights as lowered at nnet/opt.py:123-151 (flip of the result)."""
    dw = corr_grad_weights(x, dy, kshape, border_mode, subsample, filter_dilation, num_groups, real)
    return np.ascontiguousarray(_flip(dw)) if filter_flip else dw


def conv2d_grad_inputs(w, dy, imshape, border_mode="valid", subsample=(1, 1),
                       filter_dilation=(1, 1), num_groups=1, filter_flip=True, real="float"):
    """AbstractConv2d_gradInputs as lowered at nnet/opt.py:182-207 (flip of the kernel)."""
    return corr_grad_inputs(_flip(w) if filter_flip else w, dy, imshape, border_mode, subsample,
                            filter_dilation, num_groups, real)


def bias_relu(y, bias=None, relu=False):
    """Elemwise epilogue y + b[None,:,None,None], then relu(x) = 0.5*(x+|x|) (nnet/nnet.py:2242)."""
    if bias is not None:
        y = y + np.asarray(bias, y.dtype).reshape(1, -1, 1, 1)
    if relu:
        y = (0.5 * (y + np.abs(y))).astype(y.dtype)
    return y


def maxpool2x2(x, real="float"):
    dt = _np_real(real)
    x = np.ascontiguousarray(x, dtype=dt)
    N, C, H, W = x.shape
    y = np.empty((N, C, H // 2, W // 2), dt)
    lib(real).oracle_maxpool2x2(x.ctypes.data, y.ctypes.data, N, C, H, W)
    return y


def rel_err(a, b):
    """max|a-b| / max|b|: the error measure used by every parity test."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    if a.shape != b.shape:
        raise AssertionError("shape mismatch %r vs %r" % (a.shape, b.shape))
    if b.size == 0:
        return 0.0
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / (den if den > 0 else 1.0))


def maxpool2x2_grad(x, y, gy):
    """MaxPoolGrad.perform for ws = stride = (2, 2), pad 0, ignore_border=True
    (theano/tensor/signal/pool.py:1139-1186): inside every window the positions whose value
    equals the pooled maximum receive the window's gy; positions no window covers get 0."""
    x, y, gy = np.asarray(x), np.asarray(y), np.asarray(gy)
    n, c, h, w = x.shape
    ho, wo = h // 2, w // 2
    gx = np.zeros_like(x)
    for i in range(2):
        for j in range(2):
            win = x[:, :, i:2 * ho:2, j:2 * wo:2]
            gx[:, :, i:2 * ho:2, j:2 * wo:2] = np.where(win == y, gy, np.zeros_like(gy))
    return gx



def epilogue(y, bias=None, residual=None, alpha=1.0, beta=1.0, relu=False, slope=0.0):
    """act(alpha * y + bias + beta * residual) with the reference's leaky ReLU
    0.5 * ((1 + slope) * v + (1 - slope) * |v|) (theano/tensor/nnet/nnet.py:2242-2250)."""
    v = np.asarray(y, np.float64) * alpha
    if bias is not None:
        v = v + np.asarray(bias, np.float64).reshape(1, -1, 1, 1)
    if residual is not None:
        v = v + beta * np.asarray(residual, np.float64)
    if relu:
        v = 0.5 * ((1 + slope) * v + (1 - slope) * np.abs(v))
    return v.astype(np.asarray(y).dtype)
