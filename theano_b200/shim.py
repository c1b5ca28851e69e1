"""ctypes binding of ``libb200conv.so`` and the numpy-level convolution calls.

This is the layer the Theano ops call from ``perform``: numpy arrays in the
reference's layouts (NCHW images, OIHW filters) go in, numpy arrays come out.
Nothing here computes a convolution on the CPU; without the CUDA library or a
B200 every call raises.

Semantics follow the reference ops (theano/tensor/nnet/corr.py:592,685,801)
plus the ``filter_flip`` of the abstract ops they are lowered from
(theano/tensor/nnet/abstract_conv.py:2454,2737,3041).
"""
import ctypes
import os
import threading

import numpy as np

from . import hostlogic

_HERE = os.path.dirname(os.path.abspath(__file__))
# B200CONV_LIB selects another build of the same library (the range-checked debug build)
LIB_PATH = os.environ.get("B200CONV_LIB") or os.path.join(_HERE, "libb200conv.so")

F32, F16 = 0, 1
HOST_PTRS, RELU, IN_NHWC, OUT_NHWC, IN2_NHWC = 1, 2, 4, 8, 16
FORCE_DIRECT, FORCE_UMMA, ATOMIC_SPLITK, NO_SLAB, NO_GROUP, NO_MERGE_PARITY, NO_S2D = 32, 64, 128, 256, 512, 1024, 2048
DW_F32 = 4096
POOL2X2 = 8192

E_INVALID, E_CUDA, E_NOMEM, E_TIMEOUT, E_UNSUPPORTED, E_NCCL = -1, -2, -3, -4, -5, -6


class Desc(ctypes.Structure):
    """``b200conv_desc`` of include/b200conv.h."""
    _fields_ = [(n, ctypes.c_int32) for n in (
        "N", "C", "H", "W", "K", "kH", "kW", "Ho", "Wo", "sH", "sW", "dilH", "dilW",
        "padH_l", "padH_r", "padW_l", "padW_r", "groups", "flip", "dtype")]


# name -> (restype, argtypes); also the list of symbols the header declares
_P, _I, _SZ = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_DESC = ctypes.POINTER(Desc)
SIGNATURES = {
    "b200conv_create": (_I, [_I, ctypes.POINTER(_P)]),
    "b200conv_destroy": (None, [_P]),
    "b200conv_last_error": (_I, [_P, ctypes.c_char_p, _SZ]),
    "b200conv_create_error": (_I, [ctypes.c_char_p, _SZ]),
    "b200conv_version": (ctypes.c_char_p, []),
    "b200conv_fwd": (_I, [_P, _DESC, _P, _P, _P, _P, _I]),
    "b200conv_fwd_epilogue": (_I, [_P, _DESC, _P, _P, _P, _P, _P, ctypes.c_float, ctypes.c_float, ctypes.c_float, _I]),
    "b200conv_dgrad": (_I, [_P, _DESC, _P, _P, _P, _I]),
    "b200conv_wgrad": (_I, [_P, _DESC, _P, _P, _P, _I]),
    "b200conv_wgrad_static": (_I, [_P, _DESC, _P, _P, _P, _I]),
    "b200conv_prepack": (_I, [_P, _I, _DESC, ctypes.POINTER(_P), _I]),
    "b200conv_filters_changed": (_I, [_P, _P]),
    "b200conv_maxpool2x2": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "b200conv_maxpool2x2_grad": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I]),
    "b200conv_elementwise": (_I, [_P, _I, _P, _P, _P, ctypes.c_longlong, _I, _I, ctypes.c_float, _I]),
    "b200conv_channel_sum": (_I, [_P, _P, _P, ctypes.c_longlong, _I, _I]),
    "b200conv_padded_channels": (_I, [_I, _I]),
    "b200conv_malloc": (_I, [_P, _SZ, ctypes.POINTER(_P)]),
    "b200conv_free": (_I, [_P, _P]),
    "b200conv_host_alloc": (_I, [_P, _SZ, ctypes.POINTER(_P)]),
    "b200conv_host_free": (_I, [_P, _P]),
    "b200conv_memcpy_h2d": (_I, [_P, _P, _P, _SZ]),
    "b200conv_memcpy_d2h": (_I, [_P, _P, _P, _SZ]),
    "b200conv_memcpy_h2d_bg": (_I, [_P, _P, _P, _SZ]),
    "b200conv_join_uploads": (_I, [_P]),
    "b200conv_memcpy_d2h_bg": (_I, [_P, _P, _P, _SZ]),
    "b200conv_memset": (_I, [_P, _P, _I, _SZ]),
    "b200conv_sync": (_I, [_P]),
    "b200conv_nchw_to_nhwc": (_I, [_P, _P, _P, _I, _I, _I, _I, _I]),
    "b200conv_nhwc_to_nchw": (_I, [_P, _P, _P, _I, _I, _I, _I, _I]),
    "b200conv_graph_begin": (_I, [_P]),
    "b200conv_graph_end": (_I, [_P, ctypes.POINTER(_P)]),
    "b200conv_graph_launch": (_I, [_P, _P]),
    "b200conv_graph_destroy": (_I, [_P, _P]),
    "b200conv_timer_start": (_I, [_P]),
    "b200conv_timer_stop": (_I, [_P, ctypes.POINTER(ctypes.c_float)]),
    "b200conv_launch_count": (ctypes.c_longlong, [_P]),
    "b200conv_kernel_timing": (_I, [_P, _I]),
    "b200conv_kernel_time": (_I, [_P, ctypes.c_char_p, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_I)]),
    "b200conv_set_autotune": (_I, [_P, _I]),
    "b200conv_debug_trace": (_I, [_P, _P]),
    "b200conv_set_splits": (_I, [_P, _I]),
    "b200conv_set_pair_kernels": (_I, [_P, _I]),
    "b200conv_set_stacked_taps": (_I, [_P, _I]),
    "b200conv_tuning_save": (_I, [_P, ctypes.c_char_p]),
    "b200conv_tuning_load": (_I, [_P, ctypes.c_char_p, ctypes.POINTER(_I)]),
    "b200conv_memory_info": (_I, [_P, ctypes.POINTER(_SZ), ctypes.POINTER(_SZ)]),
    "b200conv_set_wait_limit": (_I, [_P, ctypes.c_longlong]),
    "b200conv_selftest_wait": (_I, [_P]),
    "b200conv_last_algo": (ctypes.c_char_p, [_P]),
    "b200conv_flush_l2": (_I, [_P]),
    "b200conv_nccl_unique_id": (_I, [_P, _P]),
    "b200conv_nccl_init": (_I, [_P, _I, _I, _P]),
    "b200conv_allreduce_sum": (_I, [_P, _P, _SZ, _I]),
    "b200conv_allreduce_sum_async": (_I, [_P, _P, _SZ, _I]),
    "b200conv_comm_wait": (_I, [_P]),
    "b200conv_set_comm_timeout": (_I, [_P, _I]),
    "b200conv_set_sm_count": (_I, [_P, _I]),
    "b200conv_barrier": (_I, [_P]),
    "b200conv_nccl_destroy": (_I, [_P]),
}

_lib = None
_lib_lock = threading.Lock()


def load_library():
    """dlopen the CUDA library (no GPU needed for this step) and type its entry points."""
    global _lib
    with _lib_lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError("libb200conv.so is not built: run `python -m theano_b200.build`")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
    return _lib


class B200Error(RuntimeError):
    pass


def _dtype_code(dt):
    dt = np.dtype(dt)
    if dt == np.float32:
        return F32
    if dt == np.float16:
        return F16
    raise TypeError("b200conv handles float32 and float16, not %s" % dt)


class Context(object):
    """One ``b200conv_ctx``: a device, a stream, pooled memory."""

    def __init__(self, device=0):
        self.lib = load_library()
        h = _P()
        rc = self.lib.b200conv_create(int(device), ctypes.byref(h))
        if rc != 0:
            buf = ctypes.create_string_buffer(512)
            self.lib.b200conv_create_error(buf, 512)
            raise B200Error("cannot open CUDA device %d: %s" % (device, buf.value.decode()))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.b200conv_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- error mapping: geometry errors are ValueError like the reference's, the rest RuntimeError
    def check(self, rc):
        if rc == 0:
            return
        buf = ctypes.create_string_buffer(1024)
        self.lib.b200conv_last_error(self.h, buf, 1024)
        msg = buf.value.decode(errors="replace")
        if rc == E_INVALID:
            raise ValueError("CorrMM (b200conv): " + msg)
        if rc == E_NOMEM:
            raise MemoryError("b200conv: " + msg)
        raise B200Error("b200conv error %d: %s" % (rc, msg))

    # -- memory ----------------------------------------------------------------------------
    def malloc(self, nbytes):
        p = _P()
        self.check(self.lib.b200conv_malloc(self.h, int(nbytes), ctypes.byref(p)))
        return p.value

    def free(self, ptr):
        self.check(self.lib.b200conv_free(self.h, _P(ptr)))

    def pinned_empty(self, shape, dtype):
        """numpy array backed by page-locked host memory (freed with the array)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * dtype.itemsize
        p = _P()
        self.check(self.lib.b200conv_host_alloc(self.h, max(n, 1), ctypes.byref(p)))
        buf = (ctypes.c_char * max(n, 1)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        arr = arr.view(_PinnedArray)
        arr._owner = _PinnedOwner(self, p.value)
        return arr

    def h2d(self, dptr, arr):
        arr = np.ascontiguousarray(arr)
        self.check(self.lib.b200conv_memcpy_h2d(self.h, _P(dptr), _P(arr.ctypes.data), arr.nbytes))
        return arr  # caller keeps it alive until sync

    def d2h(self, arr, dptr):
        assert arr.flags.c_contiguous
        self.check(self.lib.b200conv_memcpy_d2h(self.h, _P(arr.ctypes.data), _P(dptr), arr.nbytes))

    def h2d_bg(self, dptr, arr):
        """Upload on the background stream; `join_uploads` orders later work after it."""
        assert arr.flags.c_contiguous
        self.check(self.lib.b200conv_memcpy_h2d_bg(self.h, _P(dptr), _P(arr.ctypes.data), arr.nbytes))

    def join_uploads(self):
        self.check(self.lib.b200conv_join_uploads(self.h))

    def d2h_bg(self, arr, dptr):
        """Download on the background stream once the work issued so far is done; `sync` waits for it."""
        assert arr.flags.c_contiguous
        self.check(self.lib.b200conv_memcpy_d2h_bg(self.h, _P(arr.ctypes.data), _P(dptr), arr.nbytes))

    def memset(self, dptr, value, nbytes):
        self.check(self.lib.b200conv_memset(self.h, _P(dptr), int(value), int(nbytes)))

    def sync(self):
        self.check(self.lib.b200conv_sync(self.h))

    def timer_start(self):
        self.check(self.lib.b200conv_timer_start(self.h))

    def timer_stop(self):
        ms = ctypes.c_float()
        self.check(self.lib.b200conv_timer_stop(self.h, ctypes.byref(ms)))
        return ms.value

    def kernel_timing(self, enable):
        self.check(self.lib.b200conv_kernel_timing(self.h, int(bool(enable))))

    def set_autotune(self, enable):
        """Choose between kernel variants by timing them on the first call of a geometry (default
        on); off: the static preference order."""
        self.check(self.lib.b200conv_set_autotune(self.h, int(bool(enable))))

    def set_pair_kernels(self, enable):
        """1x1 layers with deep reductions on CTA pairs (default on); off: the one-CTA kernel."""
        self.check(self.lib.b200conv_set_pair_kernels(self.h, int(bool(enable))))

    def set_stacked_taps(self, enable):
        """gradWeights of narrow float16 layers: taps of a filter row as column groups of one MMA (default on)."""
        self.check(self.lib.b200conv_set_stacked_taps(self.h, int(bool(enable))))

    def set_splits(self, n):
        """Pin the split-K slice count of gradWeights (0: chosen by the library)."""
        self.check(self.lib.b200conv_set_splits(self.h, int(n)))

    def tuning_save(self, path):
        """Write the choices made by timing (kernel variants, slice counts) to a file."""
        self.check(self.lib.b200conv_tuning_save(self.h, os.fsencode(path)))

    def tuning_load(self, path):
        """Read such a file (refused if written for another device model); returns the number of choices."""
        n = _I()
        self.check(self.lib.b200conv_tuning_load(self.h, os.fsencode(path), ctypes.byref(n)))
        return n.value

    def kernel_time(self, family):
        """(summed milliseconds, launches) of one kernel family since timing was enabled."""
        ms, n = ctypes.c_float(), _I()
        self.check(self.lib.b200conv_kernel_time(self.h, family.encode(), ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    def memory_info(self):
        """(bytes the context's pool took from the driver, free bytes of the device)."""
        a, b = _SZ(), _SZ()
        self.check(self.lib.b200conv_memory_info(self.h, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def set_wait_limit(self, clocks):
        """Bound of every device-side wait in SM clocks (default 4e9, about two seconds)."""
        self.check(self.lib.b200conv_set_wait_limit(self.h, int(clocks)))

    def selftest_wait(self):
        """Runs a kernel whose wait runs out on purpose; always raises B200Error (E_TIMEOUT)."""
        self.check(self.lib.b200conv_selftest_wait(self.h))

    def flush_l2(self):
        self.check(self.lib.b200conv_flush_l2(self.h))

    @property
    def launches(self):
        return int(self.lib.b200conv_launch_count(self.h))

    @property
    def last_algo(self):
        return self.lib.b200conv_last_algo(self.h).decode()

    def padded_channels(self, c, dtype):
        return int(self.lib.b200conv_padded_channels(int(c), _dtype_code(dtype)))

    # -- raw entry points ------------------------------------------------------------------
    def fwd(self, desc, x, w, bias, y, flags, residual=None, alpha=1.0, beta=1.0, slope=0.0):
        """y = act(alpha * conv + bias + beta * residual); the plain entry point when the
        epilogue is the default one."""
        if residual is None and alpha == 1.0 and slope == 0.0:
            self.check(self.lib.b200conv_fwd(self.h, ctypes.byref(desc), _P(x), _P(w), _P(bias), _P(y), flags))
        else:
            self.check(self.lib.b200conv_fwd_epilogue(self.h, ctypes.byref(desc), _P(x), _P(w), _P(bias),
                                                      _P(residual), _P(y), float(alpha), float(beta),
                                                      float(slope), flags))

    def dgrad(self, desc, w, dy, dx, flags):
        self.check(self.lib.b200conv_dgrad(self.h, ctypes.byref(desc), _P(w), _P(dy), _P(dx), flags))

    def wgrad(self, desc, x, dy, dw, flags):
        self.check(self.lib.b200conv_wgrad(self.h, ctypes.byref(desc), _P(x), _P(dy), _P(dw), flags))

    def wgrad_static(self, desc, x_nhwc, dy_nhwc, dw, flags=0):
        """gradWeights that allocates nothing (fixed scratch inside the library); device pointers,
        channels-last x and dy.  See b200conv_wgrad_static in include/b200conv.h for the limits."""
        self.check(self.lib.b200conv_wgrad_static(self.h, ctypes.byref(desc), _P(x_nhwc), _P(dy_nhwc), _P(dw), flags))

    def prepack(self, descs, filter_ptrs, directions=3):
        """Pack the filter banks of many layers with one launch (b200conv_prepack): `descs` are Desc
        structures, `filter_ptrs` the device pointers of the OIHW banks."""
        n = len(descs)
        arr = (Desc * n)(*descs)
        ptrs = (_P * n)(*[_P(p) for p in filter_ptrs])
        self.check(self.lib.b200conv_prepack(self.h, n, arr, ptrs, int(directions)))

    def filters_changed(self, ptr=None):
        """The filters at `ptr` (None: all) were written: their packed forms are stale."""
        self.check(self.lib.b200conv_filters_changed(self.h, _P(ptr)))

    def maxpool2x2(self, x, y, n, c, h, w, dtype, flags):
        self.check(self.lib.b200conv_maxpool2x2(self.h, _P(x), _P(y), n, c, h, w, _dtype_code(dtype), flags))

    def maxpool2x2_grad(self, x, y, gy, gx, n, c, h, w, dtype, flags):
        self.check(self.lib.b200conv_maxpool2x2_grad(self.h, _P(x), _P(y), _P(gy), _P(gx), n, c, h, w,
                                                     _dtype_code(dtype), flags))

    def nchw_to_nhwc(self, src, dst, n, c, h, w, dtype):
        self.check(self.lib.b200conv_nchw_to_nhwc(self.h, _P(src), _P(dst), n, c, h, w, _dtype_code(dtype)))

    def nhwc_to_nchw(self, src, dst, n, c, h, w, dtype):
        self.check(self.lib.b200conv_nhwc_to_nchw(self.h, _P(src), _P(dst), n, c, h, w, _dtype_code(dtype)))

    # -- CUDA graphs -------------------------------------------------------------------------
    def capture(self, fn):
        """Run ``fn()`` (device-pointer calls only) under stream capture; returns a ``Graph``.
        Call ``fn()`` once eagerly beforehand so that the memory pool is warm."""
        self.check(self.lib.b200conv_graph_begin(self.h))
        try:
            fn()
        except Exception:
            g = _P()
            self.lib.b200conv_graph_end(self.h, ctypes.byref(g))
            if g.value:
                self.lib.b200conv_graph_destroy(self.h, g)
            raise
        g = _P()
        self.check(self.lib.b200conv_graph_end(self.h, ctypes.byref(g)))
        return Graph(self, g)

    # -- data parallel ---------------------------------------------------------------------
    def nccl_unique_id(self):
        buf = ctypes.create_string_buffer(128)
        self.check(self.lib.b200conv_nccl_unique_id(self.h, buf))
        return buf.raw

    def nccl_init(self, nranks, rank, uid):
        self.check(self.lib.b200conv_nccl_init(self.h, nranks, rank, ctypes.create_string_buffer(uid, 128)))

    def allreduce_sum(self, dptr, count, dtype):
        self.check(self.lib.b200conv_allreduce_sum(self.h, _P(dptr), int(count), _dtype_code(dtype)))

    def allreduce_sum_async(self, dptr, count, dtype):
        """All-reduce on the communication stream, overlapping the calls that follow."""
        self.check(self.lib.b200conv_allreduce_sum_async(self.h, _P(dptr), int(count), _dtype_code(dtype)))

    def set_sm_count(self, sms):
        """SMs the persistent convolution kernels spread over (the rest stay free, e.g. for NCCL)."""
        self.check(self.lib.b200conv_set_sm_count(self.h, int(sms)))

    def set_comm_timeout(self, milliseconds):
        """Deadline of the host watchdog that guards synchronising calls while a communicator exists."""
        self.check(self.lib.b200conv_set_comm_timeout(self.h, int(milliseconds)))

    def comm_wait(self):
        self.check(self.lib.b200conv_comm_wait(self.h))

    def barrier(self):
        self.check(self.lib.b200conv_barrier(self.h))


class Graph(object):
    """A captured sequence of calls; ``launch()`` enqueues all of it with one driver call."""

    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle

    def launch(self):
        self.ctx.check(self.ctx.lib.b200conv_graph_launch(self.ctx.h, self.h))

    def destroy(self):
        if self.h and self.ctx.h:
            self.ctx.lib.b200conv_graph_destroy(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class _PinnedOwner(object):
    def __init__(self, ctx, ptr):
        self.ctx, self.ptr = ctx, ptr

    def __del__(self):
        try:
            if self.ctx.h:
                self.ctx.lib.b200conv_host_free(self.ctx.h, _P(self.ptr))
        except Exception:
            pass


class _PinnedArray(np.ndarray):
    _owner = None

    def __array_finalize__(self, obj):
        if obj is not None:
            self._owner = getattr(obj, "_owner", None)


_contexts = {}
_ctx_lock = threading.Lock()


def get_context(device=None):
    """Process-wide context of a device (default: ``B200CONV_DEVICE`` or LOCAL_RANK or 0)."""
    if device is None:
        device = int(os.environ.get("B200CONV_DEVICE", os.environ.get("LOCAL_RANK", "0")))
    with _ctx_lock:
        if device not in _contexts:
            _contexts[device] = Context(device)
        return _contexts[device]


def make_desc(xshape, wshape, yshape, pads, subsample, dilation, groups, flip, dtype):
    d = Desc()
    d.N, d.C, d.H, d.W = [int(v) for v in xshape]
    d.K, d.kH, d.kW = int(wshape[0]), int(wshape[2]), int(wshape[3])
    d.Ho, d.Wo = int(yshape[2]), int(yshape[3])
    d.sH, d.sW = int(subsample[0]), int(subsample[1])
    d.dilH, d.dilW = int(dilation[0]), int(dilation[1])
    (d.padH_l, d.padH_r), (d.padW_l, d.padW_r) = pads
    d.groups, d.flip, d.dtype = int(groups), int(bool(flip)), _dtype_code(dtype)
    return d


def _common(a, b):
    """Upcast like BaseCorrMM.as_common_dtype (corr.py:156-162); float64 is not handled here."""
    dt = np.promote_types(a.dtype, b.dtype)
    _dtype_code(dt)
    return np.ascontiguousarray(a, dtype=dt), np.ascontiguousarray(b, dtype=dt)


# ======================================================================================
# numpy in / numpy out (what Op.perform calls)
# ======================================================================================
def conv2d_forward(x, w, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
                   filter_flip=True, bias=None, relu=False, out=None, ctx=None, flags=0,
                   residual=None, alpha=1.0, beta=1.0, slope=0.0):
    """AbstractConv2d forward (CorrMM on flipped filters when filter_flip) with the fused
    epilogue y = act(alpha * conv + bias + beta * residual), act = leaky ReLU of `slope` when
    `relu` (slope 0: ReLU), else the identity.  x: [N,C,H,W], w: [K,C/g,kH,kW]; returns
    [N,K,Ho,Wo]."""
    x, w = _common(np.asarray(x), np.asarray(w))
    yshape, pads = hostlogic.forward_shape(x.shape, w.shape, border_mode, subsample, filter_dilation, num_groups)
    ctx = ctx or get_context()
    if out is None or out.shape != yshape or out.dtype != x.dtype or not out.flags.c_contiguous:
        out = np.empty(yshape, x.dtype)
    if out.size == 0:
        return out
    d = make_desc(x.shape, w.shape, yshape, pads, subsample, filter_dilation, num_groups, filter_flip, x.dtype)
    b = None
    if bias is not None:
        b = np.ascontiguousarray(bias, dtype=x.dtype)
        if b.shape != (w.shape[0],):
            raise ValueError("bias must have one value per filter")
    r = None
    if residual is not None:
        r = np.ascontiguousarray(residual, dtype=x.dtype)
        if r.shape != yshape:
            raise ValueError("residual must have the shape of the output %s, not %s" % (yshape, r.shape))
    ctx.fwd(d, x.ctypes.data, w.ctypes.data, b.ctypes.data if b is not None else None,
            out.ctypes.data, flags | HOST_PTRS | (RELU if relu else 0),
            residual=r.ctypes.data if r is not None else None, alpha=alpha, beta=beta, slope=slope)
    return out


def conv2d_grad_weights(x, dy, kshape=None, border_mode="valid", subsample=(1, 1),
                        filter_dilation=(1, 1), num_groups=1, filter_flip=True, out=None, ctx=None,
                        flags=0):
    """AbstractConv2d_gradWeights: x [N,C,H,W], dy [N,K,Ho,Wo] -> dw [K,C/g,kH,kW]."""
    x, dy = _common(np.asarray(x), np.asarray(dy))
    if x.ndim != 4:
        raise TypeError("img must be 4D tensor")
    if dy.ndim != 4:
        raise TypeError("topgrad must be 4D tensor")
    ksz = hostlogic.gradweights_kshape(x.shape, dy.shape, border_mode, subsample, filter_dilation, kshape)
    if x.shape[1] % num_groups:
        raise ValueError("CorrMM images and kernel must have the same stack size")
    wshape = (dy.shape[1], x.shape[1] // num_groups) + ksz
    pads = hostlogic.resolve_pads(border_mode, ksz, filter_dilation)
    hostlogic.check_consistent(x.shape, wshape, dy.shape, pads, subsample, filter_dilation, num_groups)
    ctx = ctx or get_context()
    if out is None or out.shape != wshape or out.dtype != x.dtype or not out.flags.c_contiguous:
        out = np.empty(wshape, x.dtype)
    if out.size == 0:
        return out
    d = make_desc(x.shape, wshape, dy.shape, pads, subsample, filter_dilation, num_groups, filter_flip, x.dtype)
    ctx.wgrad(d, x.ctypes.data, dy.ctypes.data, out.ctypes.data, flags | HOST_PTRS)
    return out


def conv2d_grad_inputs(w, dy, imshape=None, border_mode="valid", subsample=(1, 1),
                       filter_dilation=(1, 1), num_groups=1, filter_flip=True, out=None, ctx=None,
                       flags=0):
    """AbstractConv2d_gradInputs: w [K,C/g,kH,kW], dy [N,K,Ho,Wo] -> dx [N,C,H,W]."""
    w, dy = _common(np.asarray(w), np.asarray(dy))
    if w.ndim != 4:
        raise TypeError("kern must be 4D tensor")
    if dy.ndim != 4:
        raise TypeError("topgrad must be 4D tensor")
    hw, pads = hostlogic.gradinputs_imshape(w.shape, dy.shape, border_mode, subsample, filter_dilation, imshape)
    xshape = (dy.shape[0], w.shape[1] * num_groups) + hw
    hostlogic.check_consistent(xshape, w.shape, dy.shape, pads, subsample, filter_dilation, num_groups)
    ctx = ctx or get_context()
    if out is None or out.shape != xshape or out.dtype != w.dtype or not out.flags.c_contiguous:
        out = np.empty(xshape, w.dtype)
    if out.size == 0:
        return out
    d = make_desc(xshape, w.shape, dy.shape, pads, subsample, filter_dilation, num_groups, filter_flip, w.dtype)
    ctx.dgrad(d, w.ctypes.data, dy.ctypes.data, out.ctypes.data, flags | HOST_PTRS)
    return out


def maxpool2x2(x, ctx=None):
    """Pool(ignore_border=True, mode='max'), ws = stride = (2, 2), pad 0."""
    x = np.ascontiguousarray(x)
    n, c, h, w = x.shape
    ctx = ctx or get_context()
    out = np.empty((n, c, h // 2, w // 2), x.dtype)
    if out.size:
        ctx.maxpool2x2(x.ctypes.data, out.ctypes.data, n, c, h, w, x.dtype, HOST_PTRS)
    return out


def maxpool2x2_grad(x, y, gy, ctx=None):
    """MaxPoolGrad(ignore_border=True) of that pooling (theano/tensor/signal/pool.py:1139-1186):
    every position of x equal to its window's maximum y receives the window's gy."""
    x, y, gy = (np.ascontiguousarray(a) for a in (x, y, gy))
    n, c, h, w = x.shape
    if y.shape != (n, c, h // 2, w // 2) or gy.shape != y.shape:
        raise ValueError("MaxPoolGrad (b200conv): pooled shapes %s / %s do not match input %s"
                         % (y.shape, gy.shape, x.shape))
    if not (x.dtype == y.dtype == gy.dtype):
        raise TypeError("MaxPoolGrad (b200conv): x, y and gy must share one dtype")
    ctx = ctx or get_context()
    out = np.zeros(x.shape, x.dtype)
    if out.size and y.size:
        ctx.maxpool2x2_grad(x.ctypes.data, y.ctypes.data, gy.ctypes.data, out.ctypes.data, n, c, h, w,
                            x.dtype, HOST_PTRS)
    return out


# ======================================================================================
# device-resident tensors (activations stay on the GPU between layers, channels-last)
# ======================================================================================
class DeviceTensor(object):
    """A tensor in HBM.  ``shape`` is always the logical NCHW / OIHW shape; ``layout`` says how
    it is stored: 'nchw' (the reference's order) or 'nhwc' (channels-last, channel count padded
    to a multiple of 16 bytes: the order the tensor-core kernels read)."""

    def __init__(self, ctx, shape, dtype, layout="nchw", _ptr=None):
        self.ctx, self.shape, self.dtype, self.layout = ctx, tuple(int(s) for s in shape), np.dtype(dtype), layout
        self.owner = _ptr is None
        self.ptr = ctx.malloc(self.nbytes) if self.owner else _ptr

    def images(self, start, stop):
        """View of the images [start, stop) (both layouts keep an image contiguous); the view does
        not own the memory and must not outlive this tensor."""
        n = self.shape[0]
        if not 0 <= start <= stop <= n:
            raise ValueError("image range [%d, %d) outside 0..%d" % (start, stop, n))
        per = self.nbytes // max(n, 1)
        return DeviceTensor(self.ctx, (stop - start,) + self.shape[1:], self.dtype, self.layout,
                            _ptr=self.ptr + start * per)

    @property
    def stored_channels(self):
        return self.ctx.padded_channels(self.shape[1], self.dtype) if self.layout == "nhwc" else self.shape[1]

    @property
    def nbytes(self):
        n, c, h, w = self.shape
        return n * self.stored_channels * h * w * self.dtype.itemsize

    def free(self):
        if self.ptr and self.owner:
            self.ctx.free(self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.free()
        except Exception:
            pass

    @classmethod
    def from_host(cls, ctx, arr, layout="nchw"):
        """Upload a NCHW numpy array; with layout='nhwc' it is transposed on the device."""
        arr = np.ascontiguousarray(arr)
        t = cls(ctx, arr.shape, arr.dtype, "nchw")
        ctx.h2d(t.ptr, arr)
        if layout == "nhwc":
            u = t.to_layout("nhwc")
            ctx.sync()
            t.free()
            return u
        ctx.sync()
        return t

    def to_layout(self, layout):
        if layout == self.layout:
            return self
        n, c, h, w = self.shape
        out = DeviceTensor(self.ctx, self.shape, self.dtype, layout)
        if layout == "nhwc":
            self.ctx.nchw_to_nhwc(self.ptr, out.ptr, n, c, h, w, self.dtype)
        else:
            self.ctx.nhwc_to_nchw(self.ptr, out.ptr, n, c, h, w, self.dtype)
        return out

    def to_host(self, out=None):
        t = self.to_layout("nchw")
        if out is None:
            out = np.empty(self.shape, self.dtype)
        self.ctx.d2h(out, t.ptr)
        self.ctx.sync()
        if t is not self:
            t.free()
        return out


def device_conv2d(x, w, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
                  filter_flip=True, bias=None, relu=False, out_layout=None, out=None, flags=0,
                  residual=None, alpha=1.0, beta=1.0, slope=0.0, pool=False):
    """Forward on DeviceTensors (w, bias in 'nchw' storage = plain OIHW / vector); asynchronous.
    `residual`: a DeviceTensor with the shape and layout of the output.  `pool`: 2x2 max pooling of the
    activated result inside the kernel's epilogue (channels-last tensors, even output height and width);
    the result then has half the rows and columns.  Geometries whose epilogue cannot pool raise B200Error
    (E_UNSUPPORTED): run `device_maxpool2x2` on the unpooled result instead."""
    ctx = x.ctx
    yshape, pads = hostlogic.forward_shape(x.shape, w.shape, border_mode, subsample, filter_dilation, num_groups)
    out_layout = out_layout or x.layout
    oshape = (yshape[0], yshape[1], yshape[2] // 2, yshape[3] // 2) if pool else yshape
    if pool:
        if residual is not None or out_layout != "nhwc" or x.layout != "nhwc":
            raise ValueError("the pooling epilogue takes channels-last tensors and no residual")
        flags |= POOL2X2
    if out is None:
        out = DeviceTensor(ctx, oshape, x.dtype, out_layout)
    elif tuple(out.shape) != tuple(oshape):
        raise ValueError("output tensor has shape %s, expected %s" % (out.shape, oshape))
    d = make_desc(x.shape, w.shape, yshape, pads, subsample, filter_dilation, num_groups, filter_flip, x.dtype)
    f = flags | (IN_NHWC if x.layout == "nhwc" else 0) | (OUT_NHWC if out.layout == "nhwc" else 0) | (RELU if relu else 0)
    if residual is not None and (residual.shape != tuple(yshape) or residual.layout != out.layout):
        raise ValueError("residual must have the shape and layout of the output")
    if bias is not None and int(np.prod(bias.shape)) != int(w.shape[0]):
        raise ValueError("bias must have one value per filter (%d), not %d" % (w.shape[0], int(np.prod(bias.shape))))
    ctx.fwd(d, x.ptr, w.ptr, bias.ptr if bias is not None else None, out.ptr, f,
            residual=residual.ptr if residual is not None else None, alpha=alpha, beta=beta, slope=slope)
    return out


def device_grad_inputs(w, dy, imshape, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1),
                       num_groups=1, filter_flip=True, out_layout=None, out=None, flags=0):
    ctx = dy.ctx
    hw, pads = hostlogic.gradinputs_imshape(w.shape, dy.shape, border_mode, subsample, filter_dilation, imshape)
    xshape = (dy.shape[0], w.shape[1] * num_groups) + hw
    hostlogic.check_consistent(xshape, w.shape, dy.shape, pads, subsample, filter_dilation, num_groups)
    out_layout = out_layout or dy.layout
    if out is None:
        out = DeviceTensor(ctx, xshape, dy.dtype, out_layout)
    d = make_desc(xshape, w.shape, dy.shape, pads, subsample, filter_dilation, num_groups, filter_flip, dy.dtype)
    f = flags | (IN_NHWC if dy.layout == "nhwc" else 0) | (OUT_NHWC if out.layout == "nhwc" else 0)
    ctx.dgrad(d, w.ptr, dy.ptr, out.ptr, f)
    return out


def device_grad_weights(x, dy, kshape, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1),
                        num_groups=1, filter_flip=True, out=None, flags=0):
    ctx = x.ctx
    ksz = hostlogic.gradweights_kshape(x.shape, dy.shape, border_mode, subsample, filter_dilation, kshape)
    wshape = (dy.shape[1], x.shape[1] // num_groups) + ksz
    pads = hostlogic.resolve_pads(border_mode, ksz, filter_dilation)
    hostlogic.check_consistent(x.shape, wshape, dy.shape, pads, subsample, filter_dilation, num_groups)
    if out is None:
        out = DeviceTensor(ctx, wshape, x.dtype, "nchw")
    d = make_desc(x.shape, wshape, dy.shape, pads, subsample, filter_dilation, num_groups, filter_flip, x.dtype)
    f = flags | (IN_NHWC if x.layout == "nhwc" else 0) | (IN2_NHWC if dy.layout == "nhwc" else 0)
    if out.dtype == np.float32 and x.dtype == np.float16:
        f |= DW_F32              # float16 tensors, gradient kept in float32 (e.g. an all-reduce bucket)
    elif out.dtype != x.dtype:
        raise TypeError("gradWeights output must have the data type of the tensors, or float32")
    ctx.wgrad(d, x.ptr, dy.ptr, out.ptr, f)
    return out


def layer_desc(xshape, wshape, border_mode="valid", subsample=(1, 1), filter_dilation=(1, 1), num_groups=1,
               filter_flip=True, dtype=np.float32):
    """The geometry descriptor the convolution calls build for a layer (for Context.prepack)."""
    yshape, pads = hostlogic.forward_shape(xshape, wshape, border_mode, subsample, filter_dilation, num_groups)
    return make_desc(xshape, wshape, yshape, pads, subsample, filter_dilation, num_groups, filter_flip, dtype)


EW_OPS = {"add": 0, "mul": 1, "sub": 2, "rsub": 3, "div": 4, "rdiv": 5, "max": 6, "abs": 7, "sgn": 8, "neg": 9}


def device_elementwise(op, a, b=None, out=None):
    """out = op(a, b) element by element on a channels-last DeviceTensor `a`; `b` is another
    DeviceTensor of the same shape and layout, a Python number, a 1-D numpy array or a DeviceTensor
    vector with one value per channel (broadcast like b.dimshuffle('x', 0, 'x', 'x')), or None for
    the unary ops 'abs', 'sgn', 'neg'.  'rsub' / 'rdiv' compute b - a / b / a."""
    ctx = a.ctx
    if a.layout != "nhwc":
        raise ValueError("element-wise device ops take channels-last tensors")
    n, c, h, w = a.shape
    if out is None:
        out = DeviceTensor(ctx, a.shape, a.dtype, "nhwc")
    elif out.shape != a.shape or out.layout != "nhwc" or out.dtype != a.dtype:
        raise ValueError("output must have the shape, layout and dtype of the first operand")
    code = EW_OPS[op]
    keep = None
    if b is None:
        if op not in ("abs", "sgn", "neg"):
            raise ValueError("'%s' needs a second operand" % op)
        kind, bptr, scalar = 3, None, 0.0
    elif isinstance(b, DeviceTensor) and len(b.shape) == 4 and b.shape == a.shape:
        if b.layout != "nhwc" or b.dtype != a.dtype:
            raise ValueError("operands must share layout and dtype")
        kind, bptr, scalar = 0, b.ptr, 0.0
    elif np.isscalar(b) or (isinstance(b, np.ndarray) and b.size == 1):
        kind, bptr, scalar = 1, None, float(np.asarray(b).reshape(()))
    else:
        vec = np.ascontiguousarray(np.asarray(b).ravel(), dtype=a.dtype)
        if vec.size != c:
            raise ValueError("per-channel operand must have %d values, not %d" % (c, vec.size))
        keep = DeviceTensor(ctx, (1, c, 1, 1), a.dtype, "nchw")
        ctx.h2d(keep.ptr, vec)
        ctx.sync()                       # the host vector may be freed by the caller
        kind, bptr, scalar = 2, keep.ptr, 0.0
    ctx.check(ctx.lib.b200conv_elementwise(ctx.h, code, _P(a.ptr), _P(bptr), _P(out.ptr), n * h * w, c, kind,
                                           scalar, _dtype_code(a.dtype)))
    if keep is not None:
        keep.free()                      # pooled and stream ordered: reused only after the kernel above
    return out


def device_channel_sum(x):
    """Sum over batch, rows and columns per channel (Sum{axis=[0, 2, 3]}) of a channels-last
    DeviceTensor; returns a host vector of the tensor's dtype."""
    ctx = x.ctx
    if x.layout != "nhwc":
        raise ValueError("channel sum takes a channels-last tensor")
    n, c, h, w = x.shape
    out = np.zeros(c, x.dtype)
    if n * h * w == 0 or c == 0:
        return out
    d = DeviceTensor(ctx, (1, c, 1, 1), x.dtype, "nchw")
    ctx.check(ctx.lib.b200conv_channel_sum(ctx.h, _P(x.ptr), _P(d.ptr), n * h * w, c, _dtype_code(x.dtype)))
    ctx.d2h(out, d.ptr)
    ctx.sync()
    d.free()
    return out


def device_maxpool2x2(x, out=None):
    ctx = x.ctx
    n, c, h, w = x.shape
    if out is None:
        out = DeviceTensor(ctx, (n, c, h // 2, w // 2), x.dtype, x.layout)
    ctx.maxpool2x2(x.ptr, out.ptr, n, c, h, w, x.dtype, IN_NHWC if x.layout == "nhwc" else 0)
    return out


def device_maxpool2x2_grad(x, y, gy, out=None):
    """gradient of `device_maxpool2x2` on device tensors of one layout."""
    ctx = x.ctx
    n, c, h, w = x.shape
    if not (x.layout == y.layout == gy.layout):
        raise ValueError("MaxPoolGrad (b200conv): tensors must share one layout")
    if out is None:
        out = DeviceTensor(ctx, x.shape, x.dtype, x.layout)
    ctx.maxpool2x2_grad(x.ptr, y.ptr, gy.ptr, out.ptr, n, c, h, w, x.dtype, IN_NHWC if x.layout == "nhwc" else 0)
    return out
