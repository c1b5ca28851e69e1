/*
 * b200conv: C ABI of the B200 (sm_100a) 2-D convolution library.
 *
 * The library replaces, for float32 and float16, the three directions of the reference
 * routine corrMM() (theano/tensor/nnet/c_code/corr_gemm.c:101-114) together with the host
 * logic that the reference generates around it (theano/tensor/nnet/corr.py:250-589).
 * Tensors use the reference's layouts: images and output maps are C-contiguous NCHW,
 * filters are OIHW with C/groups input channels per filter.  All functions return 0 on
 * success or a negative B200CONV_E_* code; the text of the last error of a context is
 * available through b200conv_last_error().  Nothing here throws or aborts the process.
 *
 * Plain pointers and sizes only: the library can be bound from ctypes, cffi or C.
 */
#ifndef B200CONV_H_
#define B200CONV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200conv_ctx b200conv_ctx;
typedef struct b200conv_graph b200conv_graph;

enum {
  B200CONV_OK = 0,
  B200CONV_E_INVALID = -1, /* bad argument or shape inconsistency (reference: ValueError,
                              corr_gemm.c:164-237, corr.py:408-533) */
  B200CONV_E_CUDA = -2,    /* CUDA runtime / driver failure (reference: RuntimeError) */
  B200CONV_E_NOMEM = -3,   /* device or pinned-host allocation failed */
  B200CONV_E_TIMEOUT = -4, /* a bounded device-side wait ran out */
  B200CONV_E_UNSUPPORTED = -5,
  B200CONV_E_NCCL = -6
};

enum { B200CONV_F32 = 0, B200CONV_F16 = 1 };

/* Flags (bitwise or). */
enum {
  B200CONV_HOST_PTRS = 1 << 0,   /* tensor pointers are host memory: the call copies inputs to
                                    the device, runs, copies the result back and synchronises */
  B200CONV_RELU = 1 << 1,        /* forward only: y = relu(conv + bias), relu(v) = 0.5*(v+|v|)
                                    (theano/tensor/nnet/nnet.py:2242-2243) */
  B200CONV_IN_NHWC = 1 << 2,     /* device pointers only: the image-like INPUT (x for forward and
                                    gradWeights, dy for the two gradients) is channels-last with
                                    the channel count padded as b200conv_padded_channels() says */
  B200CONV_OUT_NHWC = 1 << 3,    /* device pointers only: the image-like OUTPUT (y or dx) is
                                    written channels-last (padded channels are written as 0) */
  B200CONV_IN2_NHWC = 1 << 4,    /* gradWeights only: dy is channels-last */
  B200CONV_FORCE_DIRECT = 1 << 5,/* use the CUDA-core direct kernels (cross-check path) */
  B200CONV_FORCE_UMMA = 1 << 6,  /* fail with E_UNSUPPORTED instead of using the direct kernels */
  B200CONV_ATOMIC_SPLITK = 1 << 7,/* gradWeights: combine split-K slices with floating-point
                                    atomics instead of the ordered (deterministic) reduction */
  B200CONV_NO_SLAB = 1 << 8,     /* forward / gradInputs: fetch the activations once per filter tap
                                    (the general kernel) even where the slab kernel applies */
  B200CONV_NO_GROUP = 1 << 9,    /* gradWeights: one filter tap per work item (the general kernel)
                                    even where taps can share their operands */
  B200CONV_NO_MERGE_PARITY = 1 << 10,/* strided gradInputs with few channels: one launch per stride
                                    parity class even where the classes can be merged into one */
  B200CONV_NO_S2D = 1 << 11,     /* forward, stride 2 with at most 4 channels: keep the pixels as they
                                    are even where 2 x 2 pixel blocks can be turned into channels */
  B200CONV_DW_F32 = 1 << 12,     /* gradWeights: store dw as float32 even for float16 tensors (the sum
                                    is float32 anyway); for gradient buckets that are all-reduced in
                                    float32 */
  B200CONV_POOL2X2 = 1 << 13     /* forward, channels-last device tensors: y = maxpool2x2(act(conv + bias)) in one
                                    kernel (Pool{ignore_border=True, mode='max'} with ws = stride = (2, 2),
                                    theano/tensor/signal/pool.py:524-574, applied in the epilogue); y is
                                    [N][Ho/2][Wo/2][Kp]; Ho and Wo must be even; geometries whose epilogue cannot pool
                                    return B200CONV_E_UNSUPPORTED (run the two calls instead) */
};

/*
 * Geometry of one convolution, with pads already resolved ('half'/'full' are turned into
 * numbers by the caller exactly as corr.py:375-395 does).  bottom = [N,C,H,W],
 * weights = [K, C/groups, kH, kW], top = [N,K,Ho,Wo] with
 * Ho = floor((H + padH_l + padH_r - ((kH-1)*dilH + 1)) / sH) + 1 (corr_gemm.c:175-185).
 * flip != 0 selects true convolution (AbstractConv2d filter_flip=True: the filters are
 * rotated by 180 degrees, theano/tensor/nnet/opt.py:84-92); flip == 0 is CorrMM itself.
 */
typedef struct b200conv_desc {
  int32_t N, C, H, W;
  int32_t K, kH, kW;
  int32_t Ho, Wo;
  int32_t sH, sW;
  int32_t dilH, dilW;
  int32_t padH_l, padH_r, padW_l, padW_r;
  int32_t groups;
  int32_t flip;
  int32_t dtype; /* B200CONV_F32 or B200CONV_F16; accumulation is always float32 */
} b200conv_desc;

/* ---- context ------------------------------------------------------------------------ */
/* One context per device and host thread of control; calls on one context are serialised
 * by an internal mutex and run on the context's own CUDA stream. */
int b200conv_create(int device, b200conv_ctx** out);
void b200conv_destroy(b200conv_ctx* ctx);
/* Copies the last error text (NUL terminated) into buf; returns its length. */
int b200conv_last_error(b200conv_ctx* ctx, char* buf, size_t n);
/* Same for failures of b200conv_create itself (no context yet). */
int b200conv_create_error(char* buf, size_t n);
const char* b200conv_version(void);

/* ---- the three directions ----------------------------------------------------------- */
/* Replaces corrMM(direction 0), corr_gemm.c:297-339 (+ the Elemwise bias/ReLU that follows
 * it in compiled graphs).  bias may be NULL; otherwise K values of the tensor dtype. */
int b200conv_fwd(b200conv_ctx* ctx, const b200conv_desc* d, const void* x, const void* w,
                 const void* bias, void* y, int flags);
/* Forward with a wider fused epilogue (the elementwise ops that follow a convolution in compiled
 * graphs; the reference leaves them to its Elemwise fusion, theano/tensor/opt.py:7451-7469, its GPU
 * back end merges scale and accumulate into the convolution call, gpuarray/opt_util.py:100-280):
 *   y = act(alpha * conv(x, w) + bias + beta * residual)
 * act = identity without B200CONV_RELU, else leaky ReLU of that slope in the reference's form
 * 0.5 * ((1 + slope) * v + (1 - slope) * |v|) (theano/tensor/nnet/nnet.py:2242-2250); slope 0 = ReLU.
 * bias and residual may be NULL; residual has the shape and layout of y (host NCHW with HOST_PTRS,
 * channels-last with OUT_NHWC).  b200conv_fwd == this call with alpha 1, no residual, slope 0. */
int b200conv_fwd_epilogue(b200conv_ctx* ctx, const b200conv_desc* d, const void* x, const void* w,
                          const void* bias, const void* residual, void* y, float alpha, float beta,
                          float slope, int flags);

/* Replaces corrMM(direction 2), corr_gemm.c:486-529: dx = gradient wrt the image. */
int b200conv_dgrad(b200conv_ctx* ctx, const b200conv_desc* d, const void* w, const void* dy,
                   void* dx, int flags);
/* Replaces corrMM(direction 1), corr_gemm.c:372-456: dw = gradient wrt the filters. */
int b200conv_wgrad(b200conv_ctx* ctx, const b200conv_desc* d, const void* x, const void* dy,
                   void* dw, int flags);

/*
 * gradWeights that allocates nothing.  No counterpart in the reference (its corrMM allocates
 * its column and per-thread weight buffers on every call, corr_gemm.c:239-260,374-381).
 *
 * Who needs it: programs that may not call cudaMalloc while they run.  Typical cases are a host
 * application that gave all device memory to its own allocator at start-up (a later cudaMalloc
 * from a library fails or eats into its arena), a serving or training loop that must not stall
 * (cudaMalloc and cudaFree synchronise the whole device), and deployments with a fixed memory
 * budget that is audited once after warm-up.  b200conv_wgrad() keeps its split-K slabs in
 * pooled memory that can grow through cudaMalloc; this variant keeps them in a fixed 32 MiB
 * array inside the library image (so every GPU that loads the library carries those 32 MiB until
 * the process exits) and calls no allocating routine of CUDA or of any other library.
 *
 * x and dy must be channels-last device tensors (as with IN_NHWC | IN2_NHWC), dw is the OIHW
 * output on the device; flags may carry B200CONV_ATOMIC_SPLITK.  Limits: the tensor-core
 * geometries only (otherwise B200CONV_E_UNSUPPORTED), and one slab kH*kW*K*(C/groups)*4 bytes
 * must fit in the 32 MiB (otherwise B200CONV_E_INVALID with the sizes in the error text); when
 * fewer slabs fit than b200conv_wgrad would use, the reduction is cut into fewer, longer slices.
 * The first call on a device looks up the device address of the array
 * (cudaGetSymbolAddress); with lazy module loading that call, or the first launch, is also where
 * the CUDA runtime loads the library's code and the 32 MiB array onto that device.  So the
 * first call per device is a warm-up: make it before any stream capture begins and before the
 * phase in which nothing may be allocated.
 * All calls on a device share the one array and it keeps the contents of the previous call (what
 * must start at zero is cleared by the call itself): two calls whose kernels overlap on the GPU,
 * from different contexts or streams, race on it.  Calls on one context are ordered and safe.
 */
int b200conv_wgrad_static(b200conv_ctx* ctx, const b200conv_desc* d, const void* x_nhwc,
                          const void* dy_nhwc, void* dw, int flags);

/*
 * Filter packing ahead of time.  Forward and gradInputs read the filters in a tap-major packed
 * form that they otherwise rebuild from OIHW on every call (one small kernel per call: with
 * dozens of layers per step these launches add up).  b200conv_prepack() builds the packed forms of
 * `count` filter banks with ONE launch per data type (directions: bit 0 = forward, bit 1 =
 * gradInputs) into buffers the context keeps; later b200conv_fwd / b200conv_dgrad calls with the
 * same filter pointer and geometry (channels-last device tensors) use them and launch no packing
 * kernel.  A training loop calls it once per step after the optimizer has updated the filters (the
 * call can be part of a captured graph: a replay packs whatever the filter buffers then hold).
 * b200conv_filters_changed(w) marks the packed forms of one bank (NULL: of all) stale: calls pack
 * per call again until the next prepack.  Writing to a filter buffer without either call makes
 * later calls use stale filters.  Banks whose geometry has no packed form of this kind (1x1
 * forward banks are read in place; few-channel stems and merged small groups pack differently)
 * are skipped.  No counterpart in the reference (BLAS reads OIHW as it is).
 */
int b200conv_prepack(b200conv_ctx* ctx, int count, const b200conv_desc* descs, const void* const* filters,
                     int directions);
int b200conv_filters_changed(b200conv_ctx* ctx, const void* w);

/* Pool(ignore_border=True, mode='max') with ws = stride = (2,2), pad 0
 * (theano/tensor/signal/pool.py:524-574).  flags: HOST_PTRS, IN_NHWC (then output is NHWC too).
 * One difference from the reference on non-finite data: the maximum is taken with fmaxf, which returns
 * the other operand when one is NaN, whereas the reference's `>` comparisons keep a NaN that comes first in
 * a window; on finite data the results are identical. */
int b200conv_maxpool2x2(b200conv_ctx* ctx, const void* x, void* y, int N, int C, int H, int W,
                        int dtype, int flags);

/* Gradient of that pooling, MaxPoolGrad(ignore_border=True) (theano/tensor/signal/pool.py:1139-1186):
 * gx = gy of the window wherever x equals the window's maximum y, else 0 (also in the last row /
 * column of an odd-sized image, which no window covers).  x, gx: N x C x H x W; y, gy:
 * N x C x H/2 x W/2.  flags: HOST_PTRS, IN_NHWC (then all four tensors are channels-last). */
int b200conv_maxpool2x2_grad(b200conv_ctx* ctx, const void* x, const void* y, const void* gy, void* gx,
                             int N, int C, int H, int W, int dtype, int flags);

/* ---- element-wise ops on device tensors ------------------------------------------------ */
/* The Elemwise nodes that sit between convolution ops in compiled graphs (bias add, the rectifier
 * 0.5 * (v + |v|) and its gradient, residual add, scale) and the bias gradient Sum{axis=[0,2,3]},
 * on channels-last device tensors, so that activations need not visit the host for them; the
 * reference's GPU back end keeps them on the device the same way (theano/gpuarray/elemwise.py:86).
 * out = op(a, b) element by element; a and out are channels-last tensors of N*H*W pixels with C
 * channels (stored with padded channels); b is, by b_kind, 0: a tensor of the same shape, 1: the
 * scalar `scalar`, 2: a device vector of C values of the tensor dtype (one per channel, the
 * reference's b.dimshuffle('x', 0, 'x', 'x')), 3: absent (unary ops).  out may alias a or b. */
enum {
  B200CONV_EW_ADD = 0, B200CONV_EW_MUL = 1, B200CONV_EW_SUB = 2 /* a - b */, B200CONV_EW_RSUB = 3 /* b - a */,
  B200CONV_EW_DIV = 4 /* a / b */, B200CONV_EW_RDIV = 5 /* b / a */, B200CONV_EW_MAX = 6,
  B200CONV_EW_ABS = 7, B200CONV_EW_SGN = 8, B200CONV_EW_NEG = 9
};
int b200conv_elementwise(b200conv_ctx* ctx, int op, const void* a, const void* b, void* out, long long pixels,
                         int C, int b_kind, float scalar, int dtype);
/* out[c] = sum over the pixels of x[pixel][c]: C values of the tensor dtype in device memory,
 * accumulated in float32 in a fixed order. */
int b200conv_channel_sum(b200conv_ctx* ctx, const void* x, void* out, long long pixels, int C, int dtype);

/* ---- device-resident tensors -------------------------------------------------------- */
/* Channel count of the channels-last device layout (rounded up to 16 bytes). */
int b200conv_padded_channels(int C, int dtype);
int b200conv_malloc(b200conv_ctx* ctx, size_t bytes, void** dptr);   /* pooled, stream ordered */
int b200conv_free(b200conv_ctx* ctx, void* dptr);
int b200conv_host_alloc(b200conv_ctx* ctx, size_t bytes, void** hptr); /* pinned host memory */
int b200conv_host_free(b200conv_ctx* ctx, void* hptr);
int b200conv_memcpy_h2d(b200conv_ctx* ctx, void* dst, const void* src, size_t bytes);  /* async */
int b200conv_memcpy_d2h(b200conv_ctx* ctx, void* dst, const void* src, size_t bytes);  /* async */
/* Background copies for callers that overlap transfers with compute (PCIe moves both ways at once):
 * _h2d_bg copies on an upload stream of the context, b200conv_join_uploads makes everything issued
 * afterwards on the context wait for the uploads issued so far; _d2h_bg copies on a download stream
 * once everything issued so far on the context has finished.  b200conv_sync also waits for the
 * downloads.  The source of an upload must stay untouched until it was joined and a later sync returned.
 * No counterpart in the reference (its ops take host arrays). */
int b200conv_memcpy_h2d_bg(b200conv_ctx* ctx, void* dptr, const void* hptr, size_t bytes);
int b200conv_join_uploads(b200conv_ctx* ctx);
int b200conv_memcpy_d2h_bg(b200conv_ctx* ctx, void* hptr, const void* dptr, size_t bytes);
int b200conv_memset(b200conv_ctx* ctx, void* dst, int value, size_t bytes);            /* async */
int b200conv_sync(b200conv_ctx* ctx);
/* NCHW <-> channels-last conversion kernels (device pointers). */
int b200conv_nchw_to_nhwc(b200conv_ctx* ctx, const void* src, void* dst, int N, int C, int H,
                          int W, int dtype);
int b200conv_nhwc_to_nchw(b200conv_ctx* ctx, const void* src, void* dst, int N, int C, int H,
                          int W, int dtype);

/* ---- CUDA graphs ----------------------------------------------------------------------
 * The reference pays interpreter and launch overhead per node on every call of a compiled
 * function (lazylinker_c.c:514-553).  Here a sequence of device-pointer calls (fwd, dgrad, wgrad,
 * pooling, layout conversion, all-reduce) can be recorded once between graph_begin and graph_end
 * and replayed with one launch.  Run the sequence once before capturing it (kernel attributes
 * and the memory pool are then warm); the pointers and shapes are frozen into the graph; the
 * temporaries the calls used stay reserved until graph_destroy.  Host-pointer calls, sync,
 * timer_stop and barrier are refused while a capture is open. */
int b200conv_graph_begin(b200conv_ctx* ctx);
int b200conv_graph_end(b200conv_ctx* ctx, b200conv_graph** graph);
int b200conv_graph_launch(b200conv_ctx* ctx, b200conv_graph* graph);
int b200conv_graph_destroy(b200conv_ctx* ctx, b200conv_graph* graph);

/* ---- measurement -------------------------------------------------------------------- */
/* CUDA-event stopwatch on the context's stream: start, enqueue work, stop (synchronises). */
int b200conv_timer_start(b200conv_ctx* ctx);
int b200conv_timer_stop(b200conv_ctx* ctx, float* ms);
/* Number of kernels this context has launched so far (copies and memsets not counted). */
long long b200conv_launch_count(b200conv_ctx* ctx);
/* Per-kernel timing.  While enabled, every launch of the library's own kernels is bracketed by
 * CUDA events on the context's stream; b200conv_kernel_time() then returns the summed duration
 * and the launch count of one kernel family since timing was enabled: "conv_umma" (forward and
 * gradInputs main kernel), "wgrad_umma", "wgrad_reduce", "transpose", "pack", "direct", "pool". */
int b200conv_kernel_timing(b200conv_ctx* ctx, int enable);
int b200conv_kernel_time(b200conv_ctx* ctx, const char* family, float* total_ms, int* launches);
/* Forward and gradInputs have two tensor-core kernels (activations fetched once per channel
 * block, or once per filter tap).  By default the first call of a geometry times both and the
 * context remembers the faster one; with enable = 0 the first is always used where it applies
 * (B200CONV_NO_SLAB still forces the second). */
int b200conv_set_autotune(b200conv_ctx* ctx, int enable);
/* 1x1 layers (float16, channels-last, at least 256 channels, filters in whole 64-blocks) run on pairs of
 * CTAs that share the filter tile (tcgen05 cta_group::2); enable = 0 keeps them on the one-CTA kernel
 * (the cross-check of the parity tests). */
int b200conv_set_pair_kernels(b200conv_ctx* ctx, int enable);
/* gradWeights of float16 layers with at most 64 channels per group computes the taps of a filter row as column
 * groups of one MMA (the operand descriptor's leading-dimension offset is the taps' spacing) instead of one
 * half-empty MMA per tap; enable = 0 keeps one MMA per tap (the cross-check of the parity tests). */
int b200conv_set_stacked_taps(b200conv_ctx* ctx, int enable);
/* gradWeights cuts its reduction into slices (split-K); the count comes from a model of the busiest
 * SM's work and, with selection by timing on, from timing that count against half and twice of it
 * on the first call of a geometry.  b200conv_set_splits(n > 0) pins the count (tests, tuning by
 * hand); 0 gives the choice back to the library. */
int b200conv_set_splits(b200conv_ctx* ctx, int splits);
/* The choices made by timing (kernel variant per geometry, slice counts) written to / read from a
 * text file, so that a later process starts with them instead of timing again: the persistent form
 * of the cache the reference's meta-optimizer keeps per process (theano/gpuarray/opt.py:2144-2222;
 * flags metaopt.*, theano/configdefaults.py:1545-1551).  A file written on another device model or
 * for another SM count is refused.  *loaded = number of choices read. */
int b200conv_tuning_save(b200conv_ctx* ctx, const char* path);
int b200conv_tuning_load(b200conv_ctx* ctx, const char* path, int* loaded);
/* Development aid: while dbuf (device memory, 32 x int64 per SM) is set, the slab convolution
 * kernel stores clock64() stamps of its phases there (CTA start, set-up done, first operands
 * landed, last MMA issued, accumulator complete, epilogue done, exit); NULL switches it off. */
int b200conv_debug_trace(b200conv_ctx* ctx, void* dbuf);
/* Bytes the context's memory pool has obtained from the driver so far, and the device's free
 * memory (either pointer may be NULL).  For checks that a code path allocates nothing. */
int b200conv_memory_info(b200conv_ctx* ctx, size_t* pool_bytes, size_t* device_free_bytes);
/* Every wait inside the kernels (on a TMA copy, an MMA commit, an accumulator hand-over) is bounded:
 * when it runs out the kernel writes a status word, gives up and returns, and the next
 * synchronising call returns B200CONV_E_TIMEOUT; the context stays usable.  The bound is given in
 * SM clocks (default 4e9, about two seconds).  b200conv_selftest_wait() runs a one-CTA kernel that
 * waits on a barrier nobody arrives on, so that this path can be exercised on purpose: it returns
 * B200CONV_E_TIMEOUT after about the bound (plus a quarter of it, the kernel's grace period for
 * work in flight), never anything else, and nothing on the GPU is disturbed.  No counterpart in
 * the reference (its CPU loops cannot stall on a device). */
int b200conv_set_wait_limit(b200conv_ctx* ctx, long long clocks);
int b200conv_selftest_wait(b200conv_ctx* ctx);
/* Name of the kernel family the last fwd/dgrad/wgrad call used: "umma" or "direct". */
const char* b200conv_last_algo(b200conv_ctx* ctx);
/* Writes `bytes` of device scratch to evict the L2 cache between timed iterations. */
int b200conv_flush_l2(b200conv_ctx* ctx);

/* ---- data parallel (NCCL) ----------------------------------------------------------- */
/* The reference has no collective; data-parallel training sums the filter gradients of the
 * batch shards, which is what the per-thread partial sum of corr_gemm.c:443-455 does inside
 * one process.  id is an opaque 128-byte NCCL unique id made on rank 0 and handed to the
 * other ranks by the caller (file, socket, store). */
int b200conv_nccl_unique_id(b200conv_ctx* ctx, void* id128);
int b200conv_nccl_init(b200conv_ctx* ctx, int nranks, int rank, const void* id128);
int b200conv_allreduce_sum(b200conv_ctx* ctx, void* dbuf, size_t count, int dtype);
/* Same reduction on a second stream: it starts when the work enqueued so far has finished and
 * runs beside the convolution calls that follow; several may be queued (they run in the order
 * issued).  A buffer must not be touched until
 * b200conv_comm_wait() (orders the main stream after the reduction, no host wait),
 * b200conv_sync(), b200conv_timer_stop() or b200conv_barrier(). */
int b200conv_allreduce_sum_async(b200conv_ctx* ctx, void* dbuf, size_t count, int dtype);
int b200conv_comm_wait(b200conv_ctx* ctx);
/* The convolution kernels are persistent: one CTA per SM that takes all of the SM's shared memory,
 * so a collective's kernels find no room until a convolution kernel ends, and then hold up the
 * next one.  b200conv_set_sm_count(ctx, n) makes every later launch of this context use n SMs
 * (default: all): leaving as many SMs free as NCCL may use CTAs (NCCL_MAX_CTAS) lets the
 * all-reduces run beside the backward pass without either side waiting for the other. */
int b200conv_set_sm_count(b200conv_ctx* ctx, int sms);
/* Failure detection.  While a communicator exists, every synchronising call (sync, timer_stop,
 * barrier, host-pointer calls) waits under a host watchdog instead of blocking in the driver: it
 * polls the stream and ncclCommGetAsyncError; on an asynchronous NCCL error, or when a collective
 * has not finished after the timeout (default 60 s), it calls ncclCommAbort and returns
 * B200CONV_E_NCCL.  The context stays usable without the communicator; survivors build a new one
 * with b200conv_nccl_init.  No counterpart in the reference (one process, no peers to lose). */
int b200conv_set_comm_timeout(b200conv_ctx* ctx, int milliseconds);
int b200conv_barrier(b200conv_ctx* ctx);
int b200conv_nccl_destroy(b200conv_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* B200CONV_H_ */
