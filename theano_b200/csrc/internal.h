// Declarations shared by the translation units of libb200conv (not part of the C ABI).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/b200conv.h"

namespace b200 {

// cudaFuncSetAttribute applies to the device that is current when it is called, so a process
// that opens contexts on several devices has to repeat it on each: one bit per device.
struct PerDeviceOnce {
  std::atomic<unsigned long long> done{0};
  // Runs `set()` (returning cudaError_t) unless it already ran on the current device.
  template <class F> cudaError_t ensure(F set) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = dev >= 0 && dev < 64 ? 1ULL << dev : 0ULL;
    if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
    e = set();
    if (e == cudaSuccess && bit) done.fetch_or(bit, std::memory_order_release);
    return e;
  }
};

// Codes a kernel writes to the device status word when it gives up.
enum : int { kStatusOk = 0, kStatusTimeout = 1, kStatusBadIndex = 2 };

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
inline long long cdiv(long long a, long long b) { return (a + b - 1) / b; }
inline size_t elem_size(int dtype) { return dtype == B200CONV_F16 ? 2 : 4; }
// Channels-last tensors pad the channel count so that one pixel is a multiple of 16 bytes
// (tensor-map strides must be).
inline int pad_channels(int c, int dtype) { return round_up(c < 1 ? 1 : c, dtype == B200CONV_F16 ? 8 : 4); }

// ---- implicit-GEMM convolution (conv_umma.cu) -----------------------------------------
// One "tap" of the reduction: a spatial offset into one activation view and the filter
// slice that multiplies it.
struct ConvTap {
  int16_t dh, dw;   // offset added to the output-tile origin (in the view's pixel grid)
  int16_t view;     // which activation tensor map
  int16_t wmat;     // which packed filter matrix
};
constexpr int kMaxTaps = 64;
constexpr int kMaxViews = 9;

// Forward epilogue: y = act(alpha * conv + bias + beta * residual); with `relu` set
// act(v) = lin * v + abs * |v|  (ReLU: 0.5, 0.5; leaky ReLU of slope s: 0.5 * (1 + s), 0.5 * (1 - s),
// the reference's formula, theano/tensor/nnet/nnet.py:2242-2250), else the identity.  `residual` has
// the layout of the output.  Defaults (alpha 1, no residual, 0.5 / 0.5) reproduce bias + ReLU.
struct ConvEpilogue {
  const void* residual;
  float alpha, beta, lin, abs;
  int pool;          // 1: 2x2 max pooling (stride 2) of the activated result inside the epilogue; the output tensor has
                     // half the rows and columns (slab kernel with staged TMA stores only)
};
inline ConvEpilogue default_epilogue() { return ConvEpilogue{nullptr, 1.f, 0.f, 0.5f, 0.5f, 0}; }

struct alignas(64) UmmaConvParams {
  CUtensorMap views[kMaxViews];  // 5-D (c_in_group, group, w, h, n) channels-last views
  CUtensorMap wmap;              // 3-D (k_red, n_out, wmat*groups + g) packed filters
  ConvTap taps[kMaxTaps];
  int ntaps;
  int kblocks;                   // ceil(reduction channels per group / channels per stage)
  int groups;
  int Wt, Ht, Nimg;              // extent of the output pixel grid this launch covers
  int bw, bh, bn;                // pixel tile (bw*bh*bn <= 128 rows of the accumulator)
  int tiles_w, tiles_h, tiles_n, tiles_co;
  int n_out;                     // output channels per group
  void* out;
  const float* bias;             // per output channel (groups*n_out) or null
  long long out_sn, out_sc, out_sh, out_sw, out_off;  // element strides / offset of `out`
  long long out_elems;           // elements of `out` this launch may touch (checked in the range-checked build)
  int relu;
  ConvEpilogue epi;
  int* status;
  long long wait_clocks;          // bound of every device-side wait, in SM clocks
};

// Launches the kernel for `total tiles`; kind: 0 = tf32 (float32 data), 1 = f16.
int conv_umma_bn(int n_out);      // accumulator columns used for n_out outputs per group
cudaError_t launch_conv_umma(const UmmaConvParams& p, int dtype, int num_sms, cudaStream_t s);

// ---- implicit GEMM with one activation slab per channel block (conv_slab.cu) ---------------
// For launches whose taps all read the same view: the slab (output tile plus halo) is loaded
// once per channel block and every tap is a row offset into it.
struct alignas(64) SlabConvParams {
  CUtensorMap view;              // 5-D (c_in_group, group, w, h, n), box (kBK, 1, Ws, Hs, nb)
  CUtensorMap wmap;              // 3-D packed filters, box (kBK, BN, 1)
  int16_t tap_shift[kMaxTaps];   // row offset of the tap inside the slab
  int16_t tap_wmat[kMaxTaps];
  int ntaps;
  int kblocks;
  int groups;
  int Wt, Ht, Nimg;              // output grid
  int wt, th, nb;                // output columns / rows / images per tile
  int Ws, Hs;                    // slab columns / rows per image (tile + halo)
  int dw_min, dh_min;            // view coordinate of slab column / row 0 relative to the tile origin
  int tiles_w, tiles_h, tiles_n, tiles_co;
  int n_acc;                     // 128-row accumulators in use (<= 512 / BN)
  int slab_bytes;                // bytes of one slab buffer (1024-byte multiple)
  int b_stages;                  // filter-tile ring depth
  int s_stages;                  // slab ring depth (2 .. 6)
  int tps;                       // filter taps per stage of the filter ring (narrow tiles: several taps share a barrier round)
  int n_out;
  void* out;
  const float* bias;
  long long out_sn, out_sc, out_sh, out_sw, out_off;
  long long out_elems;           // elements of `out` this launch may touch (checked in the range-checked build)
  int relu;
  ConvEpilogue epi;
  int* status;
  long long wait_clocks;          // bound of every device-side wait, in SM clocks
  long long* trace;              // optional: 16 clock64 stamps per CTA (phase timing), or null
  // Channels-last outputs are written by TMA: the epilogue warps put 128-byte channel chunks (32
  // float32 / 64 float16) of the tile into shared memory (rows = the tile's pixels, dense) and one
  // thread per chunk stores the box (chunk, wt, th, nb) through out_map.
  CUtensorMap out_map;           // 4-D (channel, w, h, n) over the output view
  int tma_out;                   // 1: epilogue through out_map, 0: direct stores
  int stage_off;                 // byte offset of the staging buffers in dynamic shared memory
  int stage_reserved;            // bytes set aside for them behind the filter ring (0: they reuse the
                                 // operand buffers, which are dead when a CTA's only tile is done)
  int stage_bytes;               // bytes of one staging buffer (1024-byte multiple)
  int stage_nbuf;                // staging buffers (a multiple of the number of warp groups)
};
constexpr int kSlabStageBytes = 64 * 1024;    // staging buffers of the TMA-store epilogue (all groups)
constexpr int kSlabSmemBudget = 220 * 1024;   // slab buffers + filter ring; the rest of the 227 KB
                                              // holds barriers and the epilogue's transpose tiles
cudaError_t launch_conv_slab(const SlabConvParams& p, int dtype, int bn, int num_sms, cudaStream_t s);

// ---- 1x1 layers on CTA pairs (gemm_pair.cu): float16, tiles of 256 pixels x 256 filters ------------
struct alignas(64) PairGemmParams {
  CUtensorMap view;              // 5-D (c, group = 1, pixel, 1, 1) over the activations, box (64, 1, 128, 1, 1)
  CUtensorMap wmap;              // 3-D packed filters, box (64, 128, 1)
  CUtensorMap out_map;           // 4-D (channel, pixel, 1, 1) over the output, box (64, 128, 1, 1)
  int kblocks;                   // ceil(channels / 64)
  int tiles_pix, tiles_co;       // 256-pixel tiles, 256-filter tiles
  int pixels, n_out;
  int stages;                    // ring depth (2 .. 5)
  const float* bias;
  int relu;
  ConvEpilogue epi;
  int* status;
  long long wait_clocks;
};
int gemm_pair_smem_bytes(int stages);
cudaError_t launch_gemm_pair(const PairGemmParams& p, int num_sms, cudaStream_t s);

// ---- implicit-GEMM filter gradient (wgrad_umma.cu) -------------------------------------
struct alignas(64) UmmaWgradParams {
  CUtensorMap dy_map;            // 5-D (k_in_group, group, wo, ho, n) over dy, box 32/64 channels
  CUtensorMap x_views[kMaxViews];// 5-D views over x (stride parity classes)
  ConvTap taps[kMaxTaps];        // wmat = flat filter tap index i*kW + j (after flip)
  int ntaps;
  int groups;
  int Kg, Cg;                    // filters / channels per group
  int Wo, Ho, Nimg;
  int bw, bh, bn;                // pixel box per stage (bw*bh*bn <= wgrad_pix(dtype))
  int tiles_w, tiles_h, tiles_n; // pixel tiles covering (Wo, Ho, N)
  int ktiles, ctiles;            // 128-filter tiles, BN-channel tiles
  int splits;                    // split-K slices
  float* partial;                // [splits][taps_total][K][Cg] float32 (or the final buffer)
  long long partial_elems;       // its extent (checked in the range-checked build)
  int taps_total;                // kH*kW
  int atomic;                    // 1: red.add into partial[0] instead of per-split slabs
  int* status;
  long long wait_clocks;          // bound of every device-side wait, in SM clocks
  long long* trace;              // optional: 16 clock counters per CTA (phase timing), or null
};
// Pixels (reduction rows) per pipeline stage of the gradWeights kernels.  A float16 MMA consumes 16
// rows, a tf32 MMA 8: twice the rows for float16 give every stage the same number of MMAs, so that the
// issuing thread's per-stage hand-over (a few hundred clocks) weighs the same.
// With 256 channel columns a float16 stage of 128 pixels is 96 KB, and only two fit the shared memory: too
// few copies in flight for the latency of L2 and HBM.  Those launches use 64-pixel stages (four of them).
#ifndef B200_WGRAD_PIX_WIDE
#define B200_WGRAD_PIX_WIDE 64
#endif
constexpr int kWgradPixF32 = 64, kWgradPixF16 = 128, kWgradPixF16Wide = B200_WGRAD_PIX_WIDE;
inline int wgrad_pix(int dtype, int bn_cols = 0) {
  return dtype == B200CONV_F16 ? (bn_cols >= 256 ? kWgradPixF16Wide : kWgradPixF16) : kWgradPixF32;
}
cudaError_t launch_wgrad_umma(const UmmaWgradParams& p, int dtype, int bn_cols, int num_sms,
                              cudaStream_t s);
// The same work on pairs of CTAs (wgrad_pair.cu): float16, 256-filter x 256-channel tiles, stages of 64 pixels;
// `ktiles` / `ctiles` count 256-wide tiles.
cudaError_t launch_wgrad_pair(const UmmaWgradParams& p, int num_sms, cudaStream_t s);
// Sums split-K slabs and writes the OIHW gradient: out[k][c][tap] = sum_s partial[s][tap][k][c].
cudaError_t launch_wgrad_reduce(const float* partial, void* dw, int splits, int taps, int K,
                                int Cg, int dtype, cudaStream_t s);

// ---- filter gradient with tap groups sharing their operands (wgrad_group.cu) -------------
// Taps that read the same view with the same row offset differ only by a column offset.  With
// the reduction pixels laid out on a grid whose rows are padded by that column span, a tap's x
// operand is the shared x tile advanced by (dw - dw_min) rows, so one dy tile and one x tile per
// stage serve up to four taps (four 128 x 128 accumulators in TMEM).
constexpr int kMaxTapGroups = 32;
struct alignas(64) GroupWgradParams {
  CUtensorMap dy_map;              // box (atom, 1, Wa, th, nb)
  CUtensorMap x_views[kMaxViews];  // box (atom, 1, Wb, th, nb), one per stride parity class
  int16_t grp_view[kMaxTapGroups], grp_dh[kMaxTapGroups], grp_first[kMaxTapGroups], grp_n[kMaxTapGroups];
  int16_t view_dwmin[kMaxViews];
  int16_t tap_off[kMaxTaps];       // dw - dw_min of the tap's view: row offset into the x tile
  int16_t tap_wmat[kMaxTaps];      // filter tap index in OIHW order (after flip)
  int stack_step;                  // > 0: at most 64 channels and the taps of every group this many rows apart:
                                   // a group's taps are column groups of one MMA (0: one MMA per tap)
  int ngroups;
  int groups;                      // convolution groups
  int Kg, Cg;
  int Wo, Ho, Nimg;
  int Wa, Wb, th, nb;              // dy / x box widths, rows and images per stage
  int wt;                          // output columns owned by a tile (== Wo in full-width mode)
  int rows_a, rows_b;              // box rows Wa*th*nb, Wb*th*nb
  int tiles_w, tiles_h, tiles_n;
  int ktiles, ctiles;
  int splits;
  float* partial;                  // [splits][taps_total][K][Cg]
  long long partial_elems;         // its extent (checked in the range-checked build)
  int taps_total;
  int atomic;
  int* status;
  long long wait_clocks;          // bound of every device-side wait, in SM clocks
  long long* trace;                // optional: 16 clock counters per CTA (phase timing), or null
};
cudaError_t launch_wgrad_group(const GroupWgradParams& p, int dtype, int num_sms, cudaStream_t s);

// ---- strided gradInputs with few channels: parity classes merged into channels ---------------
// src[u][cls] = filter tap (i * kW + j, correlation coordinates) that class `cls` applies at the
// merged offset u, or -1 when the class has no tap there.
constexpr int kMaxParityClasses = 16;
struct MergedTapTable {
  int16_t src[kMaxTaps][kMaxParityClasses];
};
// dst[u][cls * C + c][kf] (`rows` rows per offset, the ones past ncls * C zero; row length ldw, zero
// padded) = w[kf][c][tap src[u][cls]] (flipped storage position when flip), zero where src is -1.
cudaError_t launch_pack_filters_merged(const void* w, void* dst, int K, int C, int kH, int kW, int flip,
                                       const MergedTapTable& tb, int nu, int ncls, int rows, int ldw,
                                       int dtype, cudaStream_t s);
// dx[n][c][h][w] (or channels-last with Cp channels, pad channels zeroed) =
// tmp[n][h / sH][w / sW][((h % sH) * sW + w % sW) * C + c], tmp channels-last with Ct channels.
cudaError_t launch_depth_to_space(const void* tmp, void* dx, int N, int C, int H, int W, int sH, int sW,
                                  int Ct, int Cp, int nhwc, int dtype, cudaStream_t s);

// ---- layout kernels (layout.cu) ---------------------------------------------------------
// in[b][r][s] (row length ld_in) -> out[b][s][r] (row length ld_out, zero filled past R).
cudaError_t launch_transpose(const void* in, void* out, int B, int R, int S, int ld_in,
                             int ld_out, int dtype, cudaStream_t s);
// Filter packing; mode 0: forward (rows = filters, cols = channels),
// mode 1: input gradient (rows = channels, cols = filters).  dst[(tap*groups+g)][rows][ldc].
cudaError_t launch_pack_filters(const void* w, void* dst, int K, int Cg, int kH, int kW,
                                int groups, int flip, int mode, int ldc, int dtype,
                                cudaStream_t s);
// Many filter banks packed by one launch (b200conv_prepack): the grid of job j is gx * gy * gz
// blocks of launch_pack_filters' own grid, starting at block first_block.
struct PackJob {
  const void* src;
  void* dst;
  int K, Cg, kH, kW, groups, flip, mode, ldc;
  int gx, gy, first_block;
};
constexpr int kPackBatchJobs = 56;             // 56 x 64 bytes stay below the 4 KB kernel-parameter limit
struct PackBatch {
  PackJob jobs[kPackBatchJobs];
  int njobs;
};
void pack_filters_grid(int Kg, int Cg, int groups, int mode, int ldc, int taps, int* gx, int* gy, int* gz);
cudaError_t launch_pack_filters_batch(const PackBatch& b, int total_blocks, int dtype, cudaStream_t s);
// Row folding for layers with very few input channels (see layout.cu).
cudaError_t launch_pad_fold(const void* src, void* dst, int N, int C, int H, int W, int Cp, int Wp,
                            int pad_l, int nhwc_in, int dtype, cudaStream_t s);
cudaError_t launch_pack_filters_fold(const void* w, void* dst, int K, int C, int kH, int kW, int Cp,
                                     int ld, int flip, int dtype, cudaStream_t s);
// Space-to-depth form of stride-2 layers with very few channels (see layout.cu).
constexpr int kS2dChannels = 16;   // channels of one 2 x 2 pixel block: 4 x C <= 16
constexpr int kS2dPixels = 4;      // consecutive blocks one filter row may span
cudaError_t launch_pad_s2d(const void* src, void* dst, int N, int C, int H, int W, int Cp_in, int H2,
                           int Wq, int q0, int nhwc_in, int dtype, cudaStream_t s);
cudaError_t launch_pack_filters_s2d(const void* w, void* dst, int K, int C, int kH, int kW, int ntaps,
                                    int t0, int q0, int padH, int padW, int ld, int flip, int dtype,
                                    cudaStream_t s);
cudaError_t launch_wgrad_reduce_s2d(const float* partial, void* dw, int splits, int K, int C, int kH,
                                    int kW, int ntaps, int t0, int q0, int padH, int padW, int ld, int flip,
                                    int dtype, cudaStream_t s);
cudaError_t launch_wgrad_reduce_fold(const float* partial, void* dw, int splits, int K, int C, int kH,
                                     int kW, int Cp, int ld, int flip, int dtype, cudaStream_t s);
// Block-diagonal filters for merged groups (extract = 0) and the inverse for the gradient (1).
cudaError_t launch_merge_groups(const void* src, void* dst, int K, int Cg, int Kg, int m, int taps,
                                int extract, int dtype, cudaStream_t s);
cudaError_t launch_convert_bias(const void* bias, float* dst, int n, int dtype, cudaStream_t s);
cudaError_t launch_convert_to_half(const float* src, void* dst, int n, cudaStream_t s);
cudaError_t launch_maxpool2x2(const void* x, void* y, int N, int C, int H, int W, int nhwc,
                              int Cp, int dtype, cudaStream_t s);
cudaError_t launch_maxpool2x2_grad(const void* x, const void* y, const void* gy, void* gx, int N, int C,
                                   int H, int W, int nhwc, int Cp, int dtype, cudaStream_t s);
cudaError_t launch_fill_l2(void* buf, size_t bytes, cudaStream_t s);

// ---- element-wise kernels on channels-last tensors and the per-channel sum (elementwise.cu) ----
enum : int { kEwAdd = 0, kEwMul, kEwSub, kEwRSub, kEwDiv, kEwRDiv, kEwMax, kEwAbs, kEwSgn, kEwNeg, kEwCount };
// out = op(a, b) over `elems` stored elements (a multiple of Cp); b_kind 0: tensor, 1: scalar s, 2: float32 vector
// of Cp values indexed by the stored channel, 3: unary.
cudaError_t launch_elementwise(const void* a, const void* b, const float* chan, void* out, long long elems, int C,
                               int Cp, int op, int b_kind, float s, int dtype, cudaStream_t st);
int channel_sum_blocks(long long pixels);          // rows of Cp floats the partial buffer needs
cudaError_t launch_channel_sum(const void* x, float* partial, float* out, long long pixels, int C, int Cp, int dtype,
                               cudaStream_t st);

// ---- bounded-wait self-test (selftest.cu): one CTA waits, with `limit`, on a barrier nobody arrives on
cudaError_t launch_wait_selftest(int* status, long long limit, cudaStream_t s);

// ---- CUDA-core direct kernels (conv_direct.cu) ---------------------------------------------
cudaError_t launch_direct_fwd(const b200conv_desc& d, const void* x, const void* w,
                              const float* bias, void* y, int relu, const ConvEpilogue& epi, cudaStream_t s);
cudaError_t launch_direct_dgrad(const b200conv_desc& d, const void* w, const void* dy, void* dx,
                                cudaStream_t s);
cudaError_t launch_direct_wgrad(const b200conv_desc& d, const void* x, const void* dy, void* dw,
                                cudaStream_t s);

}  // namespace b200
