// Memory-bound helper kernels: NCHW <-> channels-last transposes, filter packing for the
// implicit-GEMM kernels, bias conversion, 2x2 max pooling and the L2 flush.
#include "internal.h"

namespace b200 {
namespace {

// in[b][r][s] -> out[b][s][r]; 32x32 tiles through shared memory so that both the read
// (along s) and the write (along r) are coalesced.  Rows r in [R, ld_out) are zero filled.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int S,
                                 int ld_in, int ld_out) {
  __shared__ T tile[32][33];
  const long long b = blockIdx.z;
  const T* src = in + b * R * ld_in;
  T* dst = out + b * S * ld_out;
  const int r0 = blockIdx.y * 32, s0 = blockIdx.x * 32;
  for (int dr = threadIdx.y; dr < 32; dr += blockDim.y) {
    const int r = r0 + dr, s = s0 + threadIdx.x;
    tile[dr][threadIdx.x] = (r < R && s < S) ? src[1LL * r * ld_in + s] : T(0);
  }
  __syncthreads();
  for (int ds = threadIdx.y; ds < 32; ds += blockDim.y) {
    const int s = s0 + ds, r = r0 + threadIdx.x;
    if (s < S && r < ld_out) dst[1LL * s * ld_out + r] = tile[threadIdx.x][ds];
  }
}

// Filters OIHW w[K][Cg][kH][kW] -> dst[(tap*groups + g)][rows][ldc] (zero padded columns):
//   mode 0 (forward):        rows = filters of the group, cols = channels,
//                            tap t = i*kW + j multiplies the pixel at offset (i, j);
//   mode 1 (input gradient): rows = channels, cols = filters of the group.
// With flip the correlation tap (i, j) reads w[..][kH-1-i][kW-1-j].
// One block moves a small patch of (filters x channels) for a chunk of taps through shared
// memory: the read runs along (channel, tap), which is contiguous in OIHW, the write along the
// destination's column index.  The patch is 8 filters x 32 channels for mode 0 and 32 filters x
// 8 channels for mode 1, so that 32 consecutive destination columns are written together and
// there are enough blocks to fill the GPU.
constexpr int kPackTaps = 9;
// MODE and the tap count (TAPS = kH * kW for the usual 1 and 9, 0 = any, read at run time) are
// template parameters: the element loop divides by patch width x taps, and with run-time divisors
// those divisions, not the memory traffic, set the pace (47 MB of ResNet-50 filters took 0.4 ms).
template <typename T, int MODE, int TAPS>
__device__ __forceinline__ void pack_filters_block_t(const T* __restrict__ w, T* __restrict__ dst, int K, int Cg,
                                                     int kH, int kW, int groups, int flip, int ldc,
                                                     int bx, int by, int bz, T* tile) {
  constexpr int PK = MODE == 0 ? 8 : 32, PC = MODE == 0 ? 32 : 8;
  constexpr int pitch = PC * kPackTaps + 1;
  const int Kg = K / groups, T_ = TAPS > 0 ? TAPS : kH * kW;
  const int g = bz;
  const int k0 = by * PK, c0 = bx * PC;
  const int rows = MODE == 0 ? Kg : Cg;
  const int tid = threadIdx.y * 32 + threadIdx.x;
  for (int t0 = 0; t0 < T_; t0 += kPackTaps) {
    const int nt = min(kPackTaps, T_ - t0);
    // load: for one filter, PC channels x all taps are contiguous in memory
    for (int i = tid; i < PK * PC * T_; i += 256) {
      const int kk = i / (PC * T_), rem = i % (PC * T_);
      const int cc = rem / T_, tt = rem % T_;
      if (tt < t0 || tt >= t0 + nt) continue;
      const int kq = k0 + kk;
      T v = T(0);
      if (kq < Kg && c0 + cc < Cg) v = w[(1LL * (g * Kg + kq) * Cg + c0 + cc) * T_ + tt];
      tile[kk * pitch + cc * kPackTaps + (tt - t0)] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const int src_tap = t0 + tt;                       // position in the filter as stored
      const int i = src_tap / kW, j = src_tap % kW;
      const int tap = flip ? (kH - 1 - i) * kW + (kW - 1 - j) : src_tap;   // correlation tap it serves
      T* d = dst + 1LL * (tap * groups + g) * rows * ldc;
      const int rr = threadIdx.y, xx = threadIdx.x;
      if (MODE == 0) {       // row = filter (8 per block), col = channel (32 per block)
        const int kq = k0 + rr, c = c0 + xx;
        if (kq < Kg && c < ldc) d[1LL * kq * ldc + c] = c < Cg ? tile[rr * pitch + xx * kPackTaps + tt] : T(0);
      } else {               // row = channel (8 per block), col = filter (32 per block)
        const int c = c0 + rr, kq = k0 + xx;
        if (c < Cg && kq < ldc) d[1LL * c * ldc + kq] = kq < Kg ? tile[xx * pitch + rr * kPackTaps + tt] : T(0);
      }
    }
    __syncthreads();
  }
}

template <typename T>
__device__ __forceinline__ void pack_filters_block(const T* __restrict__ w, T* __restrict__ dst, int K, int Cg,
                                                   int kH, int kW, int groups, int flip, int mode, int ldc,
                                                   int bx, int by, int bz) {
  __shared__ T tile[256 * kPackTaps + 40];
  const int taps = kH * kW;
  if (mode == 0) {
    if (taps == 9) pack_filters_block_t<T, 0, 9>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
    else if (taps == 1) pack_filters_block_t<T, 0, 1>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
    else pack_filters_block_t<T, 0, 0>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
  } else {
    if (taps == 9) pack_filters_block_t<T, 1, 9>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
    else if (taps == 1) pack_filters_block_t<T, 1, 1>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
    else pack_filters_block_t<T, 1, 0>(w, dst, K, Cg, kH, kW, groups, flip, ldc, bx, by, bz, tile);
  }
}

template <typename T>
__global__ void pack_filters_kernel(const T* __restrict__ w, T* __restrict__ dst, int K, int Cg,
                                    int kH, int kW, int groups, int flip, int mode, int ldc) {
  pack_filters_block<T>(w, dst, K, Cg, kH, kW, groups, flip, mode, ldc, blockIdx.x, blockIdx.y, blockIdx.z);
}

// Many filter banks in one launch: block b belongs to the job j with first_block[j] <= b <
// first_block[j + 1] and does there what block (bx, by, bz) of pack_filters_kernel would do.
// 1x1 banks for gradInputs are plain transposes [K][C] -> [C][ldc]: 64 x 64 tiles through shared memory, read
// along c and written along k in 128-byte runs (the general patch kernel moves 16-byte runs here).
template <typename T>
__device__ __forceinline__ void transpose_1x1_block(const T* __restrict__ w, T* __restrict__ dst, int K, int Cg, int groups,
                                                    int ldc, int bx, int by, int bz) {
  __shared__ T tile[64][65];
  const int Kg = K / groups;
  const int k0 = bx * 64, c0 = by * 64, g = bz;
  const int tid = threadIdx.y * 32 + threadIdx.x;
  for (int i = tid; i < 64 * 64; i += 256) {
    const int kk = i >> 6, cc = i & 63;
    T v = T(0);
    if (k0 + kk < Kg && c0 + cc < Cg) v = w[(1LL * (g * Kg + k0 + kk)) * Cg + c0 + cc];
    tile[kk][cc] = v;
  }
  __syncthreads();
  T* d = dst + 1LL * g * Cg * ldc;
  for (int i = tid; i < 64 * 64; i += 256) {
    const int cc = i >> 6, kk = i & 63;
    if (c0 + cc < Cg && k0 + kk < ldc) d[1LL * (c0 + cc) * ldc + k0 + kk] = tile[kk][cc];
  }
}

template <typename T>
__global__ void pack_filters_batch_kernel(const __grid_constant__ PackBatch b) {
  int j = 0;
  while (j + 1 < b.njobs && static_cast<int>(blockIdx.x) >= b.jobs[j + 1].first_block) ++j;
  const PackJob& q = b.jobs[j];
  int local = blockIdx.x - q.first_block;
  const int bx = local % q.gx;
  local /= q.gx;
  const int by = local % q.gy, bz = local / q.gy;
  if (q.kH * q.kW == 1 && q.mode == 1) {
    transpose_1x1_block<T>(static_cast<const T*>(q.src), static_cast<T*>(q.dst), q.K, q.Cg, q.groups, q.ldc, bx, by, bz);
    return;
  }
  pack_filters_block<T>(static_cast<const T*>(q.src), static_cast<T*>(q.dst), q.K, q.Cg, q.kH, q.kW, q.groups, q.flip,
                        q.mode, q.ldc, bx, by, bz);
}

// Few-channel layers ("row folding"): the image is copied channels-last with explicit zero
// columns left and right, [N][H][Wp][Cp], so that the kW * Cp values under one filter row are
// contiguous and can serve as one reduction block of the implicit GEMM.  One thread per output
// pixel; src is NCHW (nhwc_in = 0) or channels-last [N][H][W][Cp].
template <typename T>
__global__ void pad_fold_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int C, int H,
                                int W, int Cp, int Wp, int pad_l, int nhwc_in) {
  const long long total = 1LL * N * H * Wp;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int wp = idx % Wp;
    const int h = (idx / Wp) % H;
    const int n = idx / (1LL * Wp * H);
    const int w = wp - pad_l;
    const bool inside = w >= 0 && w < W;
    if (Cp * sizeof(T) == 16) {
      // one pixel is 16 bytes: assemble it in registers, store it once
      uint4 px = make_uint4(0, 0, 0, 0);
      if (inside) {
        if (nhwc_in) {
          px = *reinterpret_cast<const uint4*>(src + ((1LL * n * H + h) * W + w) * Cp);
        } else {
          T* v = reinterpret_cast<T*>(&px);
          for (int c = 0; c < C; ++c) v[c] = src[((1LL * n * C + c) * H + h) * W + w];
        }
      }
      *reinterpret_cast<uint4*>(dst + idx * Cp) = px;
      continue;
    }
    T* d = dst + idx * Cp;
    for (int c = 0; c < Cp; ++c) {
      T v = T(0);
      if (inside && c < C)
        v = nhwc_in ? src[((1LL * n * H + h) * W + w) * Cp + c] : src[((1LL * n * C + c) * H + h) * W + w];
      d[c] = v;
    }
  }
}

// Folded filters: dst[i][k][j*Cp + c] = w[k][c][i'][j'] (zero elsewhere up to ld columns), where
// (i', j') = (i, j) or the flipped position.
template <typename T>
__global__ void pack_filters_fold_kernel(const T* __restrict__ w, T* __restrict__ dst, int K, int C,
                                         int kH, int kW, int Cp, int ld, int flip) {
  const long long total = 1LL * kH * K * ld;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int col = idx % ld;
    const int k = (idx / ld) % K;
    const int i = idx / (1LL * ld * K);
    const int j = col / Cp, c = col % Cp;
    T v = T(0);
    if (j < kW && c < C) {
      const int wi = flip ? kH - 1 - i : i, wj = flip ? kW - 1 - j : j;
      v = w[((1LL * k * C + c) * kH + wi) * kW + wj];
    }
    dst[idx] = v;
  }
}

// Space-to-depth for stride-2 layers with very few channels (the 7x7 stride-2 stems): a 2 x 2 block
// of input pixels becomes one pixel of kS2dChannels channels,
//   dst[n][h2][q][(dy*2 + dx)*C + c] = src[n][c][2*h2 + dy][2*(q + q0) + dx]
// with zeros outside the image and in the unused channels.  The layer then is a stride-1 layer over
// dst whose filter rows span a few consecutive pixels: one contiguous reduction block per row.
// One thread per dst pixel; src is NCHW (nhwc_in = 0) or channels-last [N][H][W][Cp_in].
template <typename T, int C>
__global__ void pad_s2d_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int H,
                               int W, int Cp_in, int H2, int Wq, int q0, int nhwc_in) {
  const long long total = 1LL * N * H2 * Wq;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int q = idx % Wq;
    const int h2 = (idx / Wq) % H2;
    const int n = idx / (1LL * Wq * H2);
    __align__(16) T v[kS2dChannels];
#pragma unroll
    for (int i = 0; i < kS2dChannels; ++i) v[i] = T(0);
#pragma unroll
    for (int par = 0; par < 4; ++par) {
      const int h = 2 * h2 + (par >> 1), w = 2 * (q + q0) + (par & 1);
      if (h < H && w >= 0 && w < W) {
        if (nhwc_in && Cp_in * sizeof(T) == 16) {     // one source pixel is one 16-byte load
          const uint4 px = *reinterpret_cast<const uint4*>(src + ((1LL * n * H + h) * W + w) * Cp_in);
          const T* e = reinterpret_cast<const T*>(&px);
#pragma unroll
          for (int c = 0; c < C; ++c) v[par * C + c] = e[c];
        } else {
#pragma unroll
          for (int c = 0; c < C; ++c)
            v[par * C + c] = nhwc_in ? src[((1LL * n * H + h) * W + w) * Cp_in + c]
                                     : src[((1LL * n * C + c) * H + h) * W + w];
        }
      }
    }
    uint4* d = reinterpret_cast<uint4*>(dst + idx * kS2dChannels);
    const uint4* sv = reinterpret_cast<const uint4*>(v);
#pragma unroll
    for (int i = 0; i < (int)(kS2dChannels * sizeof(T) / 16); ++i) d[i] = sv[i];
  }
}

// Filters for the space-to-depth form: dst[t][k][j*kS2dChannels + (dy*2 + dx)*C + c] is the filter
// element that multiplies input pixel (2*(t + t0) + dy, 2*(j + q0) + dx) relative to the output
// position times the stride, i.e. tap (i, jj) = (2*(t + t0) + dy + padH, 2*(j + q0) + dx + padW);
// zero where that tap does not exist.
template <typename T>
__global__ void pack_filters_s2d_kernel(const T* __restrict__ w, T* __restrict__ dst, int K, int C,
                                        int kH, int kW, int ntaps, int t0, int q0, int padH, int padW,
                                        int ld, int flip) {
  const long long total = 1LL * ntaps * K * ld;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int col = idx % ld;
    const int k = (idx / ld) % K;
    const int t = idx / (1LL * ld * K);
    const int j = col / kS2dChannels, r = col % kS2dChannels;
    T v = T(0);
    if (r < 4 * C) {
      const int par = r / C, c = r % C;
      const int i = 2 * (t + t0) + (par >> 1) + padH, jj = 2 * (j + q0) + (par & 1) + padW;
      if (i >= 0 && i < kH && jj >= 0 && jj < kW) {
        const int wi = flip ? kH - 1 - i : i, wj = flip ? kW - 1 - jj : jj;
        v = w[((1LL * k * C + c) * kH + wi) * kW + wj];
      }
    }
    dst[idx] = v;
  }
}

// Filter gradient of the space-to-depth form: dw[k][c][i'][j'] = sum_s partial[s][t][k][col] with
// (t, col) the place pack_filters_s2d_kernel gives tap (i, jj).
template <typename T>
__global__ void wgrad_reduce_s2d_kernel(const float* __restrict__ partial, T* __restrict__ dw, int splits,
                                        int K, int C, int kH, int kW, int ntaps, int t0, int q0, int padH,
                                        int padW, int ld, int flip) {
  const long long total = 1LL * K * C * kH * kW;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int wj = idx % kW;
    const int wi = (idx / kW) % kH;
    const int c = (idx / (1LL * kW * kH)) % C;
    const int k = idx / (1LL * kW * kH * C);
    const int i = flip ? kH - 1 - wi : wi, jj = flip ? kW - 1 - wj : wj;
    const int ah = i - padH, aw = jj - padW;                 // offsets from 2 * the output position
    const int th = ah >= 0 ? ah / 2 : -((1 - ah) / 2), tw = aw >= 0 ? aw / 2 : -((1 - aw) / 2);   // floor
    const int par = (ah - 2 * th) * 2 + (aw - 2 * tw);
    const int t = th - t0, col = (tw - q0) * kS2dChannels + par * C + c;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s)
      acc += partial[((1LL * s * ntaps + t) * K + k) * ld + col];
    dw[idx] = static_cast<T>(acc);
  }
}

// Folded filter gradient: dw[k][c][i'][j'] = sum_s partial[s][i][k][j*Cp + c].
template <typename T>
__global__ void wgrad_reduce_fold_kernel(const float* __restrict__ partial, T* __restrict__ dw,
                                         int splits, int K, int C, int kH, int kW, int Cp, int ld,
                                         int flip) {
  const long long total = 1LL * K * C * kH * kW;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int wj = idx % kW;
    const int wi = (idx / kW) % kH;
    const int c = (idx / (1LL * kW * kH)) % C;
    const int k = idx / (1LL * kW * kH * C);
    const int i = flip ? kH - 1 - wi : wi, j = flip ? kW - 1 - wj : wj;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s)
      acc += partial[((1LL * s * kH + i) * K + k) * ld + j * Cp + c];
    dw[idx] = static_cast<T>(acc);
  }
}

// Grouped convolutions with few channels per group: m neighbouring groups are merged into one
// group with block-diagonal filters, so that a reduction block of the MMA is filled with real
// channels.  expand: wm[k][c'][t] = w[k][c' % Cg][t] if column block c'/Cg belongs to filter k's
// group, else 0 (wm has m*Cg columns).  extract is the inverse for the filter gradient.
template <typename T>
__global__ void merge_groups_kernel(const T* __restrict__ src, T* __restrict__ dst, int K, int Cg,
                                    int Kg, int m, int taps, int extract) {
  const int CgE = Cg * m;
  const long long total = 1LL * K * (extract ? Cg : CgE) * taps;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int t = idx % taps;
    if (extract) {
      const int c = (idx / taps) % Cg;
      const int k = idx / (1LL * taps * Cg);
      const int blk = (k % (Kg * m)) / Kg;
      dst[idx] = src[(1LL * k * CgE + blk * Cg + c) * taps + t];
    } else {
      const int ce = (idx / taps) % CgE;
      const int k = idx / (1LL * taps * CgE);
      const int blk = (k % (Kg * m)) / Kg;
      dst[idx] = (ce / Cg == blk) ? src[(1LL * k * Cg + ce % Cg) * taps + t] : T(0);
    }
  }
}

template <typename T>
__global__ void convert_bias_kernel(const T* __restrict__ b, float* __restrict__ dst, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = static_cast<float>(b[i]);
}

// NCHW: one thread per output element.  NHWC: one thread per (pixel, channel) with the
// channel fastest, so neighbouring threads read neighbouring addresses.
template <typename T>
__global__ void maxpool2x2_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int C, int H,
                                  int W, int nhwc, int Cp) {
  const int Ho = H / 2, Wo = W / 2;
  const int Cx = nhwc ? Cp : C;
  const long long total = 1LL * N * Cx * Ho * Wo;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    if (nhwc) {
      const int c = idx % Cp;
      const int ow = (idx / Cp) % Wo;
      const int oh = (idx / (1LL * Cp * Wo)) % Ho;
      const int n = idx / (1LL * Cp * Wo * Ho);
      const T* p = x + ((1LL * n * H + 2 * oh) * W + 2 * ow) * Cp + c;
      float m = static_cast<float>(p[0]);
      m = fmaxf(m, static_cast<float>(p[Cp]));
      m = fmaxf(m, static_cast<float>(p[1LL * W * Cp]));
      m = fmaxf(m, static_cast<float>(p[1LL * W * Cp + Cp]));
      y[idx] = static_cast<T>(m);
    } else {
      const int ow = idx % Wo;
      const int oh = (idx / Wo) % Ho;
      const long long nc = idx / (1LL * Wo * Ho);
      const T* p = x + (nc * H + 2 * oh) * W + 2 * ow;
      float m = static_cast<float>(p[0]);
      m = fmaxf(m, static_cast<float>(p[1]));
      m = fmaxf(m, static_cast<float>(p[W]));
      m = fmaxf(m, static_cast<float>(p[W + 1]));
      y[idx] = static_cast<T>(m);
    }
  }
}

// Gradient of the 2x2 / stride 2 max pooling: one thread per input element (so every element of
// gx is written): gx = gy of its window if x equals the window maximum, else 0.
template <typename T>
__global__ void maxpool2x2_grad_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                       const T* __restrict__ gy, T* __restrict__ gx, int N, int C, int H,
                                       int W, int nhwc, int Cp) {
  const int Ho = H / 2, Wo = W / 2;
  const int Cx = nhwc ? Cp : C;
  const long long total = 1LL * N * Cx * H * W;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    int h, w;
    long long o;            // index of the window in y / gy
    if (nhwc) {
      const int c = idx % Cp;
      w = (idx / Cp) % W;
      h = (idx / (1LL * Cp * W)) % H;
      const long long n = idx / (1LL * Cp * W * H);
      o = ((n * Ho + h / 2) * Wo + w / 2) * Cp + c;
    } else {
      w = idx % W;
      h = (idx / W) % H;
      const long long nc = idx / (1LL * W * H);
      o = (nc * Ho + h / 2) * Wo + w / 2;
    }
    T g = static_cast<T>(0.f);
    if (h < 2 * Ho && w < 2 * Wo && static_cast<float>(x[idx]) == static_cast<float>(y[o])) g = gy[o];
    gx[idx] = g;
  }
}

template <typename T>
__global__ void pack_filters_merged_kernel(const T* __restrict__ w, T* __restrict__ dst, int K, int C, int kH,
                                           int kW, int flip, MergedTapTable tb, int nu, int ncls, int rows, int ldw) {
  const long long total = 1LL * nu * rows * ldw;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int kf = idx % ldw;
    const int row = (idx / ldw) % rows;
    const int u = idx / (1LL * ldw * rows);
    const int cls = row / C, c = row % C;
    const int tap = cls < ncls ? tb.src[u][cls] : -1;     // rows past ncls * C are zero padding
    T v = T(0);
    if (tap >= 0 && kf < K) {
      const int i = tap / kW, j = tap % kW;
      const int pos = flip ? (kH - 1 - i) * kW + (kW - 1 - j) : tap;
      v = w[(1LL * kf * C + c) * kH * kW + pos];
    }
    dst[idx] = v;
  }
}

// NCHW output: one thread per element.  Channels-last output: one thread per pixel, which reads
// its C values (contiguous in tmp) and writes the whole padded channel vector in 16-byte pieces.
template <typename T>
__global__ void depth_to_space_kernel(const T* __restrict__ tmp, T* __restrict__ dx, int N, int C, int H, int W,
                                      int sH, int sW, int Ct, int Cp, int nhwc) {
  const int Hq = (H + sH - 1) / sH, Wq = (W + sW - 1) / sW;
  if (nhwc) {
    constexpr int kVec = 16 / static_cast<int>(sizeof(T));      // Cp is a multiple of kVec
    const long long total = 1LL * N * H * W;
    for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
         idx += 1LL * gridDim.x * blockDim.x) {
      const int w = idx % W, h = (idx / W) % H;
      const long long n = idx / (1LL * W * H);
      const int cls = (h % sH) * sW + (w % sW);
      const T* src = tmp + ((n * Hq + h / sH) * Wq + w / sW) * Ct + cls * C;
      T* dst = dx + idx * Cp;
      for (int c0 = 0; c0 < Cp; c0 += kVec) {
        T v[kVec];
#pragma unroll
        for (int q = 0; q < kVec; ++q) v[q] = c0 + q < C ? src[c0 + q] : T(0);
        *reinterpret_cast<uint4*>(dst + c0) = *reinterpret_cast<const uint4*>(v);
      }
    }
    return;
  }
  const long long total = 1LL * N * C * H * W;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int w = idx % W, h = (idx / W) % H, c = (idx / (1LL * W * H)) % C;
    const long long n = idx / (1LL * W * H * C);
    const int cls = (h % sH) * sW + (w % sW);
    dx[idx] = tmp[((n * Hq + h / sH) * Wq + w / sW) * Ct + cls * C + c];
  }
}

__global__ void fill_kernel(uint4* buf, size_t n16) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    buf[i] = make_uint4(0, 0, 0, 0);
}

int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = 148LL * 32;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

cudaError_t launch_transpose(const void* in, void* out, int B, int R, int S, int ld_in,
                             int ld_out, int dtype, cudaStream_t s) {
  if (B == 0 || S == 0 || ld_out == 0) return cudaSuccess;
  const int rows = R > ld_out ? R : ld_out;
  for (int b0 = 0; b0 < B; b0 += 65535) {  // gridDim.z limit
    const int nb = (B - b0) < 65535 ? (B - b0) : 65535;
    dim3 grid((S + 31) / 32, (rows + 31) / 32, nb), block(32, 8);
    if (dtype == B200CONV_F16)
      transpose_kernel<__half><<<grid, block, 0, s>>>(
          static_cast<const __half*>(in) + 1LL * b0 * R * ld_in,
          static_cast<__half*>(out) + 1LL * b0 * S * ld_out, R, S, ld_in, ld_out);
    else
      transpose_kernel<float><<<grid, block, 0, s>>>(
          static_cast<const float*>(in) + 1LL * b0 * R * ld_in,
          static_cast<float*>(out) + 1LL * b0 * S * ld_out, R, S, ld_in, ld_out);
  }
  return cudaGetLastError();
}

void pack_filters_grid(int Kg, int Cg, int groups, int mode, int ldc, int taps, int* gx, int* gy, int* gz) {
  if (taps == 1 && mode == 1) {            // the batched kernel's transposing path: 64 x 64 tiles
    *gx = (ldc + 63) / 64;
    *gy = (Cg + 63) / 64;
    *gz = groups;
    return;
  }
  // the patch grid covers the padded column range [0, ldc) of the destination as well
  const int cols_c = mode == 0 ? ldc : Cg, cols_k = mode == 0 ? Kg : ldc;
  const int PK = mode == 0 ? 8 : 32, PC = mode == 0 ? 32 : 8;
  *gx = (cols_c + PC - 1) / PC;
  *gy = (cols_k + PK - 1) / PK;
  *gz = groups;
}

cudaError_t launch_pack_filters_batch(const PackBatch& b, int total_blocks, int dtype, cudaStream_t s) {
  if (b.njobs == 0 || total_blocks == 0) return cudaSuccess;
  if (dtype == B200CONV_F16) pack_filters_batch_kernel<__half><<<total_blocks, dim3(32, 8), 0, s>>>(b);
  else pack_filters_batch_kernel<float><<<total_blocks, dim3(32, 8), 0, s>>>(b);
  return cudaGetLastError();
}

cudaError_t launch_pack_filters(const void* w, void* dst, int K, int Cg, int kH, int kW,
                                int groups, int flip, int mode, int ldc, int dtype,
                                cudaStream_t s) {
  const int Kg = K / groups;
  if (1LL * kH * kW * K * Cg == 0) return cudaSuccess;
  // the patch grid covers the padded column range [0, ldc) of the destination as well
  const int cols_c = mode == 0 ? ldc : Cg, cols_k = mode == 0 ? Kg : ldc;
  const int PK = mode == 0 ? 8 : 32, PC = mode == 0 ? 32 : 8;
  dim3 grid((cols_c + PC - 1) / PC, (cols_k + PK - 1) / PK, groups), block(32, 8);
  if (dtype == B200CONV_F16)
    pack_filters_kernel<__half><<<grid, block, 0, s>>>(static_cast<const __half*>(w),
                                                       static_cast<__half*>(dst), K, Cg, kH, kW,
                                                       groups, flip, mode, ldc);
  else
    pack_filters_kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(w),
                                                      static_cast<float*>(dst), K, Cg, kH, kW, groups,
                                                      flip, mode, ldc);
  return cudaGetLastError();
}

cudaError_t launch_pad_fold(const void* src, void* dst, int N, int C, int H, int W, int Cp, int Wp,
                            int pad_l, int nhwc_in, int dtype, cudaStream_t s) {
  const long long total = 1LL * N * H * Wp;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    pad_fold_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(src), static_cast<__half*>(dst), N, C, H, W, Cp, Wp, pad_l, nhwc_in);
  else
    pad_fold_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(src), static_cast<float*>(dst), N, C, H, W, Cp, Wp, pad_l, nhwc_in);
  return cudaGetLastError();
}

cudaError_t launch_pack_filters_fold(const void* w, void* dst, int K, int C, int kH, int kW, int Cp,
                                     int ld, int flip, int dtype, cudaStream_t s) {
  const long long total = 1LL * kH * K * ld;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    pack_filters_fold_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(w), static_cast<__half*>(dst), K, C, kH, kW, Cp, ld, flip);
  else
    pack_filters_fold_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(w), static_cast<float*>(dst), K, C, kH, kW, Cp, ld, flip);
  return cudaGetLastError();
}

cudaError_t launch_wgrad_reduce_s2d(const float* partial, void* dw, int splits, int K, int C, int kH,
                                    int kW, int ntaps, int t0, int q0, int padH, int padW, int ld, int flip,
                                    int dtype, cudaStream_t s) {
  const long long total = 1LL * K * C * kH * kW;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    wgrad_reduce_s2d_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        partial, static_cast<__half*>(dw), splits, K, C, kH, kW, ntaps, t0, q0, padH, padW, ld, flip);
  else
    wgrad_reduce_s2d_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        partial, static_cast<float*>(dw), splits, K, C, kH, kW, ntaps, t0, q0, padH, padW, ld, flip);
  return cudaGetLastError();
}

template <typename T>
cudaError_t pad_s2d_typed(const void* src, void* dst, int N, int C, int H, int W, int Cp_in, int H2, int Wq,
                          int q0, int nhwc_in, cudaStream_t s) {
  const long long total = 1LL * N * H2 * Wq;
  const T* in = static_cast<const T*>(src);
  T* out = static_cast<T*>(dst);
  const int grid = grid_for(total, 256);
  switch (C) {   // the channel count as a constant keeps the assembled pixel in registers
    case 1: pad_s2d_kernel<T, 1><<<grid, 256, 0, s>>>(in, out, N, H, W, Cp_in, H2, Wq, q0, nhwc_in); break;
    case 2: pad_s2d_kernel<T, 2><<<grid, 256, 0, s>>>(in, out, N, H, W, Cp_in, H2, Wq, q0, nhwc_in); break;
    case 3: pad_s2d_kernel<T, 3><<<grid, 256, 0, s>>>(in, out, N, H, W, Cp_in, H2, Wq, q0, nhwc_in); break;
    case 4: pad_s2d_kernel<T, 4><<<grid, 256, 0, s>>>(in, out, N, H, W, Cp_in, H2, Wq, q0, nhwc_in); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_pad_s2d(const void* src, void* dst, int N, int C, int H, int W, int Cp_in, int H2,
                           int Wq, int q0, int nhwc_in, int dtype, cudaStream_t s) {
  if (1LL * N * H2 * Wq == 0) return cudaSuccess;
  return dtype == B200CONV_F16 ? pad_s2d_typed<__half>(src, dst, N, C, H, W, Cp_in, H2, Wq, q0, nhwc_in, s)
                               : pad_s2d_typed<float>(src, dst, N, C, H, W, Cp_in, H2, Wq, q0, nhwc_in, s);
}

cudaError_t launch_pack_filters_s2d(const void* w, void* dst, int K, int C, int kH, int kW, int ntaps,
                                    int t0, int q0, int padH, int padW, int ld, int flip, int dtype,
                                    cudaStream_t s) {
  const long long total = 1LL * ntaps * K * ld;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    pack_filters_s2d_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(w), static_cast<__half*>(dst), K, C, kH, kW, ntaps, t0, q0, padH, padW, ld, flip);
  else
    pack_filters_s2d_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(w), static_cast<float*>(dst), K, C, kH, kW, ntaps, t0, q0, padH, padW, ld, flip);
  return cudaGetLastError();
}

cudaError_t launch_wgrad_reduce_fold(const float* partial, void* dw, int splits, int K, int C, int kH,
                                     int kW, int Cp, int ld, int flip, int dtype, cudaStream_t s) {
  const long long total = 1LL * K * C * kH * kW;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    wgrad_reduce_fold_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        partial, static_cast<__half*>(dw), splits, K, C, kH, kW, Cp, ld, flip);
  else
    wgrad_reduce_fold_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        partial, static_cast<float*>(dw), splits, K, C, kH, kW, Cp, ld, flip);
  return cudaGetLastError();
}

cudaError_t launch_merge_groups(const void* src, void* dst, int K, int Cg, int Kg, int m, int taps,
                                int extract, int dtype, cudaStream_t s) {
  const long long total = 1LL * K * (extract ? Cg : Cg * m) * taps;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    merge_groups_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(src), static_cast<__half*>(dst), K, Cg, Kg, m, taps, extract);
  else
    merge_groups_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(src), static_cast<float*>(dst), K, Cg, Kg, m, taps, extract);
  return cudaGetLastError();
}

cudaError_t launch_convert_bias(const void* bias, float* dst, int n, int dtype, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    convert_bias_kernel<__half><<<(n + 255) / 256, 256, 0, s>>>(static_cast<const __half*>(bias), dst, n);
  else
    convert_bias_kernel<float><<<(n + 255) / 256, 256, 0, s>>>(static_cast<const float*>(bias), dst, n);
  return cudaGetLastError();
}

__global__ void convert_to_half_kernel(const float* __restrict__ src, __half* __restrict__ dst, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2half_rn(src[i]);
}
cudaError_t launch_convert_to_half(const float* src, void* dst, int n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  convert_to_half_kernel<<<(n + 255) / 256, 256, 0, s>>>(src, static_cast<__half*>(dst), n);
  return cudaGetLastError();
}

cudaError_t launch_maxpool2x2(const void* x, void* y, int N, int C, int H, int W, int nhwc,
                              int Cp, int dtype, cudaStream_t s) {
  const long long total = 1LL * N * (nhwc ? Cp : C) * (H / 2) * (W / 2);
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    maxpool2x2_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), N, C, H, W, nhwc, Cp);
  else
    maxpool2x2_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(x), static_cast<float*>(y), N, C, H, W, nhwc, Cp);
  return cudaGetLastError();
}

cudaError_t launch_maxpool2x2_grad(const void* x, const void* y, const void* gy, void* gx, int N, int C,
                                   int H, int W, int nhwc, int Cp, int dtype, cudaStream_t s) {
  const long long total = 1LL * N * (nhwc ? Cp : C) * H * W;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    maxpool2x2_grad_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(y), static_cast<const __half*>(gy),
        static_cast<__half*>(gx), N, C, H, W, nhwc, Cp);
  else
    maxpool2x2_grad_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(x), static_cast<const float*>(y), static_cast<const float*>(gy),
        static_cast<float*>(gx), N, C, H, W, nhwc, Cp);
  return cudaGetLastError();
}

cudaError_t launch_pack_filters_merged(const void* w, void* dst, int K, int C, int kH, int kW, int flip,
                                       const MergedTapTable& tb, int nu, int ncls, int rows, int ldw,
                                       int dtype, cudaStream_t s) {
  const long long total = 1LL * nu * rows * ldw;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    pack_filters_merged_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(w), static_cast<__half*>(dst), K, C, kH, kW, flip, tb, nu, ncls, rows, ldw);
  else
    pack_filters_merged_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(w), static_cast<float*>(dst), K, C, kH, kW, flip, tb, nu, ncls, rows, ldw);
  return cudaGetLastError();
}

cudaError_t launch_depth_to_space(const void* tmp, void* dx, int N, int C, int H, int W, int sH, int sW,
                                  int Ct, int Cp, int nhwc, int dtype, cudaStream_t s) {
  const long long total = 1LL * N * (nhwc ? 1 : C) * H * W;
  if (total == 0) return cudaSuccess;
  if (dtype == B200CONV_F16)
    depth_to_space_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const __half*>(tmp), static_cast<__half*>(dx), N, C, H, W, sH, sW, Ct, Cp, nhwc);
  else
    depth_to_space_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        static_cast<const float*>(tmp), static_cast<float*>(dx), N, C, H, W, sH, sW, Ct, Cp, nhwc);
  return cudaGetLastError();
}

cudaError_t launch_fill_l2(void* buf, size_t bytes, cudaStream_t s) {
  fill_kernel<<<148 * 8, 256, 0, s>>>(static_cast<uint4*>(buf), bytes / 16);
  return cudaGetLastError();
}

}  // namespace b200
