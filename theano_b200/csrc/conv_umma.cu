// Implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   out[pixel, co] = sum over taps t, channels c of  view_t[pixel + offset_t, c] * filt_t[co, c]
//
// The accumulator tile is 128 output pixels (TMEM lanes) x BN output channels (TMEM
// columns, float32).  A pixel tile is a box bw x bh x bn of the output grid (columns, rows,
// images); for one tap and one block of 32 float32 / 64 float16 channels the activation
// operand is a single TMA box of a channels-last view, landing in shared memory as 128-byte
// rows in the 128-byte-swizzled K-major layout the MMA reads.  Zero padding is the TMA
// out-of-bounds fill; stride > 1 is expressed by views that start at a parity offset with
// doubled pitches; dilation and the input-gradient case only change the tap offsets.
// The same kernel therefore serves forward and gradInputs.
//
// Warp roles (672 threads, one CTA per SM, persistent over tiles):
//   warps 0, 18-20  TMA producers   warp 1   MMA issuer + TMEM owner
//   warps 2-17 epilogue: TMEM -> registers -> (+bias, ReLU) -> global (NCHW or channels-last)
// Shared-memory stages are recycled through full/empty mbarriers; two TMEM accumulators
// let the epilogue of tile i overlap the main loop of tile i+1.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kRows = 128;            // accumulator lanes = pixels per tile
constexpr int kRowBytes = 128;        // one swizzle row: 32 tf32 or 64 f16 channels
constexpr int kABytes = kRows * kRowBytes;
constexpr int kEpilogueWarps = 16;
// One thread gets a TMA box accepted about every 300 clocks, whatever its size; a stage is two
// boxes and at most 512 clocks of MMAs.  Four producer warps share the issue: warp 0 and the
// three warps after the epilogue warps; producer pw issues the activation box (pw even) or the
// filter box (pw odd) of every second stage (parity pw / 2).
constexpr int kProducers = 4;
constexpr int kFirstExtraProducer = 2 + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstExtraProducer + kProducers - 1);
constexpr int kSmemBudget = 200 * 1024;

template <int BN> constexpr int stage_bytes() { return kABytes + BN * kRowBytes; }
template <int BN> constexpr int num_stages() {
  return (kSmemBudget / stage_bytes<BN>()) > 8 ? 8 : (kSmemBudget / stage_bytes<BN>());
}

struct Bars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

template <typename T> struct OutPack;
template <> struct OutPack<float> {
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct OutPack<__half> {
  static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};

template <MmaKind KIND, int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_umma_kernel(const __grid_constant__ UmmaConvParams p) {
  using OutT = typename std::conditional<KIND == MmaKind::TF32, float, __half>::type;
  constexpr int kStages = num_stages<BN>();
  constexpr int kBK = KIND == MmaKind::TF32 ? 32 : 64;   // channels per stage
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, false, false, kRows, BN);
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * stage_bytes<BN>());

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const int rows_used = p.bw * p.bh * p.bn;
  const uint32_t tx_bytes = rows_used * kRowBytes + BN * kRowBytes;
  const int kiters = p.ntaps * p.kblocks;
  // tile counts fit 32 bits (the launcher checks): 64-bit divisions per tile would cost each
  // role about a thousand clocks, a fifth of a small tile
  const uint32_t total = static_cast<uint32_t>(p.tiles_w) * p.tiles_h * p.tiles_n * p.groups * p.tiles_co;
  const uint32_t co_groups = static_cast<uint32_t>(p.tiles_co) * p.groups, tiles_wh = static_cast<uint32_t>(p.tiles_w) * p.tiles_h;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 32 * kEpilogueWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Rows of the A stage that no TMA box ever writes must not hold NaN patterns that would
  // spill into *valid* lanes: they cannot (each accumulator lane depends on its own A row
  // only), so they are left as they are.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0 || warp >= kFirstExtraProducer) {
    // every lane follows the loop (warp-uniform control flow and addresses), one elected lane issues
    const bool leader = elect_one();
    const int pw = warp == 0 ? 0 : warp - kFirstExtraProducer + 1;
    const bool b_box = (pw & 1) != 0;
    const uint32_t my_parity = pw >> 1;
    if (leader) {
      for (int v = 0; v < kMaxViews; ++v) tma_prefetch_desc(&p.views[v]);
      tma_prefetch_desc(&p.wmap);
    }
    int stage = 0;
    uint32_t phase = 0, idx = 0;
    bool ok = true;
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int g = (t / static_cast<uint32_t>(p.tiles_co)) % static_cast<uint32_t>(p.groups);
      const uint32_t pt = t / co_groups;
      const int w0 = (pt % static_cast<uint32_t>(p.tiles_w)) * p.bw;
      const int h0 = ((pt / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h)) * p.bh;
      const int n0 = (pt / tiles_wh) * p.bn;
      for (int tap = 0; tap < p.ntaps && ok; ++tap) {
        const ConvTap tp = p.taps[tap];
        for (int kb = 0; kb < p.kblocks; ++kb, ++idx) {
          if ((idx & 1) == my_parity) {
            if (!uniform_wait(&bars->empty[stage], phase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
            uint8_t* sa = smem + stage * stage_bytes<BN>();
            if (leader) {
              if (!b_box) {
                mbar_expect_tx(&bars->full[stage], tx_bytes);
                tma_load_5d(sa, &p.views[tp.view], &bars->full[stage], kb * kBK, g, w0 + tp.dw,
                            h0 + tp.dh, n0);
              } else {
                tma_load_3d(sa + kABytes, &p.wmap, &bars->full[stage], kb * kBK, co_t * BN,
                            tp.wmat * p.groups + g);
              }
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else if (warp == 1) {
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int it = 0;
    const uint64_t desc_bits = smem_desc(0, 16, 1024);
    const uint32_t desc_hi = static_cast<uint32_t>(desc_bits >> 32);
    const uint32_t lo_base = static_cast<uint32_t>(desc_bits) + (smem_u32(smem) >> 4);
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      if (!uniform_wait(&bars->acc_empty[buf], aphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem + buf * BN;
      for (int k = 0; k < kiters; ++k) {
        if (!uniform_wait(&bars->full[stage], phase, bars, p.wait_clocks)) { ok = false; break; }
        tc_fence_after();
        // 8 tf32 / 16 f16 channels = 32 bytes along the swizzled row per MMA: only the address
        // field of the descriptors changes (by 2 units of 16 bytes)
        const uint32_t a_lo = lo_base + stage * (stage_bytes<BN>() >> 4);
        const uint32_t b_lo = a_lo + (kABytes >> 4);
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_words<KIND>(d_tmem, a_lo + 2 * kk, b_lo + 2 * kk, desc_hi, kIdesc, (k | kk) != 0);
          umma_commit(&bars->empty[stage]);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (ok && leader) umma_commit(&bars->acc_full[buf]);
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else {
    // Epilogue, 16 warps: warp w reads TMEM lanes [32*(w%4), +32) (the hardware's rule) and, of
    // those rows, every fourth 32-column chunk.  One warp keeps only a few stores in flight, so
    // the SM's store bandwidth is reached through the number of warps.
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int rw = row % p.bw, rh = (row / p.bw) % p.bh, rn = row / (p.bw * p.bh);
    OutT* out = static_cast<OutT*>(p.out);
    const bool rowwise = p.out_sc == 1 && ((p.n_out * sizeof(OutT)) & 15) == 0;
    bool ok = true;
    int it = 0;
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int g = (t / static_cast<uint32_t>(p.tiles_co)) % static_cast<uint32_t>(p.groups);
      const uint32_t pt = t / co_groups;
      const int w = (pt % static_cast<uint32_t>(p.tiles_w)) * p.bw + rw;
      const int h = ((pt / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h)) * p.bh + rh;
      const int n = (pt / tiles_wh) * p.bn + rn;
      const bool valid = row < rows_used && w < p.Wt && h < p.Ht && n < p.Nimg;
      if (!warp_wait_or_abort(&bars->acc_full[buf], aphase, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      OutT* pix = out + (p.out_off + n * p.out_sn + h * p.out_sh + w * p.out_sw) + 1LL * g * p.n_out * p.out_sc;
      const OutT* res = p.epi.residual ? static_cast<const OutT*>(p.epi.residual) + (pix - out) : nullptr;
      const int co_base = co_t * BN;
#pragma unroll 1
      for (int ch = sub; ch < BN / 32; ch += kEpilogueWarps / 4) {
        const int co0 = co_base + ch * 32;          // first channel (within the group) of the chunk
        if (co0 >= p.n_out) break;
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN + ch * 32, r);
        tmem_ld_wait();
        if (!valid) continue;
        const float* bias = p.bias ? p.bias + g * p.n_out + co0 : nullptr;
        if (rowwise) {   // n_out is a whole number of 16-byte pieces: a piece is all in or all out
#pragma unroll
          for (int j = 0; j < 32; j += 16 / sizeof(OutT)) {
            if (co0 + j >= p.n_out) break;
            float f[16 / sizeof(OutT)];
#pragma unroll
            for (int q = 0; q < 16 / (int)sizeof(OutT); ++q) {
              f[q] = p.epi.alpha * __uint_as_float(r[j + q]);
              if (bias) f[q] += bias[j + q];
              if (res) f[q] += p.epi.beta * static_cast<float>(res[co0 + j + q]);
              if (p.relu) f[q] = p.epi.lin * f[q] + p.epi.abs * fabsf(f[q]);
            }
            if (!B200_IN_RANGE((pix - out) + co0 + j >= 0 && (pix - out) + co0 + j + 16 / (long long)sizeof(OutT) <= p.out_elems, p.status))
              continue;
            if (sizeof(OutT) == 4) {
              *reinterpret_cast<float4*>(pix + co0 + j) = make_float4(f[0], f[1], f[2], f[3]);
            } else {
              uint4 pk;
              uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __half2 h2 = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
                pw[q] = *reinterpret_cast<uint32_t*>(&h2);
              }
              *reinterpret_cast<uint4*>(pix + co0 + j) = pk;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (co0 + j < p.n_out) {
              float v = p.epi.alpha * __uint_as_float(r[j]);
              if (bias) v += bias[j];
              if (res) v += p.epi.beta * static_cast<float>(res[(co0 + j) * p.out_sc]);
              if (p.relu) v = p.epi.lin * v + p.epi.abs * fabsf(v);
              if (B200_IN_RANGE((pix - out) + (co0 + j) * p.out_sc >= 0 && (pix - out) + (co0 + j) * p.out_sc < p.out_elems, p.status))
                OutPack<OutT>::store(pix + (co0 + j) * p.out_sc, v);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusTimeout);
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort) abort_grace(p.wait_clocks);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <MmaKind KIND, int BN>
cudaError_t launch_one(const UmmaConvParams& p, long long total, int num_sms, cudaStream_t s) {
  constexpr int smem = num_stages<BN>() * stage_bytes<BN>() + sizeof(Bars) + 1024;
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] { return cudaFuncSetAttribute(conv_umma_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (e != cudaSuccess) return e;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  conv_umma_kernel<KIND, BN><<<grid, kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

// Accumulator width: the smallest of 32/64/128/256 columns that holds the group's outputs.
int conv_umma_bn(int n_out) { return n_out <= 32 ? 32 : n_out <= 64 ? 64 : n_out <= 128 ? 128 : 256; }

cudaError_t launch_conv_umma(const UmmaConvParams& p, int dtype, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.tiles_w * p.tiles_h * p.tiles_n * p.groups * p.tiles_co;
  if (total == 0 || p.ntaps == 0) return cudaSuccess;
  if (total >= (1LL << 31)) return cudaErrorInvalidValue;
  const int bn = conv_umma_bn(p.n_out);
  const bool f16 = dtype == B200CONV_F16;
#define B200_CASE(BNV)                                                                  \
  case BNV:                                                                             \
    return f16 ? launch_one<MmaKind::F16, BNV>(p, total, num_sms, s)                    \
               : launch_one<MmaKind::TF32, BNV>(p, total, num_sms, s);
  switch (bn) {
    B200_CASE(32)
    B200_CASE(64)
    B200_CASE(128)
    B200_CASE(256)
  }
#undef B200_CASE
  return cudaErrorInvalidValue;
}

}  // namespace b200
