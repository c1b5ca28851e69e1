// Filter gradient on pairs of CTAs (tcgen05.mma.cta_group::2), float16, layers with at least 256
// filters and 256 channels per group.
//
//   dW[tap][k, c] = sum over output pixels q of  dy[q, k] * x_view_tap[q + offset_tap, c]
//
// One CTA with a 128 x 256 accumulator needs, per stage of 64 pixels, 16 KB of dy and 32 KB of x from
// L2 for 512 clocks of MMAs: 94 B/clk where an SM gets 73.  Here two CTAs of a cluster compute a tile of
// 256 filters x 256 channels together: each loads the dy rows of ITS 128 filters and HALF of the x tile
// (128 channels) into its own shared memory with plain TMA loads, one thread of the even CTA issues MMAs
// of M = 256 over both CTAs' operands, and each CTA's TMEM receives its 128 filter rows x 256 channels.
// Per CTA that is 32 KB per 512 clocks: 64 B/clk.  No load is shared between CTAs by the copy engine.
//
// Work items, split-K slices, slab layout and the reduction kernel are those of wgrad_umma.cu; an item is
// (256-filter tile, 256-channel tile, group, tap, slice) and both CTAs of a pair walk the same items.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 32 * (2 + kEpilogueWarps);
constexpr int kPix = kWgradPixF16Wide;                 // reduction rows (pixels) per stage: 64
constexpr int kBoxBytes = kPix * 128;                  // one TMA box: 64 pixels x 64 channels of float16
constexpr int kBoxes = 4;                              // per CTA and stage: 2 of dy (128 filters), 2 of x (128 channels)
constexpr int kStageBytes = kBoxes * kBoxBytes;        // 32 KB
constexpr int kStages = 6;
constexpr int kBN = 256;

struct alignas(16) Bars {
  uint64_t full[kStages];        // even CTA: both CTAs' boxes of a stage have landed
  uint64_t empty[kStages];       // each CTA: the MMAs reading the stage are done
  uint64_t acc_full[2];          // each CTA: the item's accumulator is complete
  uint64_t acc_empty[2];         // even CTA: both CTAs' epilogues have read the accumulator
  uint32_t tmem_base;
  volatile int abort;
};

struct Item {
  int kt, ct, g, tap, sp;
  uint32_t t_begin, t_end;
};

__device__ __forceinline__ Item decode(uint32_t it, const UmmaWgradParams& p, uint32_t per_split, uint32_t pix_tiles) {
  Item r;
  r.sp = it % static_cast<uint32_t>(p.splits);
  it /= static_cast<uint32_t>(p.splits);
  r.tap = it % static_cast<uint32_t>(p.ntaps);
  it /= static_cast<uint32_t>(p.ntaps);
  r.g = it % static_cast<uint32_t>(p.groups);
  it /= static_cast<uint32_t>(p.groups);
  r.ct = it % static_cast<uint32_t>(p.ctiles);
  r.kt = it / static_cast<uint32_t>(p.ctiles);
  r.t_begin = r.sp * per_split;
  r.t_end = r.t_begin + per_split < pix_tiles ? r.t_begin + per_split : pix_tiles;
  return r;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
wgrad_pair_kernel(const __grid_constant__ UmmaWgradParams p) {
  constexpr int kK = 16;                                           // reduction rows per MMA
  constexpr uint32_t kStep = (kK * 128) >> 4;
  constexpr uint32_t kIdesc = instr_desc(false, true, true, 256, kBN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * kStageBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int rows_used = p.bw * p.bh * p.bn;
  const int ksteps = (rows_used + kK - 1) / kK;
  const uint32_t pix_tiles = static_cast<uint32_t>(p.tiles_w) * p.tiles_h * p.tiles_n;
  const uint32_t per_split = (pix_tiles + p.splits - 1) / p.splits;
  const uint32_t total = static_cast<uint32_t>(p.ktiles) * p.ctiles * p.groups * p.ntaps * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2);                           // one arrival per CTA of the pair
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  // Reduction rows past the pixel box are never written by TMA: clear them once so that the last MMA
  // of a stage (which reads whole groups of 16 rows) adds zeros.
  if (rows_used < ksteps * kK) {
    const int tail_rows = ksteps * kK - rows_used;
    const int boxes = kStages * kBoxes;
    for (int i = threadIdx.x; i < boxes * tail_rows * 8; i += kThreads) {
      const int box = i / (tail_rows * 8), rem = i % (tail_rows * 8);
      *(reinterpret_cast<uint4*>(smem + box * kBoxBytes + (rows_used + rem / 8) * 128) + rem % 8) = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                              // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    const bool leader = elect_one();
    if (leader) {
      for (int v = 0; v < kMaxViews; ++v) tma_prefetch_desc(&p.x_views[v]);
      tma_prefetch_desc(&p.dy_map);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t tx = 2u * kBoxes * rows_used * 128;            // both CTAs' boxes (out-of-range parts arrive as zeros)
    for (uint32_t it = pair; it < total && ok; it += npairs) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const ConvTap tp = p.taps[w.tap];
      const int k0 = w.kt * 256 + rank * 128, c0 = w.ct * kBN + rank * 128;
      int tw = static_cast<int>(w.t_begin % static_cast<uint32_t>(p.tiles_w));
      int th_ = static_cast<int>((w.t_begin / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h));
      int tn = static_cast<int>(w.t_begin / (static_cast<uint32_t>(p.tiles_w) * p.tiles_h));
      for (uint32_t t = w.t_begin; t < w.t_end; ++t) {
        const int w0 = tw * p.bw, h0 = th_ * p.bh, n0 = tn * p.bn;
        if (++tw == p.tiles_w) {
          tw = 0;
          if (++th_ == p.tiles_h) { th_ = 0; ++tn; }
        }
        if (!uniform_wait(&bars->empty[stage], phase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        uint8_t* sa = smem + stage * kStageBytes;
        if (leader) {
          if (rank == 0) mbar_expect_tx(&bars->full[stage], tx);
          tma_load_5d_pair(sa, &p.dy_map, &bars->full[stage], k0, w.g, w0, h0, n0);
          tma_load_5d_pair(sa + kBoxBytes, &p.dy_map, &bars->full[stage], k0 + 64, w.g, w0, h0, n0);
          tma_load_5d_pair(sa + 2 * kBoxBytes, &p.x_views[tp.view], &bars->full[stage], c0, w.g, w0 + tp.dw, h0 + tp.dh, n0);
          tma_load_5d_pair(sa + 3 * kBoxBytes, &p.x_views[tp.view], &bars->full[stage], c0 + 64, w.g, w0 + tp.dw, h0 + tp.dh, n0);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else if (warp == 1) {
    if (rank == 0) {
      const bool leader = elect_one();
      int stage = 0, n = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t desc_bits = smem_desc(0, kBoxBytes, 1024, kSwizzle128);
      const uint32_t desc_hi = static_cast<uint32_t>(desc_bits >> 32);
      const uint32_t lo_base = static_cast<uint32_t>(desc_bits) + (smem_u32(smem) >> 4);
      for (uint32_t it = pair; it < total && ok; it += npairs, ++n) {
        const Item w = decode(it, p, per_split, pix_tiles);
        const int buf = n & 1;
        const uint32_t aphase = (n >> 1) & 1;
        if (!uniform_wait(&bars->acc_empty[buf], aphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * kBN;
        uint32_t acc = 0u;
        for (uint32_t t = w.t_begin; t < w.t_end; ++t) {
          if (!uniform_wait(&bars->full[stage], phase, bars, p.wait_clocks)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = lo_base + stage * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + ((2 * kBoxBytes) >> 4);
          if (leader) {
            for (int ks = 0; ks < ksteps; ++ks)
              umma_words_pair_f16(d_tmem, a_lo + ks * kStep, b_lo + ks * kStep, desc_hi, kIdesc, ks == 0 ? acc : 1u);
            umma_commit_pair(&bars->empty[stage]);
          }
          acc = 1u;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok && leader) umma_commit_pair(&bars->acc_full[buf]);
      }
      if (!ok && leader) atomicExch(p.status, kStatusTimeout);
    }
  } else {
    // Epilogue, 16 warps: warp w reads TMEM lanes [32 * (w % 4), +32) = 32 of this CTA's 128 filter rows and,
    // of those, every fourth 32-column chunk; rows go to the item's slab [slice][tap][K][C/g].
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    bool ok = true;
    int n = 0;
    const int K = p.Kg * p.groups;
    for (uint32_t it = pair; it < total && ok; it += npairs, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int buf = n & 1;
      const uint32_t aphase = (n >> 1) & 1;
      if (!warp_wait_or_abort(&bars->acc_full[buf], aphase, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const int kq = w.kt * 256 + static_cast<int>(rank) * 128 + row;
      const bool valid = kq < p.Kg;
      const int slab = p.atomic ? 0 : w.sp;
      float* dst = p.partial + ((1LL * slab * p.taps_total + p.taps[w.tap].wmat) * K + w.g * p.Kg + kq) * p.Cg;
      const bool vec = (p.Cg & 3) == 0 && !p.atomic;
#pragma unroll 1
      for (int ch = sub; ch < kBN / 32; ch += kEpilogueWarps / 4) {
        const int c0 = w.ct * kBN + ch * 32;
        if (c0 >= p.Cg) break;
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + buf * kBN + ch * 32, r);
        tmem_ld_wait();
        if (valid) {
          if (vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (c0 + j < p.Cg && B200_IN_RANGE((dst - p.partial) + c0 + j >= 0 && (dst - p.partial) + c0 + j + 4 <= p.partial_elems, p.status))
                *reinterpret_cast<float4*>(dst + c0 + j) =
                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c0 + j < p.Cg && B200_IN_RANGE((dst - p.partial) + c0 + j >= 0 && (dst - p.partial) + c0 + j < p.partial_elems, p.status)) {
                if (p.atomic) atomicAdd(dst + c0 + j, __uint_as_float(r[j]));
                else dst[c0 + j] = __uint_as_float(r[j]);
              }
            }
          }
        }
      }
      // every epilogue warp of this CTA has read its part: one arrival per CTA on the even CTA's barrier
      tc_fence_before();
      named_barrier(5, 32 * kEpilogueWarps);
      if (warp == 2 && lane == 0) mbar_arrive_leader(&bars->acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusTimeout);
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort) abort_grace(p.wait_clocks);
  cluster_sync_all();                        // no CTA of the pair leaves (or frees TMEM) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
}

}  // namespace

cudaError_t launch_wgrad_pair(const UmmaWgradParams& p, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.ktiles * p.ctiles * p.groups * p.ntaps * p.splits;
  if (total == 0) return cudaSuccess;
  if (total >= (1LL << 31) || 1LL * p.tiles_w * p.tiles_h * p.tiles_n >= (1LL << 31) || p.bw * p.bh * p.bn > kPix)
    return cudaErrorInvalidValue;
  constexpr int smem = kStages * kStageBytes + sizeof(Bars) + 1024;
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] {
    return cudaFuncSetAttribute(wgrad_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (e != cudaSuccess) return e;
  const long long pairs = std::min<long long>(total, num_sms / 2);
  wgrad_pair_kernel<<<static_cast<int>(2 * pairs), kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace b200
