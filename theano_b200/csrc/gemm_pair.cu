// 1x1 convolutions (flattened to one row of pixels) on pairs of CTAs: tcgen05.mma.cta_group::2.
//
//   out[pixel, co] = sum over channels c of  x[pixel, c] * filt[co, c]
//
// With one 128 x 256 accumulator per CTA, every 64-channel block of the reduction costs a CTA 16 KB of
// activations and 32 KB of filters from L2 for 512 clocks of MMAs: 96 B/clk, where an SM gets 73.  Here two
// CTAs of a cluster (two neighbouring SMs) compute a 256 x 256 tile together: each loads its own 128
// pixels and HALF of the filter tile (128 filters) with plain TMA loads into its own shared memory, one
// thread of the even CTA issues MMAs of M = 256 that read both CTAs' operands, and each CTA's TMEM
// receives its own 128 accumulator rows.  Per CTA that is 32 KB per 512 clocks: 64 B/clk.
// No load is multicast: every CTA fetches exactly what lands in its own shared memory.
//
// Roles per CTA (608 threads): warp 0 TMA producer, warp 1 TMEM owner and (even CTA only) MMA issuer,
// 16 epilogue warps (TMEM -> registers -> scale / bias / activation -> staged TMA stores), as in the
// slab kernel.  Barriers live at the same offsets in both CTAs; "full" and "accumulator free" are
// waited on in the even CTA only and are signalled there by both CTAs.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 32 * (2 + kEpilogueWarps + 1);     // the last warp idles: same launch shape as the slab kernel
constexpr int kBN = 256;                                      // filters per pair tile (128 per CTA's filter half)
constexpr int kABytes = 128 * 128, kBBytes = 128 * 128;       // per stage and CTA: 128 pixels / 128 filters x 64 channels
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kMaxStages = 5;
constexpr int kStoreBytes = 128 * 128;                        // one staged 64-channel chunk of the CTA's 128 pixels

struct alignas(16) Bars {
  uint64_t full[kMaxStages];        // even CTA: both CTAs' loads of a stage have landed (expect_tx by its producer)
  uint64_t empty[kMaxStages];       // each CTA: the MMAs that read the stage are done (commit from the even CTA)
  uint64_t acc_full[2];             // each CTA: the tile's accumulator is complete
  uint64_t acc_empty[2];            // even CTA: both CTAs' epilogues have read the accumulator
  uint32_t tmem_base;
  volatile int abort;
};

template <typename T> __device__ __forceinline__ void unused(const T&) {}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ PairGemmParams p) {
  constexpr uint32_t kIdesc = instr_desc(false, false, false, 256, kBN);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + p.stages * kStageBytes;
  Bars* bars = reinterpret_cast<Bars*>(staging + 4 * kStoreBytes);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                       // 0: even CTA (issues the MMAs)
  const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const uint32_t total = static_cast<uint32_t>(p.tiles_pix) * p.tiles_co;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2);                         // one arrival per CTA of the pair
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {                                               // the same warp in both CTAs
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                            // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&p.view);
      tma_prefetch_desc(&p.wmap);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t t = pair; t < total && ok; t += npairs) {
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int pix0 = (t / static_cast<uint32_t>(p.tiles_co)) * 256 + rank * 128;
      for (int kb = 0; kb < p.kblocks; ++kb) {
        if (!uniform_wait(&bars->empty[stage], phase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        uint8_t* sa = smem + stage * kStageBytes;
        if (leader) {
          if (rank == 0) mbar_expect_tx(&bars->full[stage], 2 * kStageBytes);      // both CTAs' bytes
          tma_load_5d_pair(sa, &p.view, &bars->full[stage], kb * 64, 0, pix0, 0, 0);
          tma_load_3d_pair(sa + kABytes, &p.wmap, &bars->full[stage], kb * 64, co_t * kBN + rank * 128, 0);
        }
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else if (warp == 1) {
    if (rank == 0) {
      const bool leader = elect_one();
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t desc_bits = smem_desc(0, 16, 1024);
      const uint32_t desc_hi = static_cast<uint32_t>(desc_bits >> 32);
      const uint32_t lo_base = static_cast<uint32_t>(desc_bits) + (smem_u32(smem) >> 4);
      for (uint32_t t = pair; t < total && ok; t += npairs, ++it) {
        const int buf = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!uniform_wait(&bars->acc_empty[buf], aphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + buf * kBN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!uniform_wait(&bars->full[stage], phase, bars, p.wait_clocks)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = lo_base + stage * (kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (kABytes >> 4);
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_words_pair_f16(d_tmem, a_lo + 2 * kk, b_lo + 2 * kk, desc_hi, kIdesc, (kb | kk) != 0);
            umma_commit_pair(&bars->empty[stage]);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (ok && leader) umma_commit_pair(&bars->acc_full[buf]);
      }
      if (!ok && leader) atomicExch(p.status, kStatusTimeout);
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // Epilogue: warp w reads TMEM lanes [32 * (w % 4), +32) of this CTA's 128 accumulator rows; the four
    // groups of four warps take one 64-channel chunk each, stage it (swizzled like the store map expects)
    // and one thread per group stores the box.  A group waits for its staging buffer only before refilling it.
    const int quad = warp & 3, grp = (warp - 2) >> 2;
    const int drow = quad * 32 + lane;                              // this lane's pixel of the CTA's 128
    const bool issuer = quad == 0 && lane == 0;
    const bool plain = p.epi.alpha == 1.f && !p.bias && !p.relu;
    uint8_t* stg = staging + grp * kStoreBytes;
    uint8_t* srow = stg + drow * 128;
    bool ok = true;
    int it = 0, nstore = 0;
    for (uint32_t t = pair; t < total && ok; t += npairs, ++it) {
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int pix0 = (t / static_cast<uint32_t>(p.tiles_co)) * 256 + rank * 128;
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      if (!warp_wait_or_abort(&bars->acc_full[buf], aphase, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const int co_base = co_t * kBN;
      const int nstaged = min(kBN / 64, (p.n_out - co_base + 63) / 64);
      const uint32_t lane_base = tmem + buf * kBN + (static_cast<uint32_t>(quad * 32) << 16);
      if (grp < nstaged) {
        const int co0 = co_base + grp * 64;
        const float* bias = p.bias ? p.bias + co0 : nullptr;
        if (nstore > 0) {                                            // the buffer's previous box must have been read
          if (issuer) bulk_wait_read<0>();
          named_barrier(1 + grp, 128);
        }
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t r[32];
          tmem_ld32(lane_base + grp * 64 + part * 32, r);
          tmem_ld_wait();
          const float* bp = bias ? bias + part * 32 : nullptr;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t h[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float f0 = __uint_as_float(r[8 * j + 2 * q]), f1 = __uint_as_float(r[8 * j + 2 * q + 1]);
              if (!plain) {
                f0 *= p.epi.alpha; f1 *= p.epi.alpha;
                if (bp) { f0 += bp[8 * j + 2 * q]; f1 += bp[8 * j + 2 * q + 1]; }
                if (p.relu) {
                  f0 = p.epi.lin * f0 + p.epi.abs * fabsf(f0);
                  f1 = p.epi.lin * f1 + p.epi.abs * fabsf(f1);
                }
              }
              __half2 h2 = __floats2half2_rn(f0, f1);
              h[q] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(srow + (((part * 4 + j) ^ (drow & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
          }
        }
        fence_async_smem();
        named_barrier(1 + grp, 128);
        if (issuer && B200_IN_RANGE(co0 >= 0 && pix0 >= 0 && pix0 < p.pixels, p.status)) {
          tma_store_4d(&p.out_map, stg, co0, pix0, 0, 0);
          bulk_commit();
        }
        ++nstore;
      }
      // every epilogue warp of this CTA has read its part of the accumulator: one arrival per CTA on the
      // even CTA's barrier hands the accumulator back to the MMA thread
      tc_fence_before();
      named_barrier(5, 32 * kEpilogueWarps);
      if (warp == 2 && lane == 0) mbar_arrive_leader(&bars->acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusTimeout);
    if (lane == 0) bulk_wait<0>();           // this thread's stores (if it issued any) have left shared memory
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

int gemm_pair_smem_bytes(int stages) { return stages * kStageBytes + 4 * kStoreBytes + (int)sizeof(Bars) + 1024; }

cudaError_t launch_gemm_pair(const PairGemmParams& p, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.tiles_pix * p.tiles_co;
  if (total == 0 || p.kblocks == 0) return cudaSuccess;
  if (total >= (1LL << 31) || p.stages < 2 || p.stages > kMaxStages) return cudaErrorInvalidValue;
  const int smem = gemm_pair_smem_bytes(p.stages);
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] {
    return cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  });
  if (e != cudaSuccess) return e;
  long long pairs = std::min<long long>(total, num_sms / 2);
  gemm_pair_kernel<<<static_cast<int>(2 * pairs), kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace b200
