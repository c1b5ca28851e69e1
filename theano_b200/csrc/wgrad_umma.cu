// Filter gradient as an implicit GEMM on tcgen05 tensor cores.
//
//   dW[tap][k, c] = sum over output pixels q of  dy[q, k] * x_view_tap[q + offset_tap, c]
//
// Both operands are channels-last, so the reduction index (the pixel) is the slow index of
// each shared-memory row and the M/N index (filter k, channel c) is the contiguous one: the
// MMA reads both operands in MN-major form with a 128-byte swizzle (16-byte chunks for
// float16; 32-byte chunks for tf32, the only swizzled MN-major form tf32 has).  One TMA box brings
// kAtom (32 float32 / 64 float16) channels of up to 64 pixels; an operand of 128 filters or
// BN channels is a row of such boxes (leading-dimension offset = one box).
//
// Warp roles: warp 0 and the last three warps TMA producers, warp 1 MMA issuer and TMEM owner,
// 16 epilogue warps.
// Work item = (filter tile, channel tile, group, tap, split-K slice).  Each item reduces its
// slice of the pixel tiles into a TMEM accumulator (128 filters x BN channels, float32) and
// writes it to its own slab of the partial buffer, laid out [slice][tap][K][C/groups] so the
// stores are contiguous along c.  A second kernel adds the slabs in slice order (so the
// result does not depend on scheduling) and writes OIHW.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;            // a warp keeps only a few stores in flight: use many
// One thread gets a TMA box accepted every ~300 clocks whatever its size; the MMAs of a stage
// take less than the stage's 6-12 boxes would need from one thread.  Boxes are therefore spread
// over several producer warps (warp 0 and the warps after the epilogue warps) and over lanes
// within them: box j of a stage belongs to producer warp j % kProducers, lane j / kProducers.
constexpr int kProducers = 4;
constexpr int kFirstExtraProducer = 2 + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstExtraProducer + kProducers - 1);
// one TMA box in shared memory: the stage's reduction rows x 128 bytes
template <MmaKind KIND, int BN> constexpr int box_bytes() {
  return (KIND == MmaKind::TF32 ? kWgradPixF32 : BN >= 256 ? kWgradPixF16Wide : kWgradPixF16) * 128;
}
constexpr int kSmemBudget = 208 * 1024;

template <MmaKind KIND> constexpr int atom() { return KIND == MmaKind::TF32 ? 32 : 64; }
template <MmaKind KIND, int BN> constexpr int stage_bytes() {
  return (128 / atom<KIND>() + BN / atom<KIND>()) * box_bytes<KIND, BN>();
}
template <MmaKind KIND, int BN> constexpr int num_stages() {
  return (kSmemBudget / stage_bytes<KIND, BN>()) > 8 ? 8 : (kSmemBudget / stage_bytes<KIND, BN>());
}

struct Bars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

struct Item {
  int kt, ct, g, tap, sp;
  uint32_t t_begin, t_end;  // pixel-tile range of the split
};

// 32-bit arithmetic throughout (the launcher checks the counts): 64-bit divisions cost a role
// about a hundred clocks each
__device__ __forceinline__ Item decode(uint32_t it, const UmmaWgradParams& p, uint32_t per_split,
                                       uint32_t pix_tiles) {
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

// The MMA issuer's loop over the pixel tiles (pipeline stages) of one work item.  KS > 0: exactly KS
// reduction steps per stage, issued as straight-line code; KS == 0: `ksteps` steps in blocks of four.
// f16: 8-row groups 1024 bytes apart, 16-byte swizzle; tf32: 4-row groups 512 bytes apart, 32-byte
// swizzle; leading offset = next box (next kAtom channels).  Only the address field of the two
// descriptors changes from one MMA to the next: kK rows further.  Returns false when a wait ran out.
template <MmaKind KIND, int BN, int KS, bool TIMED>
__device__ __forceinline__ bool mma_tiles(Bars* bars, uint32_t d_tmem, uint32_t lo_base, uint32_t desc_hi,
                                          int ksteps, int ntiles, int& stage, uint32_t& phase,
                                          long long& t_wait, bool leader, long long limit) {
  constexpr int kAtom = atom<KIND>();
  constexpr int kABoxes = 128 / kAtom;
  constexpr int kStages = num_stages<KIND, BN>();
  constexpr int kK = KIND == MmaKind::TF32 ? 8 : 16;
  constexpr uint32_t kStep = (kK * 128) >> 4;
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, true, true, 128, BN);
  uint32_t acc = 0u;
  for (int t = 0; t < ntiles; ++t) {
    if (TIMED) {
      const long long tw = clock64();
      if (!uniform_wait(&bars->full[stage], phase, bars, limit)) return false;
      t_wait += clock64() - tw;
    } else if (!uniform_wait(&bars->full[stage], phase, bars, limit)) {
      return false;
    }
    tc_fence_after();
    const uint32_t a_lo = lo_base + stage * (stage_bytes<KIND, BN>() >> 4);
    const uint32_t b_lo = a_lo + ((kABoxes * box_bytes<KIND, BN>()) >> 4);
    if (leader) {
      if (KS > 0) {
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          umma_words<KIND>(d_tmem, a_lo + ks * kStep, b_lo + ks * kStep, desc_hi, kIdesc, ks == 0 ? acc : 1u);
      } else {
        for (int ks = 0; ks < ksteps; ++ks)
          umma_words<KIND>(d_tmem, a_lo + ks * kStep, b_lo + ks * kStep, desc_hi, kIdesc, ks == 0 ? acc : 1u);
      }
      umma_commit(&bars->empty[stage]);
    }
    acc = 1u;
    const int next = stage + 1;
    const bool wrap = next == kStages;
    stage = wrap ? 0 : next;
    phase ^= wrap ? 1u : 0u;
  }
  return true;
}

template <MmaKind KIND, int BN>
__global__ void __launch_bounds__(kThreads, 1)
wgrad_umma_kernel(const __grid_constant__ UmmaWgradParams p) {
  constexpr int kAtom = atom<KIND>();
  constexpr int kABoxes = 128 / kAtom, kBBoxes = BN / kAtom;
  constexpr int kStages = num_stages<KIND, BN>();
  constexpr int kBoxBytes = box_bytes<KIND, BN>();
  constexpr int kK = KIND == MmaKind::TF32 ? 8 : 16;       // reduction rows per MMA
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, true, true, 128, BN);
  constexpr uint32_t kSbo = KIND == MmaKind::TF32 ? 512 : 1024;
  constexpr uint64_t kLayout = KIND == MmaKind::TF32 ? kSwizzle128Base32 : kSwizzle128;
  constexpr bool kDouble = 2 * BN <= 512;
  constexpr uint32_t kTmemCols = 2 * BN > 512 ? 512 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * stage_bytes<KIND, BN>());

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  // phase timing (optional): [0] MMA thread waiting for operands, [1] its whole loop,
  // [2] first producer waiting for a free stage, [3] its whole loop, [4] kernel start to end,
  // [9] / [10] GPU-wide timer at start / end
  long long* trace = p.trace ? p.trace + blockIdx.x * 16 : nullptr;
  const long long t_begin = trace ? clock64() : 0;
  if (trace && threadIdx.x == 0) trace[9] = static_cast<long long>(global_ns());
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
      mbar_init(&bars->acc_empty[b], 32 * kEpilogueWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Reduction rows past the pixel box are never written by TMA: clear them once so that the
  // last MMA of a stage (which reads whole groups of kK rows) adds zeros.
  if (rows_used < ksteps * kK) {
    const int tail_rows = ksteps * kK - rows_used;
    const int boxes = kStages * (kABoxes + kBBoxes);
    for (int i = threadIdx.x; i < boxes * tail_rows * 8; i += kThreads) {
      const int box = i / (tail_rows * 8), rem = i % (tail_rows * 8);
      uint4* dst = reinterpret_cast<uint4*>(smem + box * kBoxBytes + (rows_used + rem / 8) * 128) + rem % 8;
      *dst = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0 || warp >= kFirstExtraProducer) {
    const int pw = warp == 0 ? 0 : warp - kFirstExtraProducer + 1;
    if (lane == 0) {
      for (int v = 0; v < kMaxViews; ++v) tma_prefetch_desc(&p.x_views[v]);
      tma_prefetch_desc(&p.dy_map);
    }
    // every lane follows the loop (warp-uniform control flow and addresses); one elected lane issues
    // this warp's boxes of a stage: pw, pw + kProducers, ...
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long t_wait = 0;
    for (uint32_t it = blockIdx.x; it < total && ok; it += gridDim.x) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const ConvTap tp = p.taps[w.tap];
      // boxes that lie wholly past the channel counts are skipped (their accumulator rows /
      // columns are never stored)
      const int a_boxes = min(kABoxes, (p.Kg - w.kt * 128 + kAtom - 1) / kAtom);
      const int b_boxes = min(kBBoxes, (p.Cg - w.ct * BN + kAtom - 1) / kAtom);
      const uint32_t tx = (a_boxes + b_boxes) * rows_used * 128;
      // tile coordinates advance by counting: 64-bit divisions per stage would cost the producers
      // more clocks than the stage's MMAs take
      int tw = static_cast<int>(w.t_begin % static_cast<uint32_t>(p.tiles_w));
      int th_ = static_cast<int>((w.t_begin / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h));
      int tn = static_cast<int>(w.t_begin / (static_cast<uint32_t>(p.tiles_w) * p.tiles_h));
      for (uint32_t t = w.t_begin; t < w.t_end; ++t) {
        const int w0 = tw * p.bw, h0 = th_ * p.bh, n0 = tn * p.bn;
        if (++tw == p.tiles_w) {
          tw = 0;
          if (++th_ == p.tiles_h) { th_ = 0; ++tn; }
        }
        const long long tw0 = trace ? clock64() : 0;
        if (!uniform_wait(&bars->empty[stage], phase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        if (trace) t_wait += clock64() - tw0;
        uint8_t* sa = smem + stage * stage_bytes<KIND, BN>();
        uint8_t* sb = sa + kABoxes * kBoxBytes;
        if (leader) {
          if (pw == 0) mbar_expect_tx(&bars->full[stage], tx);
          for (int j = pw; j < a_boxes + b_boxes; j += kProducers) {
            if (j < a_boxes)
              tma_load_5d(sa + j * kBoxBytes, &p.dy_map, &bars->full[stage], w.kt * 128 + j * kAtom, w.g,
                          w0, h0, n0);
            else
              tma_load_5d(sb + (j - a_boxes) * kBoxBytes, &p.x_views[tp.view], &bars->full[stage],
                          w.ct * BN + (j - a_boxes) * kAtom, w.g, w0 + tp.dw, h0 + tp.dh, n0);
          }
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
    if (trace && leader && pw == 0) { trace[2] = t_wait; trace[3] = clock64() - t_begin; }
  } else if (warp == 1) {
    // all lanes follow the loop and wait; one elected lane issues the MMAs and their commits
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int n = 0;
    long long t_wait = 0;
    const uint64_t desc_bits = smem_desc(0, kBoxBytes, kSbo, kLayout);
    const uint32_t desc_hi = static_cast<uint32_t>(desc_bits >> 32);
    const uint32_t lo_base = static_cast<uint32_t>(desc_bits) + (smem_u32(smem) >> 4);
    for (uint32_t it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int buf = kDouble ? (n & 1) : 0;
      const uint32_t aphase = kDouble ? ((n >> 1) & 1) : (n & 1);
      if (!uniform_wait(&bars->acc_empty[buf], aphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem + buf * BN;
      const int ntiles = static_cast<int>(w.t_end - w.t_begin);
      // the usual step counts get straight-line MMA blocks
      if (trace) ok = mma_tiles<KIND, BN, 0, true>(bars, d_tmem, lo_base, desc_hi, ksteps, ntiles, stage, phase, t_wait, leader, p.wait_clocks);
      else if (ksteps == 8) ok = mma_tiles<KIND, BN, 8, false>(bars, d_tmem, lo_base, desc_hi, ksteps, ntiles, stage, phase, t_wait, leader, p.wait_clocks);
      else if (ksteps == 7) ok = mma_tiles<KIND, BN, 7, false>(bars, d_tmem, lo_base, desc_hi, ksteps, ntiles, stage, phase, t_wait, leader, p.wait_clocks);
      else if (ksteps == 4) ok = mma_tiles<KIND, BN, 4, false>(bars, d_tmem, lo_base, desc_hi, ksteps, ntiles, stage, phase, t_wait, leader, p.wait_clocks);
      else ok = mma_tiles<KIND, BN, 0, false>(bars, d_tmem, lo_base, desc_hi, ksteps, ntiles, stage, phase, t_wait, leader, p.wait_clocks);
      if (ok && leader) umma_commit(&bars->acc_full[buf]);
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
    if (trace && leader) { trace[0] = t_wait; trace[1] = clock64() - t_begin; }
  } else {
    // warp w reads TMEM lanes [32*(w%4), +32) and every fourth 32-column chunk of them
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    bool ok = true;
    int n = 0;
    const int K = p.Kg * p.groups;
    for (uint32_t it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int buf = kDouble ? (n & 1) : 0;
      const uint32_t aphase = kDouble ? ((n >> 1) & 1) : (n & 1);
      if (!warp_wait_or_abort(&bars->acc_full[buf], aphase, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const int kq = w.kt * 128 + row;
      const bool valid = kq < p.Kg;
      const int slab = p.atomic ? 0 : w.sp;
      float* dst = p.partial +
                   ((1LL * slab * p.taps_total + p.taps[w.tap].wmat) * K + w.g * p.Kg + kq) * p.Cg;
      const bool vec = (p.Cg & 3) == 0 && !p.atomic;
#pragma unroll 1
      for (int ch = sub; ch < BN / 32; ch += kEpilogueWarps / 4) {
        const int c0 = w.ct * BN + ch * 32;
        if (c0 >= p.Cg) break;
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN + ch * 32, r);
        tmem_ld_wait();
        if (valid) {
          if (vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (c0 + j < p.Cg && B200_IN_RANGE((dst - p.partial) + c0 + j >= 0 && (dst - p.partial) + c0 + j + 4 <= p.partial_elems, p.status))
                *reinterpret_cast<float4*>(dst + c0 + j) =
                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
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
      tc_fence_before();
      mbar_arrive(&bars->acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusTimeout);
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort) abort_grace(p.wait_clocks);
  if (trace && threadIdx.x == 0) {
    trace[4] = clock64() - t_begin;
    trace[10] = static_cast<long long>(global_ns());
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// out[k][c][tap] = sum_s partial[s][tap][k][c].  A block takes kReduceElems consecutive (k, c)
// elements and all taps.  Its 256 threads are 32 groups of four elements x 8 lanes over the
// slabs: lane q adds the slabs q, q + 8, ... in that order and the eight partial sums are then
// added in lane order, so the result does not depend on scheduling (it is the same on every run)
// and no thread walks more than an eighth of the slabs (a layer with few filters and channels has
// up to one slab per SM, and one thread adding 148 of them one after the other took longer than
// the gradient kernel's tail).  The sums go to shared memory in output order [element][tap] and
// leave as one contiguous run of kReduceElems * taps values.
constexpr int kReduceElems = 128;      // (k, c) elements per block tile of the reduction kernel
constexpr int kReduceLanes = 8;
template <typename T>
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float* __restrict__ partial, T* __restrict__ dw,
                                                            int splits, int taps, long long kc) {
  extern __shared__ float tile[];
  __shared__ float4 part[kReduceLanes][kReduceElems / 4];
  const long long tiles = (kc + kReduceElems - 1) / kReduceElems;
  const bool vec = (kc & 3) == 0;
  const int q = threadIdx.x >> 5, gi = threadIdx.x & 31, e = gi * 4;
  for (long long tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const long long e0 = tl * kReduceElems;
    const int ne = static_cast<int>(kc - e0 < kReduceElems ? kc - e0 : kReduceElems);
    for (int t = 0; t < taps; ++t) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < ne) {
        const float* src = partial + 1LL * t * kc + e0 + e;
        const long long slab = 1LL * taps * kc;
        if (vec) {
#pragma unroll 4
          for (int s = q; s < splits; s += kReduceLanes) {
            const float4 v = *reinterpret_cast<const float4*>(src + s * slab);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
        } else {
          for (int s = q; s < splits; s += kReduceLanes) {
            const float* ps = src + s * slab;
            acc.x += ps[0];
            if (e + 1 < ne) acc.y += ps[1];
            if (e + 2 < ne) acc.z += ps[2];
            if (e + 3 < ne) acc.w += ps[3];
          }
        }
      }
      part[q][gi] = acc;
      __syncthreads();
      if (q == 0 && e < ne) {
        float4 sum = part[0][gi];
#pragma unroll
        for (int l = 1; l < kReduceLanes; ++l) {
          const float4 v = part[l][gi];
          sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        tile[(e + 0) * taps + t] = sum.x;
        tile[(e + 1) * taps + t] = sum.y;
        tile[(e + 2) * taps + t] = sum.z;
        tile[(e + 3) * taps + t] = sum.w;
      }
      __syncthreads();
    }
    T* dst = dw + e0 * taps;
    for (int i = threadIdx.x; i < ne * taps; i += blockDim.x) dst[i] = static_cast<T>(tile[i]);
    __syncthreads();
  }
}

template <MmaKind KIND, int BN>
cudaError_t launch_one(const UmmaWgradParams& p, long long total, int num_sms, cudaStream_t s) {
  constexpr int smem = num_stages<KIND, BN>() * stage_bytes<KIND, BN>() + sizeof(Bars) + 1024;
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] { return cudaFuncSetAttribute(wgrad_umma_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (e != cudaSuccess) return e;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  wgrad_umma_kernel<KIND, BN><<<grid, kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_wgrad_umma(const UmmaWgradParams& p, int dtype, int bn_cols, int num_sms,
                              cudaStream_t s) {
  const long long total = 1LL * p.ktiles * p.ctiles * p.groups * p.ntaps * p.splits;
  if (total == 0) return cudaSuccess;
  if (total >= (1LL << 31) || 1LL * p.tiles_w * p.tiles_h * p.tiles_n >= (1LL << 31)) return cudaErrorInvalidValue;
  const bool f16 = dtype == B200CONV_F16;
#define B200_CASE(BNV)                                                                  \
  case BNV:                                                                             \
    return f16 ? launch_one<MmaKind::F16, BNV>(p, total, num_sms, s)                    \
               : launch_one<MmaKind::TF32, BNV>(p, total, num_sms, s);
  switch (bn_cols) {
    B200_CASE(64)
    B200_CASE(128)
    B200_CASE(256)
  }
#undef B200_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_wgrad_reduce(const float* partial, void* dw, int splits, int taps, int K,
                                int Cg, int dtype, cudaStream_t s) {
  const long long kc = 1LL * K * Cg;
  if (kc == 0 || taps == 0) return cudaSuccess;
  long long g = (kc + kReduceElems - 1) / kReduceElems;
  if (g > 148 * 16) g = 148 * 16;
  const size_t smem = sizeof(float) * kReduceElems * taps;
  if (dtype == B200CONV_F16)
    wgrad_reduce_kernel<__half><<<static_cast<int>(g), 256, smem, s>>>(
        partial, static_cast<__half*>(dw), splits, taps, kc);
  else
    wgrad_reduce_kernel<float><<<static_cast<int>(g), 256, smem, s>>>(
        partial, static_cast<float*>(dw), splits, taps, kc);
  return cudaGetLastError();
}

}  // namespace b200
