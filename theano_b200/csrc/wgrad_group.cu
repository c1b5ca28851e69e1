// Filter gradient on tcgen05 tensor cores with operand sharing across filter taps.
//
//   dW[tap][k, c] = sum over output pixels q of  dy[q, k] * x_view[q + (dh, dw)_tap, c]
//
// Work item = (128-filter tile, 128-channel tile, conv group, tap group, split-K slice).  A tap
// group holds up to four taps with the same view and row offset dh; their x operands are the same
// pixels shifted by dw.  The reduction pixels of a stage are a box of the output grid whose rows
// are widened by the column span of the taps (dy reads zeros there), so "shifted by dw" is a plain
// row offset into one shared-memory x tile: per stage one dy tile and one x tile are fetched and
// every tap of the group accumulates into its own 128 x 128 TMEM accumulator.  That divides the
// number of TMA boxes per MMA.  (Measured: with MN-major operands the MMAs themselves run at about
// 0.4 of their K-major rate and bound both gradWeights kernels; which of the two is faster
// depends on the layer, so the first call of a geometry times both.)
//
// Operands are MN-major (the pixel is the slow index of a channels-last row): float16 with the
// 16-byte swizzle, tf32 with the 32-byte-atom swizzle; row offsets that are not multiples of the
// swizzle period are fine because the hardware swizzles on absolute shared-memory address bits.
// Warp roles: warp 0 and the last three warps TMA producers, warp 1 MMA issuer and TMEM owner,
// 16 epilogue warps.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;
// A thread gets one TMA box accepted every ~300 clocks: the boxes of a stage are spread over
// several producer warps (warp 0 and the warps after the epilogue warps) and their lanes, box j
// to producer j % kProducers, lane j / kProducers.
constexpr int kProducers = 4;
constexpr int kFirstExtraProducer = 2 + kEpilogueWarps;
constexpr int kThreads = 32 * (kFirstExtraProducer + kProducers - 1);
constexpr int kBN = 128;                       // channels per accumulator
// box rows = the stage's pixel rows + room for the largest column offset (16); bytes are a multiple
// of the 1024-byte swizzle period
template <MmaKind KIND> constexpr int box_rows() { return (KIND == MmaKind::TF32 ? kWgradPixF32 : kWgradPixF16) + 16; }
template <MmaKind KIND> constexpr int box_bytes() { return box_rows<KIND>() * 128; }
constexpr int kSmemBudget = 208 * 1024;
constexpr int kMaxStages = 6;

template <MmaKind KIND> constexpr int atom() { return KIND == MmaKind::TF32 ? 32 : 64; }
template <MmaKind KIND> constexpr int stage_bytes() { return (128 / atom<KIND>() + kBN / atom<KIND>()) * box_bytes<KIND>(); }
template <MmaKind KIND> constexpr int num_stages() {
  return (kSmemBudget / stage_bytes<KIND>()) > kMaxStages ? kMaxStages : (kSmemBudget / stage_bytes<KIND>());
}

struct alignas(16) Bars {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  volatile int abort;
};

struct Item {
  int kt, ct, g, grp, sp;
  uint32_t t_begin, t_end;
};

// 32-bit arithmetic throughout (the launcher checks the counts): 64-bit divisions cost a role
// about a hundred clocks each
__device__ __forceinline__ Item decode(uint32_t it, const GroupWgradParams& p, uint32_t per_split,
                                       uint32_t pix_tiles) {
  Item r;
  r.sp = it % static_cast<uint32_t>(p.splits);
  it /= static_cast<uint32_t>(p.splits);
  r.grp = it % static_cast<uint32_t>(p.ngroups);
  it /= static_cast<uint32_t>(p.ngroups);
  r.g = it % static_cast<uint32_t>(p.groups);
  it /= static_cast<uint32_t>(p.groups);
  r.ct = it % static_cast<uint32_t>(p.ctiles);
  r.kt = it / static_cast<uint32_t>(p.ctiles);
  r.t_begin = r.sp * per_split;
  r.t_end = r.t_begin + per_split < pix_tiles ? r.t_begin + per_split : pix_tiles;
  return r;
}

// The MMAs of one stage: `ksteps` reduction steps of kK rows, NT taps each (tap q accumulates into
// TMEM columns [q * kBN, +kBN) and reads the x tile toff[q] address units further).  Straight-line
// code in blocks of four steps: the issuing thread must spend fewer clocks per MMA than the MMA
// takes (64 for 128 x 128 x 8 tf32).
template <MmaKind KIND, int NT, int KS>
__device__ __forceinline__ void issue_stage(uint32_t tmem, uint32_t a_lo, uint32_t b_lo, const uint32_t (&toff)[4],
                                            uint32_t desc_hi, int ksteps, uint32_t acc, uint32_t stack_delta) {
  constexpr int kK = KIND == MmaKind::TF32 ? 8 : 16;
  constexpr uint32_t kStep = (kK * 128) >> 4;
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, true, true, 128, kBN);
  uint32_t bq[NT];
#pragma unroll
  for (int q = 0; q < NT; ++q) bq[q] = b_lo + toff[q];
  if (stack_delta) {
    // Layers with at most 64 channels: the NT taps become NT groups of 64 columns of ONE MMA.  The x operand's
    // leading-dimension offset (the distance between 64-column groups) is set to the taps' row spacing, so that
    // column group q reads the x tile q taps further: 128 x (64 NT) instead of NT half-empty 128 x 128 MMAs.
    constexpr uint32_t kIdescStack = instr_desc(KIND == MmaKind::TF32, true, true, 128, 64 * NT);
    for (int ks = 0; ks < ksteps; ++ks) {
      umma_words<KIND>(tmem, a_lo + ks * kStep, bq[0] + stack_delta + ks * kStep, desc_hi, kIdescStack, acc);
      acc = 1u;
    }
    return;
  }
  if (KS > 0) {           // exactly KS steps: straight-line code
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int q = 0; q < NT; ++q)
        umma_words<KIND>(tmem + q * kBN, a_lo + ks * kStep, bq[q] + ks * kStep, desc_hi, kIdesc, ks == 0 ? acc : 1u);
    }
    return;
  }
  int ks = 0;
  for (; ks + 4 <= ksteps; ks += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int q = 0; q < NT; ++q)
        umma_words<KIND>(tmem + q * kBN, a_lo + (ks + u) * kStep, bq[q] + (ks + u) * kStep, desc_hi, kIdesc,
                         u == 0 ? acc : 1u);
    }
    acc = 1u;
  }
  for (; ks < ksteps; ++ks) {
#pragma unroll
    for (int q = 0; q < NT; ++q)
      umma_words<KIND>(tmem + q * kBN, a_lo + ks * kStep, bq[q] + ks * kStep, desc_hi, kIdesc, acc);
    acc = 1u;
  }
}

// The MMA issuer's loop over the pixel tiles (pipeline stages) of one work item with NT taps.
// Returns false when a wait ran out.  `stage`/`phase` carry the pipeline position across items.
template <MmaKind KIND, int NT, int KS>
__device__ __forceinline__ bool mma_item(Bars* bars, uint32_t tmem, uint32_t lo_base, uint32_t desc_hi,
                                         const uint32_t (&toff)[4], int ksteps, int ntiles, int& stage,
                                         uint32_t& phase, long long& t_wait, bool timed, bool leader,
                                         long long limit, uint32_t stack_delta) {
  constexpr int kAtom = atom<KIND>();
  constexpr int kABoxes = 128 / kAtom;
  constexpr int kStages = num_stages<KIND>();
  constexpr int kBoxBytes = box_bytes<KIND>();
  uint32_t acc = 0u;
  for (int t = 0; t < ntiles; ++t) {
    if (timed) {
      const long long tw = clock64();
      if (!uniform_wait(&bars->full[stage], phase, bars, limit)) return false;
      t_wait += clock64() - tw;
    } else if (!uniform_wait(&bars->full[stage], phase, bars, limit)) {
      return false;
    }
    tc_fence_after();
    const uint32_t a_lo = lo_base + stage * (stage_bytes<KIND>() >> 4);
    const uint32_t b_lo = a_lo + ((kABoxes * kBoxBytes) >> 4);
    if (leader) {
      issue_stage<KIND, NT, KS>(tmem, a_lo, b_lo, toff, desc_hi, ksteps, acc, stack_delta);
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

template <MmaKind KIND>
__global__ void __launch_bounds__(kThreads, 1)
wgrad_group_kernel(const __grid_constant__ GroupWgradParams p) {
  constexpr int kAtom = atom<KIND>();
  constexpr int kABoxes = 128 / kAtom, kBBoxes = kBN / kAtom;
  constexpr int kStages = num_stages<KIND>();
  constexpr int kBoxBytes = box_bytes<KIND>(), kBoxRows = box_rows<KIND>();
  constexpr int kK = KIND == MmaKind::TF32 ? 8 : 16;
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, true, true, 128, kBN);
  constexpr uint32_t kSbo = KIND == MmaKind::TF32 ? 512 : 1024;
  constexpr uint64_t kLayout = KIND == MmaKind::TF32 ? kSwizzle128Base32 : kSwizzle128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * stage_bytes<KIND>());

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  // phase timing (optional): [0] MMA thread waiting for operands, [1] its whole loop,
  // [2] first producer waiting for a free stage, [3] its whole loop, [4] kernel start to end,
  // [9] / [10] GPU-wide timer at start / end
  long long* trace = p.trace ? p.trace + blockIdx.x * 16 : nullptr;
  const long long t_begin = trace ? clock64() : 0;
  if (trace && threadIdx.x == 0) trace[9] = static_cast<long long>(global_ns());
  const int ksteps = (p.rows_a + kK - 1) / kK;
  const uint32_t pix_tiles = static_cast<uint32_t>(p.tiles_w) * p.tiles_h * p.tiles_n;
  const uint32_t per_split = (pix_tiles + p.splits - 1) / p.splits;
  const uint32_t total = static_cast<uint32_t>(p.ktiles) * p.ctiles * p.groups * p.ngroups * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->acc_empty, 32 * kEpilogueWarps);
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  // Rows past the boxes are never written by TMA.  The MMA reads whole groups of kK dy rows and,
  // for the x operand, up to the largest column offset further: clear those rows once.  (dy rows
  // there must be zero; the x rows only need to be finite.)
  {
    const int boxes = kStages * (kABoxes + kBBoxes);
    const int first = min(p.rows_a, p.rows_b);
    const int nrows = kBoxRows - first;
    for (int i = threadIdx.x; i < boxes * nrows * 8; i += kThreads) {
      const int box = i / (nrows * 8), rem = i % (nrows * 8);
      const int stage_box = box % (kABoxes + kBBoxes);
      const int row = first + rem / 8;
      const int written = stage_box < kABoxes ? p.rows_a : p.rows_b;
      if (row >= written)
        *(reinterpret_cast<uint4*>(smem + box * kBoxBytes + row * 128) + rem % 8) = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
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
      const int view = p.grp_view[w.grp], dh = p.grp_dh[w.grp], dwmin = p.view_dwmin[view];
      const int a_boxes = min(kABoxes, (p.Kg - w.kt * 128 + kAtom - 1) / kAtom);
      const int b_boxes = min(kBBoxes, (p.Cg - w.ct * kBN + kAtom - 1) / kAtom);
      const uint32_t tx = (a_boxes * p.rows_a + b_boxes * p.rows_b) * 128;
      // tile coordinates advance by counting: 64-bit divisions per stage would cost the producers
      // more clocks than the stage's MMAs take
      int tw = static_cast<int>(w.t_begin % static_cast<uint32_t>(p.tiles_w));
      int th_ = static_cast<int>((w.t_begin / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h));
      int tn = static_cast<int>(w.t_begin / (static_cast<uint32_t>(p.tiles_w) * p.tiles_h));
      for (uint32_t t = w.t_begin; t < w.t_end; ++t) {
        const int w0 = tw * p.wt, h0 = th_ * p.th, n0 = tn * p.nb;
        if (++tw == p.tiles_w) {
          tw = 0;
          if (++th_ == p.tiles_h) { th_ = 0; ++tn; }
        }
        const long long tw0 = trace ? clock64() : 0;
        if (!uniform_wait(&bars->empty[stage], phase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        if (trace) t_wait += clock64() - tw0;
        uint8_t* sa = smem + stage * stage_bytes<KIND>();
        uint8_t* sb = sa + kABoxes * kBoxBytes;
        if (leader) {
          if (pw == 0) mbar_expect_tx(&bars->full[stage], tx);
          for (int j = pw; j < a_boxes + b_boxes; j += kProducers) {
            if (j < a_boxes)
              tma_load_5d(sa + j * kBoxBytes, &p.dy_map, &bars->full[stage], w.kt * 128 + j * kAtom, w.g,
                          w0, h0, n0);
            else
              tma_load_5d(sb + (j - a_boxes) * kBoxBytes, &p.x_views[view], &bars->full[stage],
                          w.ct * kBN + (j - a_boxes) * kAtom, w.g, w0 + dwmin, h0 + dh, n0);
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
    const bool timed = trace != nullptr;
    const long long lim = p.wait_clocks;
    // stacked taps: the low descriptor word carries the leading-dimension offset in bits [16, 30)
    const uint32_t stack_delta = p.stack_step > 0
        ? ((static_cast<uint32_t>(p.stack_step * 128) >> 4) - (static_cast<uint32_t>(kBoxBytes) >> 4)) << 16 : 0u;
    for (uint32_t it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int first_tap = p.grp_first[w.grp], ntap = p.grp_n[w.grp];
      // row offset of every tap's x operand, in descriptor address units (16 bytes)
      uint32_t toff[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        toff[q] = q < ntap ? static_cast<uint32_t>(p.tap_off[first_tap + q]) * (128u >> 4) : 0u;
      if (!uniform_wait(&bars->acc_empty, (n & 1) ^ 1, bars, lim)) { ok = false; break; }
      tc_fence_after();
      const int ntiles = static_cast<int>(w.t_end - w.t_begin);
      switch (ntap) {
        case 1: ok = (ksteps == 8 && !timed ? mma_item<KIND, 1, 8>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, false, leader, lim, stack_delta)
                                             : mma_item<KIND, 1, 0>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, timed, leader, lim, stack_delta)); break;
        case 2: ok = (ksteps == 8 && !timed ? mma_item<KIND, 2, 8>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, false, leader, lim, stack_delta)
                                             : mma_item<KIND, 2, 0>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, timed, leader, lim, stack_delta)); break;
        case 3: ok = (ksteps == 8 && !timed ? mma_item<KIND, 3, 8>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, false, leader, lim, stack_delta)
                                             : mma_item<KIND, 3, 0>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, timed, leader, lim, stack_delta)); break;
        default: ok = (ksteps == 8 && !timed ? mma_item<KIND, 4, 8>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, false, leader, lim, stack_delta)
                                             : mma_item<KIND, 4, 0>(bars, tmem, lo_base, desc_hi, toff, ksteps, ntiles, stage, phase, t_wait, timed, leader, lim, stack_delta)); break;
      }
      if (ok && leader) umma_commit(&bars->acc_full);
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
    if (trace && leader) { trace[0] = t_wait; trace[1] = clock64() - t_begin; }
  } else {
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int K = p.Kg * p.groups;
    bool ok = true;
    int n = 0;
    for (uint32_t it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int first_tap = p.grp_first[w.grp], ntap = p.grp_n[w.grp];
      if (!warp_wait_or_abort(&bars->acc_full, n & 1, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const int kq = w.kt * 128 + row;
      const bool valid = kq < p.Kg;
      const int slab = p.atomic ? 0 : w.sp;
      const bool vec = (p.Cg & 3) == 0 && !p.atomic;
      const int items = ntap * (kBN / 32);
#pragma unroll 1
      for (int item = sub; item < items; item += kEpilogueWarps / 4) {
        const int q = item / (kBN / 32), ch = item % (kBN / 32);
        const int c0 = w.ct * kBN + ch * 32;
        if (c0 >= p.Cg) continue;
        uint32_t r[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + q * (p.stack_step > 0 ? 64 : kBN) + ch * 32, r);
        tmem_ld_wait();
        if (!valid) continue;
        float* dst = p.partial +
                     ((1LL * slab * p.taps_total + p.tap_wmat[first_tap + q]) * K + w.g * p.Kg + kq) * p.Cg;
        if (vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (c0 + j < p.Cg && B200_IN_RANGE((dst - p.partial) + c0 + j >= 0 && (dst - p.partial) + c0 + j + 4 <= p.partial_elems, p.status))
              *reinterpret_cast<float4*>(dst + c0 + j) =
                  make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                              __uint_as_float(r[j + 3]));
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
      tc_fence_before();
      mbar_arrive(&bars->acc_empty);
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
    tmem_dealloc(tmem, 512);
  }
}

template <MmaKind KIND>
cudaError_t launch_one(const GroupWgradParams& p, long long total, int num_sms, cudaStream_t s) {
  constexpr int smem = num_stages<KIND>() * stage_bytes<KIND>() + sizeof(Bars) + 1024;
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] { return cudaFuncSetAttribute(wgrad_group_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (e != cudaSuccess) return e;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  wgrad_group_kernel<KIND><<<grid, kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_wgrad_group(const GroupWgradParams& p, int dtype, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.ktiles * p.ctiles * p.groups * p.ngroups * p.splits;
  if (total == 0) return cudaSuccess;
  if (total >= (1LL << 31) || 1LL * p.tiles_w * p.tiles_h * p.tiles_n >= (1LL << 31)) return cudaErrorInvalidValue;
  return dtype == B200CONV_F16 ? launch_one<MmaKind::F16>(p, total, num_sms, s)
                               : launch_one<MmaKind::TF32>(p, total, num_sms, s);
}

}  // namespace b200
