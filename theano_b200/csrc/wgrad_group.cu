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
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, 16 epilogue warps.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kBN = 128;                       // channels per accumulator
constexpr int kBoxRows = 80;                   // 64 pixel rows + room for the largest column offset
constexpr int kBoxBytes = kBoxRows * 128;      // 10 KB, a multiple of the 1024-byte swizzle period
constexpr int kSmemBudget = 208 * 1024;
constexpr int kMaxStages = 6;

template <MmaKind KIND> constexpr int atom() { return KIND == MmaKind::TF32 ? 32 : 64; }
template <MmaKind KIND> constexpr int stage_bytes() { return (128 / atom<KIND>() + kBN / atom<KIND>()) * kBoxBytes; }
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

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Bars* b) {
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63) {
      if (b->abort) return false;
      if (clock64() - t0 > 4000000000LL) {
        b->abort = 1;
        return false;
      }
    }
  }
}

struct Item {
  int kt, ct, g, grp, sp;
  long long t_begin, t_end;
};

__device__ __forceinline__ Item decode(long long it, const GroupWgradParams& p, long long per_split,
                                       long long pix_tiles) {
  Item r;
  r.sp = it % p.splits;
  it /= p.splits;
  r.grp = it % p.ngroups;
  it /= p.ngroups;
  r.g = it % p.groups;
  it /= p.groups;
  r.ct = it % p.ctiles;
  r.kt = it / p.ctiles;
  r.t_begin = r.sp * per_split;
  r.t_end = r.t_begin + per_split < pix_tiles ? r.t_begin + per_split : pix_tiles;
  return r;
}

template <MmaKind KIND>
__global__ void __launch_bounds__(kThreads, 1)
wgrad_group_kernel(const __grid_constant__ GroupWgradParams p) {
  constexpr int kAtom = atom<KIND>();
  constexpr int kABoxes = 128 / kAtom, kBBoxes = kBN / kAtom;
  constexpr int kStages = num_stages<KIND>();
  constexpr int kK = KIND == MmaKind::TF32 ? 8 : 16;
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, true, true, 128, kBN);
  constexpr uint32_t kSbo = KIND == MmaKind::TF32 ? 512 : 1024;
  constexpr uint64_t kLayout = KIND == MmaKind::TF32 ? kSwizzle128Base32 : kSwizzle128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * stage_bytes<KIND>());

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ksteps = (p.rows_a + kK - 1) / kK;
  const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
  const long long per_split = (pix_tiles + p.splits - 1) / p.splits;
  const long long total = 1LL * p.ktiles * p.ctiles * p.groups * p.ngroups * p.splits;

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

  if (warp == 0) {
    if (lane == 0) {
      for (int v = 0; v < kMaxViews; ++v) tma_prefetch_desc(&p.x_views[v]);
      tma_prefetch_desc(&p.dy_map);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long it = blockIdx.x; it < total && ok; it += gridDim.x) {
        const Item w = decode(it, p, per_split, pix_tiles);
        const int view = p.grp_view[w.grp], dh = p.grp_dh[w.grp], dwmin = p.view_dwmin[view];
        const int a_boxes = min(kABoxes, (p.Kg - w.kt * 128 + kAtom - 1) / kAtom);
        const int b_boxes = min(kBBoxes, (p.Cg - w.ct * kBN + kAtom - 1) / kAtom);
        const uint32_t tx = (a_boxes * p.rows_a + b_boxes * p.rows_b) * 128;
        for (long long t = w.t_begin; t < w.t_end; ++t) {
          const int w0 = (t % p.tiles_w) * p.wt;
          const int h0 = ((t / p.tiles_w) % p.tiles_h) * p.th;
          const int n0 = (t / (1LL * p.tiles_w * p.tiles_h)) * p.nb;
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, bars)) { ok = false; break; }
          uint8_t* sa = smem + stage * stage_bytes<KIND>();
          uint8_t* sb = sa + kABoxes * kBoxBytes;
          mbar_expect_tx(&bars->full[stage], tx);
          for (int b = 0; b < a_boxes; ++b)
            tma_load_5d(sa + b * kBoxBytes, &p.dy_map, &bars->full[stage], w.kt * 128 + b * kAtom, w.g,
                        w0, h0, n0);
          for (int b = 0; b < b_boxes; ++b)
            tma_load_5d(sb + b * kBoxBytes, &p.x_views[view], &bars->full[stage], w.ct * kBN + b * kAtom,
                        w.g, w0 + dwmin, h0 + dh, n0);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) atomicExch(p.status, kStatusTimeout);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int n = 0;
      for (long long it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
        const Item w = decode(it, p, per_split, pix_tiles);
        const int first_tap = p.grp_first[w.grp], ntap = p.grp_n[w.grp];
        if (!wait_or_abort(&bars->acc_empty, (n & 1) ^ 1, bars)) { ok = false; break; }
        tc_fence_after();
        bool first = true;
        for (long long t = w.t_begin; t < w.t_end; ++t) {
          if (!wait_or_abort(&bars->full[stage], phase, bars)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes<KIND>());
          const uint32_t sb = sa + kABoxes * kBoxBytes;
          for (int ks = 0; ks < ksteps; ++ks) {
            const uint64_t adesc = smem_desc(sa + ks * kK * 128, kBoxBytes, kSbo, kLayout);
            for (int q = 0; q < ntap; ++q) {
              const uint32_t boff = static_cast<uint32_t>(ks * kK + p.tap_off[first_tap + q]) * 128u;
              umma<KIND>(tmem + q * kBN, adesc, smem_desc(sb + boff, kBoxBytes, kSbo, kLayout), kIdesc,
                         first ? 0u : 1u);
            }
            first = false;
          }
          umma_commit(&bars->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full);
      }
      if (!ok) atomicExch(p.status, kStatusTimeout);
    }
  } else {
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int K = p.Kg * p.groups;
    bool ok = true;
    int n = 0;
    for (long long it = blockIdx.x; it < total && ok; it += gridDim.x, ++n) {
      const Item w = decode(it, p, per_split, pix_tiles);
      const int first_tap = p.grp_first[w.grp], ntap = p.grp_n[w.grp];
      if (!wait_or_abort(&bars->acc_full, n & 1, bars)) { ok = false; break; }
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
        tmem_ld32(tmem + (static_cast<uint32_t>(quad * 32) << 16) + q * kBN + ch * 32, r);
        tmem_ld_wait();
        if (!valid) continue;
        float* dst = p.partial +
                     ((1LL * slab * p.taps_total + p.tap_wmat[first_tap + q]) * K + w.g * p.Kg + kq) * p.Cg;
        if (vec) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (c0 + j < p.Cg)
              *reinterpret_cast<float4*>(dst + c0 + j) =
                  make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                              __uint_as_float(r[j + 3]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < p.Cg) {
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <MmaKind KIND>
cudaError_t launch_one(const GroupWgradParams& p, long long total, int num_sms, cudaStream_t s) {
  constexpr int smem = num_stages<KIND>() * stage_bytes<KIND>() + sizeof(Bars) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wgrad_group_kernel<KIND>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  wgrad_group_kernel<KIND><<<grid, kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_wgrad_group(const GroupWgradParams& p, int dtype, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.ktiles * p.ctiles * p.groups * p.ngroups * p.splits;
  if (total == 0) return cudaSuccess;
  return dtype == B200CONV_F16 ? launch_one<MmaKind::F16>(p, total, num_sms, s)
                               : launch_one<MmaKind::TF32>(p, total, num_sms, s);
}

}  // namespace b200
