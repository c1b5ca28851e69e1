// Implicit-GEMM convolution with activation reuse across filter taps (tcgen05 + TMEM).
//
// When every tap reads the same channels-last view (stride-1 forward, every parity class of
// gradInputs) the operand rows of different taps are the same pixels shifted by a constant: with
// the output tile laid out on the slab's own pixel grid (tile width + halo columns), tap (dh, dw)
// is the slab advanced by dh * Ws + dw rows.  So one TMA box brings the slab (tile + halo, 128
// bytes of channels per pixel) once per channel block, and each tap's MMA reads it through a
// shared-memory descriptor that starts at the tap's row offset.  Only the filter tile is fetched
// per tap.  Accumulator rows that fall on halo columns / rows are computed and thrown away.
//
// A CTA keeps up to 512 TMEM columns of accumulators (two 128 x 256 tiles, or four 128 x 128 ...)
// so that a filter tile serves up to 512 output pixels.  Warp roles: warp 0 streams the activation
// slabs, warp 19 the filter tiles (TMA producers), warp 1 issues the MMAs and owns the TMEM, 16 epilogue
// warps; warp 18 is a second MMA issuer: with two or more accumulators per tile each issuer takes half
// of them (different TMEM columns, the same operands, the same order of accumulation).  Producer and
// issuer loops are followed by all 32 lanes of their warp; one elected lane issues.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

constexpr int kEpilogueWarps = 16;
constexpr int kSecondIssuer = 2 + kEpilogueWarps;     // warp index
constexpr int kFilterProducer = kSecondIssuer + 1;    // warp index: streams the filter tiles (warp 0 the slabs)
constexpr int kThreads = 32 * (kFilterProducer + 1);
constexpr int kMaxBStages = 8;
constexpr int kMaxSlabStages = 6;

struct alignas(16) Bars {
  uint64_t slab_full[kMaxSlabStages];
  uint64_t slab_empty[kMaxSlabStages];
  uint64_t b_full[kMaxBStages];
  uint64_t b_empty[kMaxBStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
};

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__half>(__half* p, float v) { *p = __float2half_rn(v); }

template <MmaKind KIND, int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_slab_kernel(const __grid_constant__ SlabConvParams p) {
  using OutT = typename std::conditional<KIND == MmaKind::TF32, float, __half>::type;
  constexpr int kBK = KIND == MmaKind::TF32 ? 32 : 64;
  constexpr uint32_t kIdesc = instr_desc(KIND == MmaKind::TF32, false, false, 128, BN);
  constexpr int kBBytes = BN * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bring = smem + p.s_stages * p.slab_bytes;    // the slab ring comes first
  const int stage_b = p.tps * kBBytes;                  // bytes of one filter stage: tps taps
  Bars* bars = reinterpret_cast<Bars*>(bring + p.b_stages * stage_b + p.stage_reserved);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  long long* trace = p.trace ? p.trace + blockIdx.x * 32 : nullptr;   // 32 slots per CTA
  if (trace && threadIdx.x == 0) {
    trace[0] = clock64();
    trace[7] = static_cast<long long>(global_ns());
  }
  const uint32_t slab_tx = static_cast<uint32_t>(p.nb * p.Hs * p.Ws) * 128u;
  // tile counts fit 32 bits (the launcher checks): 64-bit divisions per tile would cost each
  // role about a thousand clocks, a fifth of a small tile
  const uint32_t total = static_cast<uint32_t>(p.tiles_w) * p.tiles_h * p.tiles_n * p.groups * p.tiles_co;
  const uint32_t co_groups = static_cast<uint32_t>(p.tiles_co) * p.groups, tiles_wh = static_cast<uint32_t>(p.tiles_w) * p.tiles_h;
  const bool dbl = 2 * p.n_acc * BN <= 512;
  const int issuers = p.n_acc >= 2 ? 2 : 1;

  if (threadIdx.x == 0) {
    // operands are released, and accumulators handed over, when every issuer's MMAs are done
    for (int s = 0; s < kMaxSlabStages; ++s) {
      mbar_init(&bars->slab_full[s], 1);
      mbar_init(&bars->slab_empty[s], issuers);
    }
    for (int s = 0; s < kMaxBStages; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], issuers);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], issuers);
      mbar_init(&bars->acc_empty[b], 32 * kEpilogueWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  if (trace && threadIdx.x == 0) trace[1] = clock64();

  if (warp == 0) {
    // Slab producer.  Every lane runs the loop (so that its control flow and address arithmetic are
    // warp-uniform); one elected lane issues the copies.  Slabs and filter tiles have a producer warp
    // each: one in-order producer stalled on a free slab buffer while the filter ring ran dry, and the
    // MMA warp then waited a full L2 latency for filters (a third of its loop on the 3x3 layers).
    const bool leader = elect_one();
    if (leader) tma_prefetch_desc(&p.view);
    int sb = 0;
    uint32_t sphase = 0;
    bool ok = true;
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int g = (t / static_cast<uint32_t>(p.tiles_co)) % static_cast<uint32_t>(p.groups);
      const uint32_t pt = t / co_groups;
      const int w0 = (pt % static_cast<uint32_t>(p.tiles_w)) * p.wt;
      const int h0 = ((pt / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h)) * p.th;
      const int n0 = (pt / tiles_wh) * p.nb;
      for (int kb = 0; kb < p.kblocks; ++kb) {
        if (!uniform_wait(&bars->slab_empty[sb], sphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        if (leader) {
          mbar_expect_tx(&bars->slab_full[sb], slab_tx);
          tma_load_5d(smem + sb * p.slab_bytes, &p.view, &bars->slab_full[sb], kb * kBK, g, w0 + p.dw_min,
                      h0 + p.dh_min, n0);
        }
        if (++sb == p.s_stages) { sb = 0; sphase ^= 1; }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else if (warp == kFilterProducer) {
    // Filter producer: the same walk over tiles, channel blocks and taps, filter tiles only.
    const bool leader = elect_one();
    if (leader) tma_prefetch_desc(&p.wmap);
    int bs = 0;
    uint32_t bphase = 0;
    bool ok = true;
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int g = (t / static_cast<uint32_t>(p.tiles_co)) % static_cast<uint32_t>(p.groups);
      for (int kb = 0; kb < p.kblocks && ok; ++kb) {
        for (int tap = 0; tap < p.ntaps; tap += p.tps) {
          if (!uniform_wait(&bars->b_empty[bs], bphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
          const int nt = min(p.tps, p.ntaps - tap);         // taps of this stage
          if (leader) {
            mbar_expect_tx(&bars->b_full[bs], nt * kBBytes);
            for (int q = 0; q < nt; ++q)
              tma_load_3d(bring + bs * stage_b + q * kBBytes, &p.wmap, &bars->b_full[bs], kb * kBK, co_t * BN,
                          p.tap_wmat[tap + q] * p.groups + g);
          }
          if (++bs == p.b_stages) { bs = 0; bphase ^= 1; }
        }
      }
    }
    if (!ok && leader) atomicExch(p.status, kStatusTimeout);
  } else if (warp == 1 || warp == kSecondIssuer) {
    // this issuer's accumulators of every tile: [a_begin, a_end)
    const int a_split = issuers == 2 ? (p.n_acc + 1) / 2 : p.n_acc;
    const int a_begin = warp == 1 ? 0 : a_split, a_end = warp == 1 ? a_split : p.n_acc;
    if (warp != 1) trace = nullptr;            // the stamps are the first issuer's
    if (a_begin < a_end) {
      // All 32 lanes follow the loop and wait on the barriers; one elected lane issues the MMAs
      // and their commits.  A lone lane (code under `if (lane == 0)`) computes every descriptor
      // on the per-thread datapath and moves it to uniform registers per MMA, which costs more
      // clocks than a 128 x 64 or 128 x 128 MMA runs.
      const bool leader = elect_one();
      if (!leader) trace = nullptr;
      int sb = 0, bs = 0;
      uint32_t sphase = 0, bphase = 0;
      bool ok = true;
      int it = 0;
      long long tw_acc = 0, tw_slab = 0, tw_b = 0;       // clocks spent waiting (only with trace)
      const long long t_loop0 = trace ? clock64() : 0;
      const uint64_t desc_bits = smem_desc(0, 16, 1024);
      const uint32_t desc_hi = static_cast<uint32_t>(desc_bits >> 32);
      const uint32_t desc_lo = static_cast<uint32_t>(desc_bits);
      for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
        // two accumulator sets when they fit the 512 TMEM columns: the epilogue of a tile then
        // runs beside the MMAs of the next one
        const int buf = dbl ? (it & 1) : 0;
        const uint32_t aphase = dbl ? ((it >> 1) & 1) : (it & 1);
        const uint32_t acc_base = tmem + buf * (p.n_acc * BN);
        long long tq = trace ? clock64() : 0;
        if (!uniform_wait(&bars->acc_empty[buf], aphase ^ 1, bars, p.wait_clocks)) { ok = false; break; }
        if (trace) tw_acc += clock64() - tq;
        tc_fence_after();
        for (int kb = 0; kb < p.kblocks && ok; ++kb) {
          tq = trace ? clock64() : 0;
          if (!uniform_wait(&bars->slab_full[sb], sphase, bars, p.wait_clocks)) { ok = false; break; }
          if (trace) tw_slab += clock64() - tq;
          if (trace && it == 0 && kb == 0) trace[2] = clock64();
          const uint32_t sbase = smem_u32(smem + sb * p.slab_bytes);
          for (int tap0 = 0; tap0 < p.ntaps; tap0 += p.tps) {
            tq = trace ? clock64() : 0;
            if (!uniform_wait(&bars->b_full[bs], bphase, bars, p.wait_clocks)) { ok = false; break; }
            if (trace) tw_b += clock64() - tq;
            tc_fence_after();
            const int nt = min(p.tps, p.ntaps - tap0);
            if (leader) {
              for (int q = 0; q < nt; ++q) {
                const int tap = tap0 + q;
                // only the address field of the two descriptors changes from MMA to MMA
                const uint32_t b_lo = desc_lo + (smem_u32(bring + bs * stage_b + q * kBBytes) >> 4);
                const uint32_t first = (kb | tap) != 0;
                uint32_t a_lo = desc_lo + ((sbase + static_cast<uint32_t>(p.tap_shift[tap] + 128 * a_begin) * 128u) >> 4);
                for (int a = a_begin; a < a_end; ++a) {
#pragma unroll
                  for (int kk = 0; kk < 4; ++kk)
                    umma_words<KIND>(acc_base + a * BN, a_lo + 2 * kk, b_lo + 2 * kk, desc_hi, kIdesc, first | (kk != 0));
                  a_lo += (128 * 128) >> 4;      // next accumulator: 128 slab rows further
                }
              }
              umma_commit(&bars->b_empty[bs]);
            }
            if (++bs == p.b_stages) { bs = 0; bphase ^= 1; }
          }
          if (ok && leader) umma_commit(&bars->slab_empty[sb]);
          if (++sb == p.s_stages) { sb = 0; sphase ^= 1; }
        }
        if (ok && leader) umma_commit(&bars->acc_full[buf]);
        if (trace && it == 0) trace[3] = clock64();
      }
      if (!ok && leader) atomicExch(p.status, kStatusTimeout);
      if (trace) {
        trace[9] = tw_acc; trace[10] = tw_slab; trace[11] = tw_b;
        trace[12] = clock64() - t_loop0; trace[13] = it;
      }
    }
  } else if (warp < kSecondIssuer) {
    // 16 epilogue warps: warp w reads TMEM lanes [32*(w%4), +32) (the hardware's rule) and, of
    // those rows, every fourth 32-column chunk.  A single warp keeps only a few stores in flight,
    // so the store bandwidth of the SM is reached by the number of warps, not by wider stores.
    const int quad = warp & 3;
    const int sub = (warp - 2) >> 2;
    OutT* out = static_cast<OutT*>(p.out);
    const int per_img = p.Hs * p.Ws;
    // channels-last output whose 32-channel groups are 16-byte aligned: 16-byte stores
    const bool rowwise = p.out_sc == 1 && ((p.n_out * sizeof(OutT)) & 15) == 0;
    bool ok = true;
    int it = 0;
    long long te_wait = 0, te_busy = 0;          // clocks of thread 64 (only with trace)
    long long tp[5] = {0, 0, 0, 0, 0};           // its epilogue phases: buffer wait, TMEM read, convert + stage, fence + barrier, store issue
    int nstore = 0;                              // chunks this warp's group has staged so far
    for (uint32_t t = blockIdx.x; t < total && ok; t += gridDim.x, ++it) {
      const int co_t = t % static_cast<uint32_t>(p.tiles_co);
      const int g = (t / static_cast<uint32_t>(p.tiles_co)) % static_cast<uint32_t>(p.groups);
      const uint32_t pt = t / co_groups;
      const int w0 = (pt % static_cast<uint32_t>(p.tiles_w)) * p.wt;
      const int h0 = ((pt / static_cast<uint32_t>(p.tiles_w)) % static_cast<uint32_t>(p.tiles_h)) * p.th;
      const int n0 = (pt / tiles_wh) * p.nb;
      const int buf = dbl ? (it & 1) : 0;
      const uint32_t aphase = dbl ? ((it >> 1) & 1) : (it & 1);
      const long long te0 = trace ? clock64() : 0;
      if (!warp_wait_or_abort(&bars->acc_full[buf], aphase, bars, lane, p.wait_clocks)) { ok = false; break; }
      tc_fence_after();
      const long long te1 = trace ? clock64() : 0;
      if (trace && it == 0 && threadIdx.x == 64) trace[4] = clock64();
      const int co_base = co_t * BN;
      const int nchunks = min(BN / 32, (p.n_out - co_base + 31) / 32);
      const uint32_t lane_base = tmem + buf * (p.n_acc * BN) + (static_cast<uint32_t>(quad * 32) << 16);

      if (p.tma_out) {
        // Groups of 4 * n_acc warps take whole 128-byte channel chunks of the tile: lane -> its pixel's
        // dense row of a staging buffer (16-byte pieces swizzled like the store map expects),
        // then one thread stores the box.  Bias and ReLU are applied on the way.  A group owns
        // `bufs` staging buffers and fills them in turn; before a buffer is refilled only the
        // store that last read it must have finished reading, so a store runs beside the next
        // chunk's (or the next tile's) TMEM reads instead of being waited for.
        const int a = sub % p.n_acc, grp = sub / p.n_acc, ngrp = (kEpilogueWarps / 4) / p.n_acc;
        const int gthreads = 128 * p.n_acc;
        const int pos = a * 128 + quad * 32 + lane;
        const int ni = pos / per_img, rem = pos % per_img;
        const int hh = rem / p.Ws, ww = rem % p.Ws;
        const bool inbox = ni < p.nb && hh < p.th && ww < p.wt;
        const int drow = (ni * p.th + hh) * p.wt + ww;
        const bool issuer = a == 0 && quad == 0 && lane == 0;   // issues all of the group's stores
        const bool plain = p.epi.alpha == 1.f && !p.bias && !p.relu;
        const int bufs = p.stage_nbuf / ngrp >= 2 ? 2 : 1;
        constexpr int kCh = 128 / static_cast<int>(sizeof(OutT));   // channels of one 128-byte staged row
        const int nstaged = min(BN / kCh, (p.n_out - co_base + kCh - 1) / kCh);
        for (int ch = grp; ch < nstaged; ch += ngrp, ++nstore) {
          uint8_t* stg = smem + p.stage_off + (grp * bufs + (bufs == 2 ? (nstore & 1) : 0)) * p.stage_bytes;
          uint8_t* srow = stg + drow * 128;
          const int co0 = co_base + ch * kCh;
          const float* bias = p.bias ? p.bias + g * p.n_out + co0 : nullptr;
          long long tq = trace ? clock64() : 0;
          if (nstore >= bufs) {                // the buffer's previous box must have been read
            if (issuer) {
              if (bufs == 2) bulk_wait_read<1>();
              else bulk_wait_read<0>();
            }
            named_barrier(1 + grp, gthreads);
          }
          if (trace) { const long long t = clock64(); tp[0] += t - tq; tq = t; }
#pragma unroll
          for (int part = 0; part < kCh / 32; ++part) {
            uint32_t r[32];
            tmem_ld32(lane_base + a * BN + ch * kCh + part * 32, r);
            tmem_ld_wait();
            if (trace) { const long long t = clock64(); tp[1] += t - tq; tq = t; }
            if (!inbox) continue;
            const float* bp = bias ? bias + part * 32 : nullptr;
            if (plain) {
              // no scale, bias or activation (gradInputs, bare forward): convert and stage only.
              // The epilogue warps are bound by their instruction issue, not by TMEM or shared memory.
              if (sizeof(OutT) == 4) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  *reinterpret_cast<uint4*>(srow + ((j ^ (drow & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t h[4];
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    __half2 h2 = __floats2half2_rn(__uint_as_float(r[8 * j + 2 * q]), __uint_as_float(r[8 * j + 2 * q + 1]));
                    h[q] = *reinterpret_cast<uint32_t*>(&h2);
                  }
                  *reinterpret_cast<uint4*>(srow + (((part * 4 + j) ^ (drow & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                }
              }
            } else if (sizeof(OutT) == 4) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float f[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  f[q] = p.epi.alpha * __uint_as_float(r[4 * j + q]);
                  if (bp) f[q] += bp[4 * j + q];
                  if (p.relu) f[q] = p.epi.lin * f[q] + p.epi.abs * fabsf(f[q]);
                }
                *reinterpret_cast<float4*>(srow + ((j ^ (drow & 7)) << 4)) = make_float4(f[0], f[1], f[2], f[3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t h[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float f0 = p.epi.alpha * __uint_as_float(r[8 * j + 2 * q]);
                  float f1 = p.epi.alpha * __uint_as_float(r[8 * j + 2 * q + 1]);
                  if (bp) { f0 += bp[8 * j + 2 * q]; f1 += bp[8 * j + 2 * q + 1]; }
                  if (p.relu) {
                    f0 = p.epi.lin * f0 + p.epi.abs * fabsf(f0);
                    f1 = p.epi.lin * f1 + p.epi.abs * fabsf(f1);
                  }
                  __half2 h2 = __floats2half2_rn(f0, f1);
                  h[q] = *reinterpret_cast<uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(srow + (((part * 4 + j) ^ (drow & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
              }
            }
          }
          if (trace) { const long long t = clock64(); tp[2] += t - tq; tq = t; }
          if (p.epi.pool) {
            // 2x2 max pooling of the staged chunk (Pool{ignore_border=True, mode='max'}, ws = stride = 2): the
            // tile's width and height are even, so every window lies inside it.  The group's threads read the
            // four staged rows of a window (16-byte pieces, un-swizzled by row), keep the maxima in registers
            // until every read is done, then write the pooled rows to the front of the same buffer, swizzled
            // for the pooled rows, and the store below moves a quarter of the bytes.
            named_barrier(1 + grp, gthreads);
            const int tig = a * 128 + quad * 32 + lane;
            const int pw = p.wt >> 1, ph = p.th >> 1;
            const int prows = p.nb * ph * pw;
            uint4 keep[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = tig + u * gthreads;
              if (i < prows * 8) {
                const int pr = i >> 3, piece = i & 7;
                const int w2 = pr % pw, h2 = (pr / pw) % ph, ni2 = pr / (pw * ph);
                const int d00 = (ni2 * p.th + 2 * h2) * p.wt + 2 * w2;
                uint4 m = *reinterpret_cast<const uint4*>(stg + d00 * 128 + ((piece ^ (d00 & 7)) << 4));
#pragma unroll
                for (int k = 1; k < 4; ++k) {
                  const int dk = d00 + (k & 1) + (k >> 1) * p.wt;
                  const uint4 v = *reinterpret_cast<const uint4*>(stg + dk * 128 + ((piece ^ (dk & 7)) << 4));
                  if (sizeof(OutT) == 4) {
                    m.x = __float_as_uint(fmaxf(__uint_as_float(m.x), __uint_as_float(v.x)));
                    m.y = __float_as_uint(fmaxf(__uint_as_float(m.y), __uint_as_float(v.y)));
                    m.z = __float_as_uint(fmaxf(__uint_as_float(m.z), __uint_as_float(v.z)));
                    m.w = __float_as_uint(fmaxf(__uint_as_float(m.w), __uint_as_float(v.w)));
                  } else {
                    __half2* mh = reinterpret_cast<__half2*>(&m);
                    const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                    for (int e = 0; e < 4; ++e) mh[e] = __hmax2(mh[e], vh[e]);
                  }
                }
                keep[u] = m;
              }
            }
            named_barrier(1 + grp, gthreads);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = tig + u * gthreads;
              if (i < prows * 8) {
                const int pr = i >> 3, piece = i & 7;
                *reinterpret_cast<uint4*>(stg + pr * 128 + ((piece ^ (pr & 7)) << 4)) = keep[u];
              }
            }
          }
          fence_async_smem();
          named_barrier(1 + grp, gthreads);
          if (trace) { const long long t = clock64(); tp[3] += t - tq; tq = t; }
          // a tiled store must not start at a negative coordinate, and its staging rows must lie
          // inside the reserved shared memory
          if (issuer && B200_IN_RANGE(g * p.n_out + co0 >= 0 && w0 >= 0 && h0 >= 0 && n0 >= 0 && w0 < p.Wt && h0 < p.Ht &&
                                      n0 < p.Nimg && ch * kCh + kCh <= BN, p.status)) {
            if (p.epi.pool) tma_store_4d(&p.out_map, stg, g * p.n_out + co0, w0 >> 1, h0 >> 1, n0);
            else tma_store_4d(&p.out_map, stg, g * p.n_out + co0, w0, h0, n0);
            bulk_commit();
          }
        }
      } else
      for (int a = 0; a < p.n_acc; ++a) {
        // this lane's output pixel for accumulator a
        const int pos = a * 128 + quad * 32 + lane;        // position on the slab grid
        const int ni = pos / per_img, rem = pos % per_img;
        const int hh = rem / p.Ws, ww = rem % p.Ws;
        const int n = n0 + ni, h = h0 + hh, w = w0 + ww;
        const bool valid = ni < p.nb && hh < p.th && ww < p.wt && n < p.Nimg && h < p.Ht && w < p.Wt;
        OutT* pix = out + (p.out_off + n * p.out_sn + h * p.out_sh + w * p.out_sw) +
                    1LL * g * p.n_out * p.out_sc;
        const OutT* res = p.epi.residual ? static_cast<const OutT*>(p.epi.residual) + (pix - out) : nullptr;
        for (int ch = sub; ch < nchunks; ch += kEpilogueWarps / 4) {
          uint32_t r[32];
          tmem_ld32(lane_base + a * BN + ch * 32, r);
          tmem_ld_wait();
          if (!valid) continue;
          const int co0 = co_base + ch * 32;
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
                  store_out<OutT>(pix + (co0 + j) * p.out_sc, v);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->acc_empty[buf]);
      if (trace && it == 0 && threadIdx.x == 64) trace[5] = clock64();
      if (trace) { te_wait += te1 - te0; te_busy += clock64() - te1; }
    }
    if (trace && threadIdx.x == 64) {
      trace[14] = te_wait; trace[15] = te_busy;
      for (int q = 0; q < 4; ++q) trace[16 + q] = tp[q];
    }
    if (p.tma_out && lane == 0) bulk_wait<0>();  // this thread's stores (if it issued any) have left shared memory
    if (!ok && lane == 0) atomicExch(p.status, kStatusTimeout);
  }

  tc_fence_before();
  __syncthreads();
  if (bars->abort) abort_grace(p.wait_clocks);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (trace && threadIdx.x == 0) {
    trace[6] = clock64();
    trace[8] = static_cast<long long>(global_ns());
  }
}

template <MmaKind KIND, int BN>
cudaError_t launch_one(const SlabConvParams& p, long long total, int num_sms, cudaStream_t s) {
  const int smem = p.s_stages * p.slab_bytes + p.b_stages * p.tps * BN * 128 + p.stage_reserved + sizeof(Bars) + 1024;
  static PerDeviceOnce configured;
  cudaError_t e = configured.ensure([] {
    return cudaFuncSetAttribute(conv_slab_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  });
  if (e != cudaSuccess) return e;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  conv_slab_kernel<KIND, BN><<<grid, kThreads, smem, s>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_conv_slab(const SlabConvParams& p, int dtype, int bn, int num_sms, cudaStream_t s) {
  const long long total = 1LL * p.tiles_w * p.tiles_h * p.tiles_n * p.groups * p.tiles_co;
  if (total == 0 || p.ntaps == 0) return cudaSuccess;
  if (total >= (1LL << 31)) return cudaErrorInvalidValue;
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
