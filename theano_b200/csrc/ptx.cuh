// Thin inline-PTX wrappers for the sm_100a features the convolution kernels use:
// mbarrier, TMA tiled loads (cp.async.bulk.tensor, no multicast), tcgen05 MMA with
// TMEM accumulators.  Every wait is bounded: a wait that runs out returns false and the
// caller records an error code instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Range-checked build (-DB200CONV_DEBUG): every global store of the tensor-core kernels, every
// tiled TMA store and every TMEM column range is checked against the extent the host passed; a
// violation writes kStatusBadIndex to the status word and the access is skipped (the host then
// fails the call).  The stand-in for a memory checker on machines where none may run.  In the
// normal build the macro is the constant true and costs nothing.
#ifdef B200CONV_DEBUG
#define B200_IN_RANGE(cond, status) ((cond) ? true : (atomicExch((status), 2 /* kStatusBadIndex */), false))
#else
#define B200_IN_RANGE(cond, status) (true)
#endif

// Upper bound on mbarrier polls before a kernel gives up (each poll may itself block
// for a hardware-defined time slice, so this is seconds, not microseconds).
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Nanoseconds of the GPU-wide timer (the same on every SM; for phase stamps that are compared
// across CTAs).
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false means the barrier never flipped.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Up to `polls` attempts as ONE opaque instruction block: the loop's branch is invisible to the
// compiler, so a warp that calls this with warp-uniform arguments stays convergent in the
// compiler's eyes and keeps its address arithmetic on the uniform datapath.  1 = phase completed.
__device__ __forceinline__ uint32_t mbar_spin(uint64_t* bar, uint32_t parity, uint32_t polls) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 n;\n\t"
      "mov.b32 n, %3;\n"
      "SPIN:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "@P bra DONE;\n\t"
      "sub.u32 n, n, 1;\n\t"
      "setp.ne.u32 P, n, 0;\n\t"
      "@P bra SPIN;\n"
      "DONE:\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(polls)
      : "memory");
  return ok;
}

// Default bound of a device-side wait, in SM clocks (about two seconds).
constexpr long long kDefaultWaitClocks = 4000000000LL;

// Wait of a whole, converged warp whose lanes all run the same loop (the MMA issuer and TMA producer
// warps: every lane follows the loop, one elected lane issues).  The result is made warp-uniform
// by a vote, so the caller's branch on it is a uniform branch.  BarsT has a `volatile int abort`
// that any waiter sets when its bound of `limit` clocks runs out; false = gave up.
template <class BarsT>
__device__ __forceinline__ bool uniform_wait(uint64_t* bar, uint32_t parity, BarsT* b, long long limit) {
  if (__all_sync(0xffffffffu, mbar_spin(bar, parity, 128))) return true;
  int ok = 1;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_spin(bar, parity, 32)) break;
    if (b->abort) { ok = 0; break; }
    if (clock64() - t0 > limit) { b->abort = 1; ok = 0; break; }
  }
  return __all_sync(0xffffffffu, ok) != 0;
}

// Abort path of the tensor-core kernels.  A role that gives up (its wait of `limit` clocks ran
// out) sets `abort`; every other role sees the flag at its next slow-path poll and stops issuing;
// all threads then meet at the kernel's closing __syncthreads.  TMA boxes requested earlier may
// still be on their way into this CTA's shared memory, and MMAs that were issued but whose commit
// nobody waited for may still be writing TMEM: the CTA therefore idles for a bounded grace period
// (a quarter of the wait limit) before it returns its TMEM and exits.  A copy or an MMA that has
// not finished by then will not finish at all (the limit is orders of magnitude above any
// latency), and the host reports B200CONV_E_TIMEOUT for the whole call anyway.
__device__ __forceinline__ void abort_grace(long long limit) {
  const long long t0 = clock64();
  while (clock64() - t0 < limit / 4) __nanosleep(1000);
}

// Warp index as a value the compiler knows to be the same in every lane.
__device__ __forceinline__ int uniform_warp_index() {
  return __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
}

// Wait of a whole warp on one barrier.  Lane 0 polls and sleeps between polls, the other lanes
// stay parked at the shuffle: hundreds of threads polling a barrier take shared-memory
// bandwidth and issue slots from the MMA operand reads and TMA writes that run meanwhile.
// Every lane then observes the completed phase itself (one poll) so that each has its own
// acquire.  All 32 lanes must call it.  BarsT has a `volatile int abort` that any waiter sets
// when its bound of `limit` clocks runs out; false = gave up.
template <class BarsT>
__device__ __forceinline__ bool warp_wait_or_abort(uint64_t* bar, uint32_t parity, BarsT* b, int lane,
                                                   long long limit) {
  int ok = 1;
  if (lane == 0 && !mbar_try_wait(bar, parity)) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
      if (mbar_try_wait(bar, parity)) break;
      __nanosleep(32);
      if ((i & 63) == 63) {
        if (b->abort) { ok = 0; break; }
        if (clock64() - t0 > limit) { b->abort = 1; ok = 0; break; }
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) ok = mbar_wait(bar, parity) ? 1 : 0;
  return ok != 0;
}

// ---- TMA ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(c4)
      : "memory");
}

// ---- CTA pairs (cta_group::2) ------------------------------------------------------------
// Two CTAs of a cluster work as one MMA unit: each holds 128 rows of A and half of B in its own shared
// memory, one thread of the even CTA issues MMAs of M = 256 for both, and each CTA's TMEM receives its
// 128 accumulator rows.  Barriers of the even CTA are addressed from the odd one by clearing the
// rank bit of the shared-memory address (the two CTAs' windows differ in that bit only).
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA loads of a CTA pair: the bytes are counted on the barrier at the same offset in the even CTA.
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                                 int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(c4)
      : "memory");
}
// Arrive on the barrier at this offset in the even CTA of the pair (from either CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerBitMask)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Shared-memory address of the same offset in the CTA of rank `rank` of this cluster.
__device__ __forceinline__ uint32_t cluster_smem_addr(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// Arrive, once every MMA issued so far by this thread has completed, on the barrier at this offset in
// both CTAs of the pair: two commits, one per CTA (issued by the even CTA's MMA thread).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   cluster_smem_addr(bar, 0))
               : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   cluster_smem_addr(bar, 1))
               : "memory");
}
__device__ __forceinline__ void umma_words_pair_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Tiled TMA store shared -> global of one 4-D box (asynchronous; tracked by the bulk groups of the
// issuing thread like the plain bulk store below).  Out-of-range parts of the box are not written.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* ssrc, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(ssrc)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Barrier among `nthreads` threads (a multiple of 32) of the CTA; id 1..15 (0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Bulk copy shared -> global (asynchronous, tracked by bulk groups of the issuing thread).
// Addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still read their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy (TMA / bulk copies).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM -----------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
enum class MmaKind { TF32, F16 };
template <MmaKind kind>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                     uint32_t idesc, uint32_t accumulate) {
  if (kind == MmaKind::TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// The same MMA with the two descriptors given as 32-bit halves.  Between the MMAs of a main loop
// only the address field (low word) changes, and the issuing thread is the bottleneck of a
// kernel as soon as it spends more clocks per MMA than the tensor pipe (a dependent instruction
// of a lone thread issues every 5 clocks or so, a taken branch costs tens): callers keep the
// loop bodies straight-line and pass  lo = (low word of the layout bits) + (address >> 4).
template <MmaKind kind>
__device__ __forceinline__ void umma_words(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                           uint32_t idesc, uint32_t accumulate) {
  if (kind == MmaKind::TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base+t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors --------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14), leading
// byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48),
// swizzle mode in [61,64).
constexpr uint64_t kSwizzle128 = 2;        // 16-byte chunks swizzled within 128 bytes
constexpr uint64_t kSwizzle128Base32 = 1;  // 32-byte chunks swizzled within 128 bytes: the only
                                           // swizzled form the MMA accepts for MN-major tf32
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint64_t layout = kSwizzle128) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= layout << 61;
  return d;
}
// Same for an operand whose first row is not on a 1024-byte boundary of the swizzle pattern
// (a row offset into a larger swizzled slab): bits [49,52) carry the phase, (address >> 7) & 7.
__device__ __forceinline__ uint64_t smem_desc_offset(uint32_t saddr, uint32_t lbo_bytes,
                                                     uint32_t sbo_bytes) {
  return smem_desc(saddr, lbo_bytes, sbo_bytes) | (static_cast<uint64_t>((saddr >> 7) & 7) << 49);
}
// Instruction descriptor (32 bit): D format f32 (1) in [4,6); A/B format in [7,10)/[10,13)
// (0 = f16, 2 = tf32); A/B major in bits 15/16 (0 = K-major, 1 = MN-major); N >> 3 in
// [17,23); M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t instr_desc(bool tf32, bool a_mn_major, bool b_mn_major,
                                                  uint32_t m, uint32_t n) {
  return (1u << 4) | ((tf32 ? 2u : 0u) << 7) | ((tf32 ? 2u : 0u) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

}  // namespace b200
