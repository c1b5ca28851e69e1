// C ABI of libb200conv: context, pooled device memory, geometry checks, tensor-map
// construction and the orchestration of the three convolution directions.
#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <thread>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "internal.h"

using namespace b200;

// ======================================================================================
// context
// ======================================================================================
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

std::mutex g_create_mu;
std::string g_create_err;

}  // namespace

// A captured sequence of calls.  Temporaries that the calls took from the pool while they were
// captured stay reserved for the graph until it is destroyed (the replays use their addresses).
struct b200conv_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  std::vector<void*> retained;
  long long launches = 0;   // kernels in the graph
};

// Host staging for the host-pointer calls.  A pageable array travels over PCIe at the speed of
// the driver's own staging copy (a single thread); here the array is cut into chunks that a few
// threads copy into (out of) pinned buffers while the DMA engine moves the previous chunk, so the
// link sees pinned transfers and the host side is copied in parallel.
class CopyPool {
 public:
  explicit CopyPool(int nthreads) {
    for (int i = 0; i < nthreads; ++i) workers_.emplace_back([this, i, nthreads] { loop(i, nthreads); });
  }
  ~CopyPool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  // memcpy(dst, src, bytes), cut into one slice per worker; returns when all of it is copied
  void copy(void* dst, const void* src, size_t bytes) {
    std::unique_lock<std::mutex> g(mu_);
    dst_ = static_cast<char*>(dst); src_ = static_cast<const char*>(src); bytes_ = bytes;
    pending_ = static_cast<int>(workers_.size());
    ++generation_;
    cv_.notify_all();
    done_.wait(g, [this] { return pending_ == 0; });
  }

 private:
  void loop(int index, int nthreads) {
    unsigned long long seen = 0;
    for (;;) {
      char* d; const char* s_; size_t n;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [&] { return stop_ || generation_ != seen; });
        if (stop_) return;
        seen = generation_;
        d = dst_; s_ = src_; n = bytes_;
      }
      const size_t per = (n / nthreads + 63) & ~static_cast<size_t>(63);
      const size_t a = std::min(n, per * index), b = index == nthreads - 1 ? n : std::min(n, per * (index + 1));
      if (b > a) memcpy(d + a, s_ + a, b - a);
      {
        std::lock_guard<std::mutex> g(mu_);
        if (--pending_ == 0) done_.notify_all();
      }
    }
  }
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_, done_;
  char* dst_ = nullptr; const char* src_ = nullptr; size_t bytes_ = 0;
  int pending_ = 0;
  unsigned long long generation_ = 0;
  bool stop_ = false;
};

constexpr size_t kStageChunk = 16u << 20;      // bytes per pinned staging buffer
constexpr size_t kStageMinBytes = 4u << 20;    // smaller arrays go the driver's way
constexpr int kStageBuffers = 2;

struct b200conv_ctx {
  int device = 0;
  int num_sms = 148;                         // SMs the persistent kernels spread over (b200conv_set_sm_count)
  int device_sms = 148;
  cudaStream_t stream = nullptr;
  std::mutex mu;
  std::string err;
  int* d_status = nullptr;
  int* h_status = nullptr;  // pinned
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  cudaEvent_t ev_tune0 = nullptr, ev_tune1 = nullptr;   // kernel selection timing
  long long launches = 0;
  const char* last_algo = "none";
  // optional per-kernel timing: an event pair around every launch of our own kernels
  bool prof = false;
  struct ProfRec { int kind; cudaEvent_t a, b; };
  std::vector<ProfRec> prof_recs;
  std::vector<cudaEvent_t> prof_pool;
  EncodeTiledFn encode = nullptr;
  // pooled device memory: free blocks by size, live blocks by address
  std::multimap<size_t, void*> free_blocks;
  std::map<void*, size_t> live;
  size_t pool_bytes = 0;
  void* l2buf = nullptr;
  size_t l2bytes = 0;
  // NCCL (loaded on demand)
  void* nccl_lib = nullptr;
  void* comm = nullptr;
  int nranks = 1, rank = 0;
  float* d_token = nullptr;
  cudaStream_t comm_stream = nullptr;       // collectives that overlap later convolutions
  cudaEvent_t ev_comm_ready = nullptr, ev_comm_done = nullptr;
  cudaStream_t up_stream = nullptr, down_stream = nullptr;   // background copies (PCIe is full duplex)
  cudaEvent_t ev_up = nullptr, ev_down = nullptr;
  bool down_pending = false;
  bool comm_pending = false;
  long long* trace = nullptr;               // debug: phase stamps of the slab kernel
  ConvEpilogue epi = default_epilogue();    // epilogue of the forward call in progress
  // forward / gradInputs kernel choice per geometry (true = slab kernel), filled by timing
  std::map<std::string, bool> algo_cache;
  // gradWeights split-K slice count per geometry and kernel, chosen by timing
  std::map<std::string, int> split_cache;
  int force_splits = 0;                     // > 0: use this slice count (tests, tuning by hand)
  bool use_pair = true;                     // 1x1 layers with deep reductions on CTA pairs (gemm_pair.cu)
  bool stack_taps = true;                   // grouped gradWeights of narrow layers: taps as column groups of one MMA
  bool autotune = true;
  // CUDA-graph capture of a sequence of calls (b200conv_graph_*)
  b200conv_graph* capturing = nullptr;
  long long graph_launch_count = 0;
  long long wait_clocks = 4000000000LL;     // bound of device-side waits (about two seconds)
  int comm_timeout_ms = 60000;              // host watchdog of streams that carry collectives
  // pinned staging of the host-pointer calls (made on first use)
  void* stage_buf[kStageBuffers] = {nullptr, nullptr};
  cudaEvent_t stage_ev[kStageBuffers] = {nullptr, nullptr};
  bool stage_busy[kStageBuffers] = {false, false};
  CopyPool* copy_pool = nullptr;
  // packed filters made ahead of time (b200conv_prepack): key -> device buffer and validity
  struct Packed { void* ptr; size_t bytes; bool valid; const void* src; };
  std::map<std::string, Packed> packed;
};

namespace {

int fail(b200conv_ctx* c, int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (c) c->err = buf;
  return code;
}

#define CU_OK(c, expr)                                                                      \
  do {                                                                                      \
    cudaError_t e_ = (expr);                                                                \
    if (e_ != cudaSuccess)                                                                  \
      return fail((c), e_ == cudaErrorMemoryAllocation ? B200CONV_E_NOMEM : B200CONV_E_CUDA, \
                  "%s: %s", #expr, cudaGetErrorString(e_));                                 \
  } while (0)

// Kernel families, for the launch counter and the optional per-kernel timing.
enum { kKConvUmma = 0, kKWgradUmma, kKWgradReduce, kKTranspose, kKPack, kKDirect, kKPool, kKCount };
const char* const kKernelNames[kKCount] = {"conv_umma", "wgrad_umma", "wgrad_reduce", "transpose",
                                           "pack", "direct", "pool"};

cudaEvent_t prof_event(b200conv_ctx* c) {
  cudaEvent_t e = nullptr;
  if (!c->prof_pool.empty()) {
    e = c->prof_pool.back();
    c->prof_pool.pop_back();
  } else {
    cudaEventCreate(&e);
  }
  return e;
}

#define KLAUNCH(c, kind, expr)                                  \
  do {                                                          \
    cudaEvent_t ea_ = nullptr, eb_ = nullptr;                   \
    const bool prof_ = (c)->prof && !(c)->capturing;            \
    if (prof_) {                                                \
      ea_ = prof_event(c);                                      \
      eb_ = prof_event(c);                                      \
      cudaEventRecord(ea_, (c)->stream);                        \
    }                                                           \
    CU_OK(c, expr);                                             \
    (c)->launches++;                                            \
    if ((c)->capturing) (c)->capturing->launches++;             \
    if (prof_) {                                                \
      cudaEventRecord(eb_, (c)->stream);                        \
      (c)->prof_recs.push_back({kind, ea_, eb_});               \
    }                                                           \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// ---- pooled allocator: blocks are recycled without returning to the driver; safe because
// every use is ordered on the context's single stream --------------------------------------
int pool_alloc(b200conv_ctx* c, size_t bytes, void** out) {
  if (bytes == 0) bytes = 256;
  bytes = (bytes + 255) & ~static_cast<size_t>(255);
  auto it = c->free_blocks.lower_bound(bytes);
  if (it != c->free_blocks.end() && it->first <= bytes + bytes / 4 + (1 << 20)) {
    *out = it->second;
    c->live[*out] = it->first;
    c->free_blocks.erase(it);
    return 0;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    // give cached blocks back to the driver and retry once
    cudaGetLastError();
    cudaStreamSynchronize(c->stream);
    for (auto& kv : c->free_blocks) {
      cudaFree(kv.second);
      c->pool_bytes -= kv.first;
    }
    c->free_blocks.clear();
    e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(c, B200CONV_E_NOMEM, "device allocation of %zu bytes failed: %s", bytes,
                  cudaGetErrorString(e));
    }
  }
  c->pool_bytes += bytes;
  c->live[p] = bytes;
  *out = p;
  return 0;
}

int pool_free(b200conv_ctx* c, void* p) {
  if (!p) return 0;
  auto it = c->live.find(p);
  if (it == c->live.end()) return fail(c, B200CONV_E_INVALID, "free of unknown device pointer %p", p);
  c->free_blocks.insert({it->second, p});
  c->live.erase(it);
  return 0;
}

// Temporaries of one call: returned to the pool when the call ends.
struct Scratch {
  b200conv_ctx* c;
  std::vector<void*> ptrs;
  explicit Scratch(b200conv_ctx* ctx) : c(ctx) {}
  ~Scratch() {
    for (void* p : ptrs) {
      if (c->capturing) c->capturing->retained.push_back(p);   // replays keep using it
      else pool_free(c, p);
    }
  }
  int get(size_t bytes, void** out) {
    int rc = pool_alloc(c, bytes, out);
    if (rc == 0) ptrs.push_back(*out);
    return rc;
  }
};

int check_status(b200conv_ctx* c) {
  // called after a stream synchronisation
  const int st = *c->h_status;
  if (st != kStatusOk) {
    *c->h_status = 0;
    cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream);
    if (st == kStatusBadIndex)
      return fail(c, B200CONV_E_CUDA, "a kernel of the range-checked build computed an index outside its buffer "
                  "(the access was skipped); results are invalid");
    return fail(c, B200CONV_E_TIMEOUT, "a device-side wait ran out (status %d); results are invalid", st);
  }
  return 0;
}

// Orders the main stream after a collective that was started on the communication stream.
int join_comm(b200conv_ctx* c) {
  if (c->comm_pending) {
    CU_OK(c, cudaStreamWaitEvent(c->stream, c->ev_comm_done, 0));
    c->comm_pending = false;
  }
  return 0;
}

// Waits for the context's stream.  With a communicator the wait is a host watchdog: a rank whose
// peers have gone would otherwise block for ever inside the collective.  The stream is polled
// together with the communicator's asynchronous error state; on an error, or when the deadline
// passes, the communicator is aborted (its kernels then leave the GPU) and the call fails with
// B200CONV_E_NCCL.  The context stays usable for single-GPU work; a new communicator needs a new
// b200conv_nccl_init on every surviving rank.
int wait_stream(b200conv_ctx* c) {
  if (!c->comm) {
    CU_OK(c, cudaStreamSynchronize(c->stream));
    return 0;
  }
  typedef int (*async_err_fn)(void*, int*);
  typedef int (*abort_fn)(void*);
  async_err_fn get_err = (async_err_fn)dlsym(c->nccl_lib, "ncclCommGetAsyncError");
  abort_fn do_abort = (abort_fn)dlsym(c->nccl_lib, "ncclCommAbort");
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(c->comm_timeout_ms);
  const char* why = nullptr;
  int nccl_state = 0;
  for (;;) {
    cudaError_t q = cudaStreamQuery(c->stream);
    if (q == cudaSuccess) return 0;
    if (q != cudaErrorNotReady) return fail(c, B200CONV_E_CUDA, "cudaStreamQuery: %s", cudaGetErrorString(q));
    if (get_err && get_err(c->comm, &nccl_state) == 0 && nccl_state != 0 && nccl_state != 7) {   // 0 ok, 7 in progress
      why = "the communicator reported an asynchronous error";
      break;
    }
    if (std::chrono::steady_clock::now() > deadline) {
      why = "a collective did not finish before the deadline";
      break;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
  if (do_abort) do_abort(c->comm);
  c->comm = nullptr;
  c->comm_pending = false;
  cudaStreamSynchronize(c->stream);              // the aborted collective's kernels have left by now
  cudaGetLastError();
  return fail(c, B200CONV_E_NCCL, "%s (NCCL state %d, watchdog %d ms): communicator aborted", why, nccl_state,
              c->comm_timeout_ms);
}

int sync_and_check(b200conv_ctx* c) {
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  int rcj = join_comm(c);
  if (rcj) return rcj;
  CU_OK(c, cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  if ((rcj = wait_stream(c))) return rcj;
  if (c->down_pending) {            // background downloads end after the work they waited for
    CU_OK(c, cudaStreamSynchronize(c->down_stream));
    c->down_pending = false;
  }
  return check_status(c);
}

// ======================================================================================
// geometry
// ======================================================================================
int floordiv(int x, int y) {
  int q = x / y;
  if ((x % y != 0) && ((x < 0) != (y < 0))) --q;
  return q;
}
int pymod(int x, int y) { return x - floordiv(x, y) * y; }

int validate(b200conv_ctx* c, const b200conv_desc* d) {
  if (!d) return fail(c, B200CONV_E_INVALID, "null descriptor");
  if (d->dtype != B200CONV_F32 && d->dtype != B200CONV_F16)
    return fail(c, B200CONV_E_INVALID, "dtype must be float32 or float16");
  if (d->N < 0 || d->C < 0 || d->K < 0 || d->H <= 0 || d->W <= 0 || d->kH <= 0 || d->kW <= 0)
    return fail(c, B200CONV_E_INVALID, "negative or empty dimension");
  if (d->sH < 1 || d->sW < 1 || d->dilH < 1 || d->dilW < 1 || d->groups < 1)
    return fail(c, B200CONV_E_INVALID, "subsample, dilation and groups must be >= 1");
  if (d->padH_l < 0 || d->padH_r < 0 || d->padW_l < 0 || d->padW_r < 0)
    return fail(c, B200CONV_E_INVALID, "pads must be resolved (>= 0)");
  if (d->C % d->groups)
    return fail(c, B200CONV_E_INVALID, "images and kernel must have the same stack size "
                "(channels %d not divisible by groups %d)", d->C, d->groups);
  if (d->K % d->groups)
    return fail(c, B200CONV_E_INVALID, "the number of filters must be divisible by the number of groups");
  const int Ho = floordiv(d->H + d->padH_l + d->padH_r - ((d->kH - 1) * d->dilH + 1), d->sH) + 1;
  const int Wo = floordiv(d->W + d->padW_l + d->padW_r - ((d->kW - 1) * d->dilW + 1), d->sW) + 1;
  if (Ho != d->Ho || Wo != d->Wo || Ho <= 0 || Wo <= 0)
    return fail(c, B200CONV_E_INVALID,
                "shape inconsistency: bottom %d %d %d %d, weight %d %d %d %d, top %d %d %d %d "
                "(expected %d %d %d %d)",
                d->N, d->C, d->H, d->W, d->K, d->C / d->groups, d->kH, d->kW, d->N, d->K, d->Ho,
                d->Wo, d->N, d->K, Ho, Wo);
  return 0;
}

// Pixel tile for a grid of Wt x Ht x N positions holding at most `cap` rows: fewest tiles,
// each tile weighted by the MMA steps it costs (`kk` rows per step); widest box on ties.
void choose_tile(int Wt, int Ht, int N, int cap, int kk, int* bw, int* bh, int* bn) {
  long long best = -1;
  *bw = *bh = *bn = 1;
  for (int w = 1; w <= std::min(Wt, cap); ++w) {
    for (int h = 1; h <= std::min(Ht, cap / w); ++h) {
      const int n = std::max(1, std::min(N, cap / (w * h)));
      const long long tiles = cdiv(Wt, w) * cdiv(Ht, h) * cdiv(N, n);
      const long long cost = tiles * (kk > 0 ? cdiv(w * h * n, kk) : 1);
      if (best < 0 || cost < best || (cost == best && w > *bw)) {
        best = cost;
        *bw = w; *bh = h; *bn = n;
      }
    }
  }
}

// 5-D channels-last view (c_in_group, group, w, h, n) of a [N][Hs][Ws][Cp] tensor that keeps
// every sH-th row and sW-th column starting at (rh, rw).
int make_view(b200conv_ctx* c, CUtensorMap* m, const void* base, int dtype, int Cg, int groups,
              int Cp, int Ws, int Hs, int N, int rh, int rw, int sH, int sW, int box_c, int bw,
              int bh, int bn, bool swizzle_32b_atoms = false) {
  const size_t es = elem_size(dtype);
  const int W2 = rw < Ws ? (Ws - rw + sW - 1) / sW : 0, H2 = rh < Hs ? (Hs - rh + sH - 1) / sH : 0;
  if (W2 <= 0 || H2 <= 0 || N <= 0 || Cg <= 0) return fail(c, B200CONV_E_INVALID, "empty view");
  cuuint64_t dims[5] = {(cuuint64_t)Cg, (cuuint64_t)groups, (cuuint64_t)W2, (cuuint64_t)H2, (cuuint64_t)N};
  cuuint64_t strides[4] = {(cuuint64_t)(groups > 1 ? Cg : Cp) * es, (cuuint64_t)sW * Cp * es,
                           (cuuint64_t)sH * Ws * Cp * es, (cuuint64_t)Hs * Ws * Cp * es};
  cuuint32_t box[5] = {(cuuint32_t)box_c, 1, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < 4; ++i)
    if (strides[i] % 16) return fail(c, B200CONV_E_UNSUPPORTED, "view stride %d not 16-byte aligned", i);
  const char* p = static_cast<const char*>(base) + (1LL * rh * Ws + rw) * Cp * es;
  if (reinterpret_cast<uintptr_t>(p) % 16) return fail(c, B200CONV_E_UNSUPPORTED, "view base not 16-byte aligned");
  CUresult r = c->encode(m, dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                         5, const_cast<char*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle_32b_atoms ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, B200CONV_E_CUDA, "cuTensorMapEncodeTiled(view) failed: %d", (int)r);
  return 0;
}

// 3-D map over packed filters [mats][rows][ldc]: (cols, rows, mats), box (box_c, box_r, 1).
int make_wmap(b200conv_ctx* c, CUtensorMap* m, const void* base, int dtype, int cols, int rows,
              int mats, int ldc, int box_c, int box_r) {
  const size_t es = elem_size(dtype);
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)mats};
  cuuint64_t strides[2] = {(cuuint64_t)ldc * es, (cuuint64_t)rows * ldc * es};
  cuuint32_t box[3] = {(cuuint32_t)box_c, (cuuint32_t)box_r, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = c->encode(m, dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                         3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, B200CONV_E_CUDA, "cuTensorMapEncodeTiled(filters) failed: %d", (int)r);
  return 0;
}

bool fits16(int v) { return v >= -32768 && v <= 32767; }

// Can the tensor-core kernels take this geometry?  (Otherwise the direct kernels do.)
bool umma_ok(const b200conv_desc& d) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const size_t es = elem_size(d.dtype);
  if (d.N == 0 || d.C == 0 || d.K == 0) return false;
  if (d.kH * d.kW > kMaxTaps) return false;
  if (d.sH * d.sW > kMaxViews) return false;
  if (d.groups > 1 && ((Cg * es) % 16 || (Kg * es) % 16)) return false;
  if (Cg * es < 16 && d.groups > 1) return false;
  // tap offsets travel as 16-bit numbers; pixel coordinates as 32-bit ones
  const int reach_h = (d.kH - 1) * d.dilH + d.padH_l, reach_w = (d.kW - 1) * d.dilW + d.padW_l;
  if (!fits16(reach_h) || !fits16(reach_w)) return false;
  if (1LL * d.H + reach_h > (1 << 30) || 1LL * d.W + reach_w > (1 << 30)) return false;
  return true;
}

// ---- forward-type launch shared by fwd and dgrad ------------------------------------------
struct FwdLikeArgs {
  const void* act;       // channels-last activations [N][Hs][Ws][Cp_in]
  int Hs, Ws, Cin_g, Cp_in;
  const void* wpacked;   // [(tap*groups+g)][n_out][ld_w]
  int ld_w, nmats;
  int n_out, groups, N;
  int dtype;
  int view_sH, view_sW;  // parity pitch of the activation views
  // Row folding (few input channels): `act` is [N][Hs][fold_Wp][Cp_in] with explicit zero columns;
  // the view's column index is the output column, its innermost extent runs over kW pixels x Cp_in
  // channels (Cin_g is that folded length) and only the filter rows remain as taps.
  bool fold = false;
  int fold_Wp = 0, fold_sW = 1;
};

// Folded activation view: (folded channel, 1, output column, input row of parity rh, image).
// Consecutive output columns start fold_sW pixels apart, so the rows of the view overlap in memory.
int make_fold_view(b200conv_ctx* c, CUtensorMap* m, const FwdLikeArgs& a, int rh, int sH, int box_c,
                   int bw, int bh, int bn) {
  const size_t es = elem_size(a.dtype);
  const int H2 = rh < a.Hs ? (a.Hs - rh + sH - 1) / sH : 0;
  if (H2 <= 0 || a.N <= 0) return fail(c, B200CONV_E_INVALID, "empty view");
  const size_t pix = (size_t)a.Cp_in * es, row = (size_t)a.fold_Wp * pix;
  cuuint64_t dims[5] = {(cuuint64_t)a.Cin_g, 1, (cuuint64_t)a.Ws, (cuuint64_t)H2, (cuuint64_t)a.N};
  cuuint64_t strides[4] = {row, (cuuint64_t)a.fold_sW * pix, (cuuint64_t)sH * row, (cuuint64_t)a.Hs * row};
  cuuint32_t box[5] = {(cuuint32_t)box_c, 1, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const char* p = static_cast<const char*>(a.act) + (size_t)rh * row;
  CUresult r = c->encode(m, a.dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                         5, const_cast<char*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(c, B200CONV_E_CUDA, "cuTensorMapEncodeTiled(folded view) failed: %d", (int)r);
  return 0;
}

int make_act_view(b200conv_ctx* c, CUtensorMap* m, const FwdLikeArgs& a, int rh, int rw, int box_c, int bw,
                  int bh, int bn) {
  if (a.fold) return make_fold_view(c, m, a, rh, a.view_sH, box_c, bw, bh, bn);
  return make_view(c, m, a.act, a.dtype, a.Cin_g, a.groups, a.Cp_in, a.Ws, a.Hs, a.N, rh, rw, a.view_sH,
                   a.view_sW, box_c, bw, bh, bn);
}

// One past the last element of `out` that a launch over a Wt x Ht x N pixel grid with these element
// strides may write (what the range-checked build compares every store index with).
long long out_extent(const FwdLikeArgs& a, int Wt, int Ht, long long sn, long long sc, long long sh, long long sw,
                     long long off) {
  return off + (a.N - 1) * sn + (Ht - 1) * sh + (Wt - 1) * sw + (1LL * a.n_out * a.groups - 1) * sc + 1;
}

// Slab variant (conv_slab.cu) for launches whose taps all read one view.  Returns 0 when it was
// launched, 2 when the geometry does not fit (the caller then uses the per-tap kernel), or an
// error code.
int try_conv_slab(b200conv_ctx* c, const FwdLikeArgs& a, const std::vector<ConvTap>& taps, int rh,
                  int rw, int Wt, int Ht, void* out, long long sn, long long sc, long long sh,
                  long long sw, long long off, const float* bias, int relu) {
  if (taps.empty() || (int)taps.size() > kMaxTaps) return 2;
  int dh_min = taps[0].dh, dh_max = taps[0].dh, dw_min = taps[0].dw, dw_max = taps[0].dw;
  for (const ConvTap& t : taps) {
    dh_min = std::min<int>(dh_min, t.dh); dh_max = std::max<int>(dh_max, t.dh);
    dw_min = std::min<int>(dw_min, t.dw); dw_max = std::max<int>(dw_max, t.dw);
  }
  const int Eh = dh_max - dh_min, Ew = dw_max - dw_min;
  const int kBK = a.dtype == B200CONV_F16 ? 64 : 32;
  int BN = conv_umma_bn(a.n_out);
#ifdef B200CONV_TUNE                       // development build: tile parameters from the environment
  if (getenv("B200_BN") && atoi(getenv("B200_BN")) <= BN) BN = atoi(getenv("B200_BN"));
#endif
  const int tiles_co = (int)cdiv(a.n_out, BN);
  const int acc_cap = std::min(512 / BN, 4);
  // Narrow tiles (few filters) have small filter tiles and short MMAs: several taps then share one
  // stage of the filter ring, so that a barrier round trip is paid per 16 to 32 KB of filters, not
  // per 4 or 8 KB (the issuing warp spends about 150 clocks per stage on the hand-over, as much as
  // the stage's MMAs take when a tap is four 128 x 64 MMAs)
  // (measured: 64 -> 64 3x3 layers 8 to 16 % faster with a filter row per stage, the 7x7 stem 8 to 16 % with four
  // taps; 128-filter tiles are better off with one tap per stage)
  const int ntap_all = (int)taps.size();
  int tps = BN <= 64 ? (ntap_all % 3 == 0 ? 3 : std::min(4, ntap_all)) : 1;
#ifdef B200CONV_TUNE
  if (getenv("B200_TPS")) tps = std::max(1, std::min({8, atoi(getenv("B200_TPS")), (int)taps.size()}));
#endif
  const int b_bytes = tps * BN * 128;
  // search the tile (wt x th x nb) with the least serial work per SM
  const int mma_clk = BN >= 256 ? 128 : BN == 128 ? 64 : BN == 64 ? 48 : 40;   // 128 x BN x 32-byte MMA
  const long long kblocks_n = cdiv(a.Cin_g, kBK);
  long long best_cost = -1, best_work = 0, best_tiles = 0;
  int b_wt = 0, b_th = 0, b_nb = 0, b_acc = 0, b_slab = 0;
  const long long es_out = (long long)elem_size(a.dtype);
  // can the output leave through tiled TMA stores at all (channels-last, whole 128-byte channel rows, aligned)?
  const bool tma_layout_ok = sc == 1 && a.n_out % (int)(128 / es_out) == 0 && !c->epi.residual &&
                             (sw * es_out) % 16 == 0 && (sh * es_out) % 16 == 0 && (sn * es_out) % 16 == 0 &&
                             reinterpret_cast<uintptr_t>(static_cast<const char*>(out) + off * es_out) % 16 == 0;
  for (int parts = 1; parts <= 16; ++parts) {
    const int wt = (int)cdiv(Wt, parts);
    if (parts > 1 && wt < 8) break;
    const int Ws = wt + Ew;
    if (Ws > 256) continue;
    const int shift_max = Eh * Ws + Ew;
    for (int th = 1; th <= Ht; ++th) {
      const int Hs = th + Eh;
      if (Hs > 256) break;
      const int per_img = Hs * Ws;
      if ((th - 1) * Ws + wt - 1 >= 128 * acc_cap) break;
      for (int nb = 1; nb <= std::min(a.N, 256); ++nb) {
        const long long last = 1LL * (nb - 1) * per_img + (th - 1) * Ws + (wt - 1);
        if (last >= 128LL * acc_cap) break;
        const int n_acc = (int)(last / 128) + 1;
        const long long rows = std::max<long long>(1LL * nb * per_img, 128LL * n_acc + shift_max);
        const long long slab_bytes = (rows * 128 + 1023) / 1024 * 1024;
        if (2 * slab_bytes + 2 * b_bytes > kSlabSmemBudget) break;
        const long long tiles = cdiv(Wt, wt) * cdiv(Ht, th) * cdiv(a.N, nb);
        const long long total = tiles * tiles_co * a.groups;
        // clocks of the busiest SM: per tile and (tap, channel block) 4 MMAs per accumulator plus
        // about 400 clocks of stage hand-over in the issuing thread
        // about 400 clocks of stage hand-over in the issuing thread; then the accumulators are read
        // out (about 1000 clocks per 128 x 32 block), beside the next tile's MMAs when two
        // accumulator sets fit the 512 TMEM columns
        // Epilogue: through staged TMA stores when the output is channels-last and the staging
        // buffers fit beside two slabs and two filter stages (about 2500 clocks of latency per tile
        // plus the tile's bytes at the SM's store rate of 32 B/clk), else lane-per-row stores from
        // registers (1200 to 2500 clocks per 128 x 32 block: 16-byte pieces scattered over the pixel rows)
        const long long dense_rows = 1LL * wt * th * nb;
        const int ngr = n_acc == 3 ? 0 : 4 / n_acc;
        const long long stg = (dense_rows * 128 + 1023) / 1024 * 1024;
        const long long min_b = std::min<long long>(3, kblocks_n * cdiv((long long)taps.size(), tps) + 1);   // filter stages the staged epilogue insists on
        if (c->epi.pool && ((wt | th) & 1)) continue;        // pooling windows must not straddle tiles
        const bool tma_fit = tma_layout_ok && ngr > 0 && ngr * stg <= kSlabStageBytes &&
                             (total <= c->num_sms ? ngr * stg <= 2 * slab_bytes + 2 * b_bytes
                                                  : 2 * slab_bytes + min_b * b_bytes + kSlabStageBytes <= kSlabSmemBudget);
        // plus about 1500 clocks per tile for the pipeline to fill again
        const long long mma_part = 1LL * kblocks_n * ((long long)taps.size() * 4LL * n_acc * mma_clk + cdiv((long long)taps.size(), tps) * 120) + 1500;
        if (c->epi.pool && !tma_fit) continue;               // pooling happens in the staged epilogue only
        const long long epi_part = tma_fit ? 2500 + dense_rows * BN * (long long)es_out / 32 : 2400LL * n_acc * (BN / 32);
        const long long per_tile = 2 * n_acc * BN <= 512 ? std::max(mma_part, epi_part) : mma_part + epi_part;
        const long long cost = cdiv(total, c->num_sms) * per_tile;
        const long long work = total * n_acc;
        if (best_cost < 0 || cost < best_cost || (cost == best_cost && work < best_work) ||
            (cost == best_cost && work == best_work && tiles < best_tiles)) {
          best_cost = cost; best_work = work; best_tiles = tiles;
          b_wt = wt; b_th = th; b_nb = nb; b_acc = n_acc; b_slab = (int)slab_bytes;
        }
      }
    }
  }
#ifndef B200_PAIR_MIN_KBLOCKS
#define B200_PAIR_MIN_KBLOCKS 4
#endif
  constexpr long long kPairMinKblocks = B200_PAIR_MIN_KBLOCKS;
  // Flattened 1x1 layers with a deep reduction and 256-filter tiles: pairs of CTAs share the filter tile
  // (each loads half of it), which brings the operand traffic from L2 under what an SM can take.
  if (best_cost < 0 && Eh == 0 && Ew == 0 && Ht == 1 && a.N == 1 && Wt > 256 && c->use_pair &&
      a.dtype == B200CONV_F16 && BN == 256 && a.n_out % 64 == 0 && a.groups == 1 && !a.fold && taps.size() == 1 &&
      kblocks_n >= kPairMinKblocks && tma_layout_ok && c->num_sms >= 2 && c->epi.beta == 0.f && !c->epi.pool) {
    PairGemmParams q;
    memset(&q, 0, sizeof q);
    int rc = make_act_view(c, &q.view, a, rh, rw, 64, 128, 1, 1);
    if (rc) return rc;
    if ((rc = make_wmap(c, &q.wmap, a.wpacked, a.dtype, a.Cin_g, a.n_out, a.nmats, a.ld_w, 64, 128))) return rc;
    cuuint64_t dims[4] = {(cuuint64_t)a.n_out, (cuuint64_t)Wt, 1, 1};
    cuuint64_t strides[3] = {(cuuint64_t)(sw * es_out), (cuuint64_t)(sh * es_out), (cuuint64_t)(sn * es_out)};
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = c->encode(&q.out_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                           const_cast<char*>(static_cast<const char*>(out) + off * es_out), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
      q.kblocks = (int)kblocks_n;
      q.tiles_pix = (int)cdiv(Wt, 256);
      q.tiles_co = (int)cdiv(a.n_out, 256);
      q.pixels = Wt; q.n_out = a.n_out;
      q.stages = 5;
      q.bias = bias; q.relu = relu; q.epi = c->epi;
      q.status = c->d_status;
      q.wait_clocks = c->wait_clocks;
      KLAUNCH(c, kKConvUmma, launch_gemm_pair(q, c->num_sms, c->stream));
      return 0;
    }
  }
  if (best_cost < 0 && Eh == 0 && Ew == 0 && Ht == 1 && a.N == 1 && Wt > 256 && !c->epi.pool) {
    // one long row of pixels without halo (a flattened 1x1 layer): whole 128-pixel accumulators,
    // as many as still leave room for a second accumulator set
    b_acc = BN >= 256 ? 1 : 2;
#ifdef B200CONV_TUNE
    if (getenv("B200_NACC")) b_acc = std::max(1, std::min(2, atoi(getenv("B200_NACC"))));
#endif
    b_wt = 128 * b_acc; b_th = 1; b_nb = 1;
    b_slab = b_wt * 128;
    best_cost = 0;
  }
  if (best_cost < 0) return 2;
  SlabConvParams p;
  memset(&p, 0, sizeof p);
  p.wt = b_wt; p.th = b_th; p.nb = b_nb; p.n_acc = b_acc;
  p.Ws = b_wt + Ew; p.Hs = b_th + Eh;
  p.dw_min = dw_min; p.dh_min = dh_min;
  p.slab_bytes = b_slab;
  p.tps = tps;
  // Ring depths for `avail` bytes.  Activations come from HBM (the longer latency, and the stream
  // that bounds most layers): the slab ring gets up to 6 buffers once the filter ring holds what
  // one tile consumes (2 to 4 stages); the filter ring then takes what is left, up to 8 stages.
  const int per_tile = (int)std::min<long long>(8, kblocks_n * cdiv((long long)taps.size(), tps));
  auto plan_rings = [&](long long avail, int* ss, int* bs) {
    if (2LL * b_slab + 2LL * b_bytes > avail) return false;
    const int fit = (int)std::min<long long>(8, (avail - 2LL * b_slab) / b_bytes);
    // a ring that holds exactly one tile's filters cannot start the next tile's filters before
    // this tile's MMAs are done: shallow reductions get one stage more than a tile consumes
    // (128 -> 512 1x1 forward: 100 -> 70 us with 3 instead of 2 stages)
    int b = std::min(fit, per_tile <= 2 ? per_tile + 1 : std::min(4, per_tile));
    const int s_ = (int)std::max<long long>(2, std::min<long long>(6, (avail - 1LL * b * b_bytes) / b_slab));
    b = (int)std::min<long long>(8, (avail - 1LL * s_ * b_slab) / b_bytes);
    *ss = s_; *bs = b;
#ifdef B200CONV_TUNE
    if (getenv("B200_SS") && getenv("B200_BS")) {
      const int es_ = atoi(getenv("B200_SS")), eb_ = atoi(getenv("B200_BS"));
      if (es_ >= 2 && es_ <= 6 && eb_ >= 2 && eb_ <= 8 && 1LL * es_ * b_slab + 1LL * eb_ * b_bytes <= avail) { *ss = es_; *bs = eb_; }
    }
#endif
    return true;
  };
  if (!plan_rings(kSlabSmemBudget, &p.s_stages, &p.b_stages)) return 2;
  {
    // TMA-store epilogue: channels-last output whose 128-byte channel chunks never straddle a
    // group, 1/2/4 accumulators (so that the 16 epilogue warps split into equal groups)
    const long long tiles = cdiv(Wt, p.wt) * cdiv(Ht, p.th) * cdiv(a.N, p.nb);
    const long long total = tiles * tiles_co * a.groups;
    const size_t es = elem_size(a.dtype);
    const long long dense_rows = 1LL * p.wt * p.th * p.nb;
    const int stage_bytes = (int)((dense_rows * 128 + 1023) / 1024 * 1024);
    const int ngroups = p.n_acc == 3 ? 0 : 4 / p.n_acc;
    const char* obase = static_cast<const char*>(out) + off * (long long)es;
    const int row_ch = (int)(128 / es);     // channels of one staged 128-byte row
    bool ok = sc == 1 && a.n_out % row_ch == 0 && ngroups > 0 && !c->epi.residual &&
              ngroups * stage_bytes <= kSlabStageBytes && p.wt <= 256 && p.th <= 256 && p.nb <= 256 &&
              (sw * es) % 16 == 0 && (sh * es) % 16 == 0 && (sn * es) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(obase) % 16 == 0;
    if (ok) {
      if (total <= c->num_sms) {
        p.stage_off = 0;                       // one tile per CTA: operands are dead by then
        p.stage_nbuf = std::min(8, (p.s_stages * b_slab + p.b_stages * b_bytes) / stage_bytes) / std::max(1, ngroups) * ngroups;
        ok = p.stage_nbuf >= ngroups;
      } else {
        int ss = 0, bs = 0;
        if (plan_rings(kSlabSmemBudget - kSlabStageBytes, &ss, &bs) && bs >= std::min(3, per_tile + 1)) {
          p.s_stages = ss;
          p.b_stages = bs;
          p.stage_off = ss * b_slab + bs * b_bytes;
          p.stage_reserved = kSlabStageBytes;
          p.stage_nbuf = kSlabStageBytes / stage_bytes / ngroups * ngroups;
        } else {
          ok = false;
        }
      }
    }
    if (c->epi.pool && !ok) return fail(c, B200CONV_E_UNSUPPORTED, "this geometry's epilogue cannot pool");
    if (ok) {
      const int pl = c->epi.pool ? 2 : 1;       // pooled output: half the rows and columns (strides are the pooled tensor's)
      cuuint64_t dims[4] = {(cuuint64_t)a.n_out * a.groups, (cuuint64_t)(Wt / pl), (cuuint64_t)(Ht / pl), (cuuint64_t)a.N};
      cuuint64_t strides[3] = {(cuuint64_t)(sw * es), (cuuint64_t)(sh * es), (cuuint64_t)(sn * es)};
      cuuint32_t box[4] = {(cuuint32_t)row_ch, (cuuint32_t)(p.wt / pl), (cuuint32_t)(p.th / pl), (cuuint32_t)p.nb};
      cuuint32_t estr[4] = {1, 1, 1, 1};
      CUresult r = c->encode(&p.out_map, a.dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                             4, const_cast<char*>(obase), dims, strides,
                             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r == CUDA_SUCCESS) {
        p.tma_out = 1;
        p.stage_bytes = stage_bytes;
      } else {
        if (c->epi.pool) return fail(c, B200CONV_E_UNSUPPORTED, "this geometry's epilogue cannot pool");
        plan_rings(kSlabSmemBudget, &p.s_stages, &p.b_stages);
        p.stage_off = p.stage_reserved = 0;
      }
    } else {
      p.stage_off = p.stage_reserved = 0;
    }
  }
  int rc = make_act_view(c, &p.view, a, rh, rw, kBK, p.Ws, p.Hs, p.nb);
  if (rc) return rc;
  rc = make_wmap(c, &p.wmap, a.wpacked, a.dtype, a.Cin_g, a.n_out, a.nmats, a.ld_w, kBK, BN);
  if (rc) return rc;
  for (const ConvTap& t : taps) {
    p.tap_shift[p.ntaps] = (int16_t)((t.dh - dh_min) * p.Ws + (t.dw - dw_min));
    p.tap_wmat[p.ntaps] = t.wmat;
    ++p.ntaps;
  }
  p.kblocks = (int)cdiv(a.Cin_g, kBK);
  p.groups = a.groups;
  p.Wt = Wt; p.Ht = Ht; p.Nimg = a.N;
  p.tiles_w = (int)cdiv(Wt, p.wt); p.tiles_h = (int)cdiv(Ht, p.th); p.tiles_n = (int)cdiv(a.N, p.nb);
  p.tiles_co = tiles_co;
  p.n_out = a.n_out;
  p.out = out; p.bias = bias;
  p.out_sn = sn; p.out_sc = sc; p.out_sh = sh; p.out_sw = sw; p.out_off = off;
  p.out_elems = out_extent(a, Wt, Ht, sn, sc, sh, sw, off);
  p.relu = relu;
  p.epi = c->epi;
  p.status = c->d_status;
  p.wait_clocks = c->wait_clocks;
  p.trace = c->trace;
#ifdef B200CONV_TUNE
  if (getenv("B200_VERBOSE"))
    fprintf(stderr, "slab: Wt %d Ht %d N %d Cin %d n_out %d taps %d | BN %d wt %d th %d nb %d n_acc %d slab %d s %d b %d tma %d nbuf %d cost %lld\n",
            Wt, Ht, a.N, a.Cin_g, a.n_out, (int)taps.size(), BN, p.wt, p.th, p.nb, p.n_acc, p.slab_bytes, p.s_stages, p.b_stages,
            p.tma_out, p.stage_nbuf, best_cost);
#endif
  KLAUNCH(c, kKConvUmma, launch_conv_slab(p, a.dtype, BN, c->num_sms, c->stream));
  return 0;
}

int run_conv_umma_one(b200conv_ctx* c, const FwdLikeArgs& a, const std::vector<ConvTap>& taps_in,
                      const std::vector<std::pair<int, int>>& view_parity, int Wt, int Ht, void* out,
                      long long sn, long long sc, long long sh, long long sw, long long off,
                      const float* bias, int relu, bool allow_slab) {
  if (allow_slab && view_parity.size() == 1) {
    const int rh = view_parity[0].first, rw = view_parity[0].second;
    if (rh < a.Hs && rw < a.Ws) {
      const int rc = try_conv_slab(c, a, taps_in, rh, rw, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu);
      if (rc != 2) return rc;
    }
  }
  UmmaConvParams p;
  memset(&p, 0, sizeof p);
  const int kBK = a.dtype == B200CONV_F16 ? 64 : 32;
  choose_tile(Wt, Ht, a.N, 128, 0, &p.bw, &p.bh, &p.bn);
  // views that exist (non-empty); taps pointing at empty views contribute nothing
  std::vector<int> remap(view_parity.size(), -1);
  int nviews = 0;
  for (size_t v = 0; v < view_parity.size(); ++v) {
    const int rh = view_parity[v].first, rw = view_parity[v].second;
    if (rh >= a.Hs || rw >= a.Ws) continue;
    int rc = make_act_view(c, &p.views[nviews], a, rh, rw, kBK, p.bw, p.bh, p.bn);
    if (rc) return rc;
    remap[v] = nviews++;
  }
  for (const ConvTap& t : taps_in) {
    if (remap[t.view] < 0) continue;
    ConvTap u = t;
    u.view = static_cast<int16_t>(remap[t.view]);
    p.taps[p.ntaps++] = u;
  }
  if (p.ntaps == 0) return 1;  // caller zero-fills
  for (int v = nviews; v < kMaxViews; ++v) p.views[v] = p.views[0];
  const int BN = conv_umma_bn(a.n_out);
  int rc = make_wmap(c, &p.wmap, a.wpacked, a.dtype, a.Cin_g, a.n_out, a.nmats, a.ld_w, kBK, BN);
  if (rc) return rc;
  p.kblocks = static_cast<int>(cdiv(a.Cin_g, kBK));
  p.groups = a.groups;
  p.Wt = Wt; p.Ht = Ht; p.Nimg = a.N;
  p.tiles_w = static_cast<int>(cdiv(Wt, p.bw));
  p.tiles_h = static_cast<int>(cdiv(Ht, p.bh));
  p.tiles_n = static_cast<int>(cdiv(a.N, p.bn));
  p.tiles_co = static_cast<int>(cdiv(a.n_out, BN));
  p.n_out = a.n_out;
  p.out = out; p.bias = bias;
  p.out_sn = sn; p.out_sc = sc; p.out_sh = sh; p.out_sw = sw; p.out_off = off;
  p.out_elems = out_extent(a, Wt, Ht, sn, sc, sh, sw, off);
  p.relu = relu;
  p.epi = c->epi;
  p.status = c->d_status;
  p.wait_clocks = c->wait_clocks;
  KLAUNCH(c, kKConvUmma, launch_conv_umma(p, a.dtype, c->num_sms, c->stream));
  return 0;
}

// Picks between the slab kernel and the per-tap kernel.  Both compute the same thing; which one
// is faster depends on the layer (halo rows wasted by the slab grid against activations fetched
// once per tap), so the first call of a geometry times both with CUDA events and the context
// remembers the winner (the reference's GPU path selects its convolution algorithm the same way,
// theano/gpuarray/opt.py:2144-2222).  While a graph is being captured the remembered choice, or
// the slab kernel, is used.
int run_conv_umma(b200conv_ctx* c, const FwdLikeArgs& a, const std::vector<ConvTap>& taps_in,
                  const std::vector<std::pair<int, int>>& view_parity, int Wt, int Ht, void* out,
                  long long sn, long long sc, long long sh, long long sw, long long off,
                  const float* bias, int relu, bool allow_slab = true) {
  if (c->epi.pool) {                  // only the slab kernel's staged epilogue pools
    if (!allow_slab || view_parity.size() != 1) return fail(c, B200CONV_E_UNSUPPORTED, "this geometry's epilogue cannot pool");
    const int rh = view_parity[0].first, rw = view_parity[0].second;
    const int rc = try_conv_slab(c, a, taps_in, rh, rw, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu);
    return rc == 2 ? fail(c, B200CONV_E_UNSUPPORTED, "this geometry's epilogue cannot pool") : rc;
  }
  if (!allow_slab || view_parity.size() != 1 || !c->autotune)
    return run_conv_umma_one(c, a, taps_in, view_parity, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu, allow_slab);
  char key[256];
  int tsum = 0;
  for (const ConvTap& t : taps_in) tsum = tsum * 31 + t.dh * 7 + t.dw;
  snprintf(key, sizeof key, "%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%zu.%d.%lld.%lld", a.dtype, a.N, a.Hs, a.Ws,
           a.Cin_g, a.n_out, a.groups, Wt, Ht, a.view_sH, a.view_sW, taps_in.size(), tsum, sc, sw);
  auto it = c->algo_cache.find(key);
  if (it != c->algo_cache.end())
    return run_conv_umma_one(c, a, taps_in, view_parity, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu, it->second);
  if (c->capturing)
    return run_conv_umma_one(c, a, taps_in, view_parity, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu, true);
  float ms[2] = {0.f, 0.f};
  if (!c->ev_tune0) {
    CU_OK(c, cudaEventCreate(&c->ev_tune0));
    CU_OK(c, cudaEventCreate(&c->ev_tune1));
  }
  for (int variant = 0; variant < 2; ++variant) {        // 0: per tap, 1: slab; two runs each, keep the second
    for (int rep = 0; rep < 2; ++rep) {
      CU_OK(c, cudaEventRecord(c->ev_tune0, c->stream));
      int rc = run_conv_umma_one(c, a, taps_in, view_parity, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu, variant == 1);
      if (rc) return rc;
      CU_OK(c, cudaEventRecord(c->ev_tune1, c->stream));
      CU_OK(c, cudaStreamSynchronize(c->stream));
      CU_OK(c, cudaEventElapsedTime(&ms[variant], c->ev_tune0, c->ev_tune1));
    }
  }
  const bool slab = ms[1] <= ms[0];
  c->algo_cache[key] = slab;
  if (!slab)   // the last run was the slab kernel: leave the output of the chosen kernel (identical up to rounding order)
    return run_conv_umma_one(c, a, taps_in, view_parity, Wt, Ht, out, sn, sc, sh, sw, off, bias, relu, false);
  return 0;
}

int to_nhwc(b200conv_ctx* c, Scratch& tmp, const void* src, int N, int C, int H, int W, int dtype,
            const void** out) {
  const int Cp = pad_channels(C, dtype);
  void* buf;
  int rc = tmp.get(elem_size(dtype) * (size_t)N * H * W * Cp, &buf);
  if (rc) return rc;
  KLAUNCH(c, kKTranspose, launch_transpose(src, buf, N, C, H * W, H * W, Cp, dtype, c->stream));
  *out = buf;
  return 0;
}

// Grouped layers with fewer channels per group than one reduction block: how many neighbouring
// groups to merge into one (block-diagonal filters); 1 = leave as is.
int merge_factor(const b200conv_desc& d) {
  if (d.groups <= 1 || d.C == 0 || d.K == 0) return 1;
  const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  int best = 1;
  for (int m = 2; m <= d.groups && Cg * m <= kBK && Kg * m <= 256; ++m)
    if (d.groups % m == 0) best = m;
  return best;
}

// Row folding applies to ungrouped layers whose whole filter row (kW pixels x padded channels)
// fits one reduction block of the MMA: the 3-channel stems of VGG and ResNet.
bool fold_ok(const b200conv_desc& d) {
  const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
  const int Cp = pad_channels(d.C, d.dtype);
  return d.groups == 1 && d.dilW == 1 && d.kW > 1 && Cp * d.kW <= kBK && Cp * 2 <= kBK && d.kH <= kMaxTaps &&
         d.sH <= kMaxViews && d.N > 0 && d.C > 0 && d.K > 0;
}
// Padded row length: left pad, the image, and enough zero columns on the right for the last
// output's kBK / Cp pixels.
int fold_width(const b200conv_desc& d) {
  const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
  const int Cp = pad_channels(d.C, d.dtype);
  return std::max(d.padW_l + d.W + d.padW_r, (d.Wo - 1) * d.sW + kBK / Cp);
}

// Space-to-depth applies to ungrouped stride-2 layers with at most 4 input channels whose filter
// rows span at most kS2dPixels blocks of 2 x 2 pixels: the 7x7 stride-2 stem of ResNet.  t0 / q0:
// first block row / column a filter touches relative to the output position; ntaps: block rows.
bool s2d_ok(const b200conv_desc& d, int* t0, int* ntaps, int* q0) {
  if (d.groups != 1 || d.sH != 2 || d.sW != 2 || d.dilH != 1 || d.dilW != 1) return false;
  if (d.N <= 0 || d.C <= 0 || d.K <= 0 || 4 * d.C > kS2dChannels) return false;
  *t0 = floordiv(-d.padH_l, 2);
  *q0 = floordiv(-d.padW_l, 2);
  *ntaps = floordiv(d.kH - 1 - d.padH_l, 2) - *t0 + 1;
  const int span = floordiv(d.kW - 1 - d.padW_l, 2) - *q0 + 1;
  return span >= 1 && span <= kS2dPixels && *ntaps >= 1 && *ntaps <= kMaxTaps;
}

// A 1x1, stride-1, unpadded convolution on channels-last tensors is a plain matrix product over
// the N*H*W pixels.  Seen as ONE image of one row of N*H*W pixels it tiles into whole 128-pixel
// tiles, where tiles cut from 56x56, 28x28, 14x14 or 7x7 images leave 12 to 25 % of the
// accumulator rows empty.
bool flatten_1x1(const b200conv_desc& d, bool all_nhwc, b200conv_desc* f) {
  if (!all_nhwc || d.kH != 1 || d.kW != 1 || d.sH != 1 || d.sW != 1) return false;
  if (d.padH_l | d.padH_r | d.padW_l | d.padW_r) return false;
  if (d.N == 1 && d.H == 1) return false;       // already one row
  const long long P = 1LL * d.N * d.H * d.W;
  if (P <= 0 || P > (1LL << 30)) return false;
  *f = d;
  f->N = 1; f->H = 1; f->W = (int)P;
  f->Ho = 1; f->Wo = (int)P;
  return true;
}

// ---- filters packed ahead of time ------------------------------------------------------------
std::string pack_key(const void* w, int K, int Cg, int kH, int kW, int groups, int flip, int mode, int ldc, int dtype) {
  char key[160];
  snprintf(key, sizeof key, "%p.%d.%d.%d.%d.%d.%d.%d.%d.%d", w, K, Cg, kH, kW, groups, flip, mode, ldc, dtype);
  return key;
}
// The packed form of `w` if b200conv_prepack made one and the filters have not been reported
// changed since; nullptr otherwise (the caller then packs into scratch memory as usual).
void* packed_lookup(b200conv_ctx* c, const void* w, int K, int Cg, int kH, int kW, int groups, int flip, int mode,
                    int ldc, int dtype) {
  if (c->packed.empty()) return nullptr;
  auto it = c->packed.find(pack_key(w, K, Cg, kH, kW, groups, flip, mode, ldc, dtype));
  return it != c->packed.end() && it->second.valid ? it->second.ptr : nullptr;
}
// Which packing the plain (not folded, merged or space-to-depth) forward (mode 0) / gradInputs
// (mode 1) path of a geometry performs; false when that path packs nothing or is not taken.
bool fold_ok(const b200conv_desc& d);
bool s2d_ok(const b200conv_desc& d, int* t0, int* ntaps, int* q0);
int merge_factor(const b200conv_desc& d);
bool plain_pack(const b200conv_desc& d, int mode, int* ldc) {
  if (!umma_ok(d) || merge_factor(d) > 1) return false;
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  if (mode == 0) {
    int a, b, e;
    if (s2d_ok(d, &a, &b, &e) || fold_ok(d)) return false;
    *ldc = pad_channels(Cg, d.dtype);
    return !(d.kH == 1 && d.kW == 1 && *ldc == Cg);        // a 1x1 bank is read in place
  }
  const int ncls = d.sH * d.sW;
  if (ncls > 1 && d.groups == 1 && ncls * d.C <= 64) return false;   // merged parity classes pack their own form
  *ldc = pad_channels(Kg, d.dtype);
  return true;
}

// ======================================================================================
// the three directions on device pointers
// ======================================================================================
int fwd_device(b200conv_ctx* c, const b200conv_desc& d, const void* x, const void* w,
               const void* bias, void* y, int flags) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const size_t es = elem_size(d.dtype);
  const bool out_nhwc = flags & B200CONV_OUT_NHWC, in_nhwc = flags & B200CONV_IN_NHWC;
  const int Kp = pad_channels(d.K, d.dtype);
  if (d.N == 0 || d.K == 0) return 0;
  if (c->epi.pool) {
    if (!out_nhwc || (d.Ho & 1) || (d.Wo & 1) || (flags & B200CONV_FORCE_DIRECT) || c->epi.residual)
      return fail(c, B200CONV_E_UNSUPPORTED, "the pooling epilogue needs a channels-last output with even height and width");
    if (merge_factor(d) > 1 || !umma_ok(d))
      return fail(c, B200CONV_E_UNSUPPORTED, "this geometry's epilogue cannot pool");
  }
  b200conv_desc flat;
  if (!(flags & B200CONV_FORCE_DIRECT) && !c->epi.pool && flatten_1x1(d, in_nhwc && out_nhwc, &flat))
    return fwd_device(c, flat, x, w, bias, y, flags);
  Scratch tmp(c);
  float* bias_f = nullptr;
  if (bias) {
    int rc = tmp.get(sizeof(float) * d.K, reinterpret_cast<void**>(&bias_f));
    if (rc) return rc;
    KLAUNCH(c, kKPack, launch_convert_bias(bias, bias_f, d.K, d.dtype, c->stream));
  }
  const int mg = (flags & B200CONV_FORCE_DIRECT) ? 1 : merge_factor(d);
  if (mg > 1) {
    b200conv_desc dm = d;
    dm.groups = d.groups / mg;
    if (umma_ok(dm)) {
      void* wm;
      int rc = tmp.get(es * (size_t)d.K * Cg * mg * d.kH * d.kW, &wm);
      if (rc) return rc;
      KLAUNCH(c, kKPack, launch_merge_groups(w, wm, d.K, Cg, Kg, mg, d.kH * d.kW, 0, d.dtype, c->stream));
      return fwd_device(c, dm, x, wm, bias, y, flags);
    }
  }
  const bool use_umma = !(flags & B200CONV_FORCE_DIRECT) && umma_ok(d);
  if (!use_umma) {
    if (flags & B200CONV_FORCE_UMMA) return fail(c, B200CONV_E_UNSUPPORTED, "geometry not covered by the tensor-core kernel");
    if (in_nhwc || out_nhwc) return fail(c, B200CONV_E_UNSUPPORTED, "direct kernels take NCHW tensors only");
    KLAUNCH(c, kKDirect, launch_direct_fwd(d, x, w, bias_f, y, (flags & B200CONV_RELU) ? 1 : 0, c->epi, c->stream));
    c->last_algo = "direct";
    return 0;
  }
  const int Cp = pad_channels(d.C, d.dtype);
  int s2_t0 = 0, s2_nt = 0, s2_q0 = 0;
  if (!(flags & B200CONV_NO_S2D) && s2d_ok(d, &s2_t0, &s2_nt, &s2_q0)) {
    // stride 2 with very few channels: 2 x 2 pixel blocks become channels, the layer a stride-1
    // layer with one tap per block row whose reduction runs over kS2dPixels consecutive blocks
    const int win = kS2dPixels * kS2dChannels;
    const int H2 = (d.H + 1) / 2, Wq = d.Wo + kS2dPixels - 1;
    void *xs, *wf;
    int rc = tmp.get(es * (size_t)d.N * H2 * Wq * kS2dChannels, &xs);
    if (rc) return rc;
    KLAUNCH(c, kKTranspose, launch_pad_s2d(x, xs, d.N, d.C, d.H, d.W, Cp, H2, Wq, s2_q0, in_nhwc ? 1 : 0,
                                           d.dtype, c->stream));
    if ((rc = tmp.get(es * (size_t)s2_nt * d.K * win, &wf))) return rc;
    KLAUNCH(c, kKPack, launch_pack_filters_s2d(w, wf, d.K, d.C, d.kH, d.kW, s2_nt, s2_t0, s2_q0, d.padH_l,
                                               d.padW_l, win, d.flip, d.dtype, c->stream));
    std::vector<ConvTap> taps;
    std::vector<std::pair<int, int>> parity(1, {0, 0});
    for (int t = 0; t < s2_nt; ++t) {
      ConvTap tp;
      tp.dh = (int16_t)(t + s2_t0); tp.dw = 0; tp.view = 0; tp.wmat = (int16_t)t;
      taps.push_back(tp);
    }
    FwdLikeArgs a;
    a.act = xs; a.Hs = H2; a.Ws = d.Wo; a.Cin_g = win; a.Cp_in = kS2dChannels;
    a.wpacked = wf; a.ld_w = win; a.nmats = s2_nt;
    a.n_out = d.K; a.groups = 1; a.N = d.N; a.dtype = d.dtype;
    a.view_sH = 1; a.view_sW = 1;
    a.fold = true; a.fold_Wp = Wq; a.fold_sW = 1;
    long long sn, sc, sh, sw;
    if (out_nhwc) {
      const int pl = c->epi.pool ? 2 : 1;
      sn = 1LL * (d.Ho / pl) * (d.Wo / pl) * Kp; sc = 1; sh = 1LL * (d.Wo / pl) * Kp; sw = Kp;
      if (Kp != d.K) CU_OK(c, cudaMemsetAsync(y, 0, es * (size_t)d.N * (d.Ho / pl) * (d.Wo / pl) * Kp, c->stream));
    } else {
      sn = 1LL * d.K * d.Ho * d.Wo; sc = 1LL * d.Ho * d.Wo; sh = d.Wo; sw = 1;
    }
    rc = run_conv_umma(c, a, taps, parity, d.Wo, d.Ho, y, sn, sc, sh, sw, 0, bias_f,
                       (flags & B200CONV_RELU) ? 1 : 0, !(flags & B200CONV_NO_SLAB));
    if (rc == 1) return fail(c, B200CONV_E_CUDA, "internal: empty space-to-depth view");
    c->last_algo = "umma";
    return rc;
  }
  if (fold_ok(d)) {
    // few input channels: one reduction block holds a whole filter row (kW pixels x Cp channels)
    const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
    const int Wp = fold_width(d);
    void *xp, *wf;
    int rc = tmp.get(es * (size_t)d.N * d.H * Wp * Cp, &xp);
    if (rc) return rc;
    KLAUNCH(c, kKTranspose, launch_pad_fold(x, xp, d.N, d.C, d.H, d.W, Cp, Wp, d.padW_l, in_nhwc ? 1 : 0,
                                            d.dtype, c->stream));
    if ((rc = tmp.get(es * (size_t)d.kH * d.K * kBK, &wf))) return rc;
    KLAUNCH(c, kKPack, launch_pack_filters_fold(w, wf, d.K, d.C, d.kH, d.kW, Cp, kBK, d.flip, d.dtype, c->stream));
    std::vector<ConvTap> taps;
    std::vector<std::pair<int, int>> parity;
    for (int i = 0; i < d.kH; ++i) {
      const int ah = i * d.dilH - d.padH_l, rh = pymod(ah, d.sH);
      int v = -1;
      for (size_t q = 0; q < parity.size(); ++q)
        if (parity[q].first == rh) v = (int)q;
      if (v < 0) { v = (int)parity.size(); parity.push_back({rh, 0}); }
      ConvTap t;
      t.dh = (int16_t)floordiv(ah, d.sH); t.dw = 0; t.view = (int16_t)v; t.wmat = (int16_t)i;
      taps.push_back(t);
    }
    FwdLikeArgs a;
    a.act = xp; a.Hs = d.H; a.Ws = d.Wo; a.Cin_g = kBK; a.Cp_in = Cp;
    a.wpacked = wf; a.ld_w = kBK; a.nmats = d.kH;
    a.n_out = d.K; a.groups = 1; a.N = d.N; a.dtype = d.dtype;
    a.view_sH = d.sH; a.view_sW = 1;
    a.fold = true; a.fold_Wp = Wp; a.fold_sW = d.sW;
    long long sn, sc, sh, sw;
    if (out_nhwc) {
      const int pl = c->epi.pool ? 2 : 1;
      sn = 1LL * (d.Ho / pl) * (d.Wo / pl) * Kp; sc = 1; sh = 1LL * (d.Wo / pl) * Kp; sw = Kp;
      if (Kp != d.K) CU_OK(c, cudaMemsetAsync(y, 0, es * (size_t)d.N * (d.Ho / pl) * (d.Wo / pl) * Kp, c->stream));
    } else {
      sn = 1LL * d.K * d.Ho * d.Wo; sc = 1LL * d.Ho * d.Wo; sh = d.Wo; sw = 1;
    }
    rc = run_conv_umma(c, a, taps, parity, d.Wo, d.Ho, y, sn, sc, sh, sw, 0, bias_f,
                       (flags & B200CONV_RELU) ? 1 : 0, !(flags & B200CONV_NO_SLAB));
    if (rc == 1) return fail(c, B200CONV_E_CUDA, "internal: empty folded view");
    c->last_algo = "umma";
    return rc;
  }
  const void* xin = x;
  if (!in_nhwc) {
    int rc = to_nhwc(c, tmp, x, d.N, d.C, d.H, d.W, d.dtype, &xin);
    if (rc) return rc;
  }
  const int ldw = pad_channels(Cg, d.dtype);
  void* wp;
  int rc = 0;
  if (d.kH == 1 && d.kW == 1 && ldw == Cg && reinterpret_cast<uintptr_t>(w) % 16 == 0) {
    // a 1x1 filter bank [K][C] already is its packed form (rows = filters, channels contiguous)
    wp = const_cast<void*>(w);
  } else {
    wp = packed_lookup(c, w, d.K, Cg, d.kH, d.kW, d.groups, d.flip, 0, ldw, d.dtype);
    if (!wp) {
      rc = tmp.get(es * (size_t)d.kH * d.kW * d.K * ldw, &wp);
      if (rc) return rc;
      KLAUNCH(c, kKPack, launch_pack_filters(w, wp, d.K, Cg, d.kH, d.kW, d.groups, d.flip, 0, ldw, d.dtype, c->stream));
    }
  }

  std::vector<ConvTap> taps;
  std::vector<std::pair<int, int>> parity;
  for (int i = 0; i < d.kH; ++i)
    for (int j = 0; j < d.kW; ++j) {
      const int ah = i * d.dilH - d.padH_l, aw = j * d.dilW - d.padW_l;
      const int rh = pymod(ah, d.sH), rw = pymod(aw, d.sW);
      int v = -1;
      for (size_t q = 0; q < parity.size(); ++q)
        if (parity[q].first == rh && parity[q].second == rw) v = (int)q;
      if (v < 0) { v = (int)parity.size(); parity.push_back({rh, rw}); }
      ConvTap t;
      t.dh = (int16_t)floordiv(ah, d.sH); t.dw = (int16_t)floordiv(aw, d.sW);
      t.view = (int16_t)v; t.wmat = (int16_t)(i * d.kW + j);
      taps.push_back(t);
    }
  FwdLikeArgs a;
  a.act = xin; a.Hs = d.H; a.Ws = d.W; a.Cin_g = Cg; a.Cp_in = Cp;
  a.wpacked = wp; a.ld_w = ldw; a.nmats = d.kH * d.kW * d.groups;
  a.n_out = Kg; a.groups = d.groups; a.N = d.N; a.dtype = d.dtype;
  a.view_sH = d.sH; a.view_sW = d.sW;
  long long sn, sc, sh, sw;
  if (out_nhwc) {
    const int pl = c->epi.pool ? 2 : 1;
    sn = 1LL * (d.Ho / pl) * (d.Wo / pl) * Kp; sc = 1; sh = 1LL * (d.Wo / pl) * Kp; sw = Kp;
    if (Kp != d.K) CU_OK(c, cudaMemsetAsync(y, 0, es * (size_t)d.N * (d.Ho / pl) * (d.Wo / pl) * Kp, c->stream));
  } else {
    sn = 1LL * d.K * d.Ho * d.Wo; sc = 1LL * d.Ho * d.Wo; sh = d.Wo; sw = 1;
  }
  rc = run_conv_umma(c, a, taps, parity, d.Wo, d.Ho, y, sn, sc, sh, sw, 0, bias_f,
                     (flags & B200CONV_RELU) ? 1 : 0, !(flags & B200CONV_NO_SLAB));
  if (rc == 1) {  // every tap fell outside the image: conv == 0, only the epilogue remains
    b200conv_desc z = d;
    z.C = 0;
    if (out_nhwc) return fail(c, B200CONV_E_UNSUPPORTED, "degenerate geometry with channels-last output");
    KLAUNCH(c, kKDirect, launch_direct_fwd(z, x, w, bias_f, y, (flags & B200CONV_RELU) ? 1 : 0, c->epi, c->stream));
    rc = 0;
  }
  c->last_algo = "umma";
  return rc;
}

int dgrad_device(b200conv_ctx* c, const b200conv_desc& d, const void* w, const void* dy, void* dx,
                 int flags) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const size_t es = elem_size(d.dtype);
  const bool out_nhwc = flags & B200CONV_OUT_NHWC, in_nhwc = flags & B200CONV_IN_NHWC;
  const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);
  if (d.N == 0 || d.C == 0) return 0;
  b200conv_desc flat;
  if (!(flags & B200CONV_FORCE_DIRECT) && flatten_1x1(d, in_nhwc && out_nhwc, &flat))
    return dgrad_device(c, flat, w, dy, dx, flags);
  const size_t dx_bytes = es * (size_t)d.N * d.H * d.W * (out_nhwc ? Cp : d.C);
  const int mg = (flags & B200CONV_FORCE_DIRECT) ? 1 : merge_factor(d);
  if (mg > 1) {
    b200conv_desc dm = d;
    dm.groups = d.groups / mg;
    if (umma_ok(dm)) {
      Scratch tm(c);
      void* wm;
      int rc = tm.get(es * (size_t)d.K * Cg * mg * d.kH * d.kW, &wm);
      if (rc) return rc;
      KLAUNCH(c, kKPack, launch_merge_groups(w, wm, d.K, Cg, Kg, mg, d.kH * d.kW, 0, d.dtype, c->stream));
      return dgrad_device(c, dm, wm, dy, dx, flags);
    }
  }
  const bool use_umma = !(flags & B200CONV_FORCE_DIRECT) && umma_ok(d);
  if (!use_umma) {
    if (flags & B200CONV_FORCE_UMMA) return fail(c, B200CONV_E_UNSUPPORTED, "geometry not covered by the tensor-core kernel");
    if (in_nhwc || out_nhwc) return fail(c, B200CONV_E_UNSUPPORTED, "direct kernels take NCHW tensors only");
    KLAUNCH(c, kKDirect, launch_direct_dgrad(d, w, dy, dx, c->stream));
    c->last_algo = "direct";
    return 0;
  }
  Scratch tmp(c);
  const void* gin = dy;
  if (!in_nhwc) {
    int rc = to_nhwc(c, tmp, dy, d.N, d.K, d.Ho, d.Wo, d.dtype, &gin);
    if (rc) return rc;
  }
  const int ldw = pad_channels(Kg, d.dtype);
  int rc;

  // Output pixels split into sH*sW parity classes; class (h0, w0) is a stride-1 problem over
  // the taps with (h0 + padH_l - i*dilH) divisible by sH (same for columns).
  struct Cls { int h0, w0, Ht, Wt; std::vector<ConvTap> taps; };
  std::vector<Cls> classes;
  bool need_zero = out_nhwc && Cp != d.C;
  for (int h0 = 0; h0 < d.sH; ++h0)
    for (int w0 = 0; w0 < d.sW; ++w0) {
      Cls k;
      k.h0 = h0; k.w0 = w0;
      k.Ht = h0 < d.H ? (d.H - h0 + d.sH - 1) / d.sH : 0;
      k.Wt = w0 < d.W ? (d.W - w0 + d.sW - 1) / d.sW : 0;
      if (k.Ht == 0 || k.Wt == 0) continue;
      for (int i = 0; i < d.kH; ++i) {
        const int th = h0 + d.padH_l - i * d.dilH;
        if (pymod(th, d.sH)) continue;
        for (int j = 0; j < d.kW; ++j) {
          const int tw = w0 + d.padW_l - j * d.dilW;
          if (pymod(tw, d.sW)) continue;
          ConvTap t;
          t.dh = (int16_t)floordiv(th, d.sH); t.dw = (int16_t)floordiv(tw, d.sW);
          t.view = 0; t.wmat = (int16_t)(i * d.kW + j);
          k.taps.push_back(t);
        }
      }
      if (k.taps.empty()) need_zero = true;
      classes.push_back(k);
    }
  // Few channels and a stride: the classes become channel blocks of ONE stride-1 problem over
  // the union of their tap offsets (a class without a tap at an offset gets a zero filter block
  // there), followed by a depth-to-space pass.  Each class alone would fill a small fraction of
  // an MMA's columns, and the gradient would be read once per class.
  const int ncls = d.sH * d.sW;
  if (ncls > 1 && ncls <= kMaxParityClasses && d.groups == 1 && ncls * d.C <= 64 &&
      (int)classes.size() == ncls && !(flags & B200CONV_NO_MERGE_PARITY)) {
    MergedTapTable tb;
    std::vector<ConvTap> utaps;
    bool fits = true;
    for (size_t k = 0; k < classes.size() && fits; ++k)
      for (const ConvTap& t : classes[k].taps) {
        size_t u = 0;
        while (u < utaps.size() && !(utaps[u].dh == t.dh && utaps[u].dw == t.dw)) ++u;
        if (u == utaps.size()) {
          if (utaps.size() == (size_t)kMaxTaps) { fits = false; break; }
          ConvTap nt = t;
          nt.wmat = (int16_t)u;
          utaps.push_back(nt);
          for (int q = 0; q < kMaxParityClasses; ++q) tb.src[u][q] = -1;
        }
        tb.src[u][classes[k].h0 * d.sW + classes[k].w0] = t.wmat;
      }
    if (!fits) utaps.clear();
    if (!utaps.empty()) {
      const int Ct = pad_channels(ncls * d.C, d.dtype);
      const int nu = (int)utaps.size(), n_out = Ct;      // padded with zero filters: whole 16-byte pieces
      const int Hq = (d.H + d.sH - 1) / d.sH, Wq = (d.W + d.sW - 1) / d.sW;
      void *wp, *merged;
      if ((rc = tmp.get(es * (size_t)nu * n_out * ldw, &wp))) return rc;
      if ((rc = tmp.get(es * (size_t)d.N * Hq * Wq * Ct, &merged))) return rc;
      KLAUNCH(c, kKPack, launch_pack_filters_merged(w, wp, d.K, d.C, d.kH, d.kW, d.flip, tb, nu, ncls, n_out,
                                                    ldw, d.dtype, c->stream));
      FwdLikeArgs a;
      a.act = gin; a.Hs = d.Ho; a.Ws = d.Wo; a.Cin_g = Kg; a.Cp_in = Kp;
      a.wpacked = wp; a.ld_w = ldw; a.nmats = nu;
      a.n_out = n_out; a.groups = 1; a.N = d.N; a.dtype = d.dtype;
      a.view_sH = 1; a.view_sW = 1;
      std::vector<std::pair<int, int>> parity(1, {0, 0});
      rc = run_conv_umma(c, a, utaps, parity, Wq, Hq, merged, 1LL * Hq * Wq * Ct, 1, 1LL * Wq * Ct, Ct, 0,
                         nullptr, 0, !(flags & B200CONV_NO_SLAB));
      if (rc) return rc == 1 ? fail(c, B200CONV_E_CUDA, "internal: empty gradient view") : rc;
      KLAUNCH(c, kKTranspose, launch_depth_to_space(merged, dx, d.N, d.C, d.H, d.W, d.sH, d.sW, Ct, Cp,
                                                    out_nhwc ? 1 : 0, d.dtype, c->stream));
      c->last_algo = "umma";
      return 0;
    }
  }
  void* wp = packed_lookup(c, w, d.K, Cg, d.kH, d.kW, d.groups, d.flip, 1, ldw, d.dtype);
  if (!wp) {
    if ((rc = tmp.get(es * (size_t)d.kH * d.kW * d.C * ldw, &wp))) return rc;
    KLAUNCH(c, kKPack, launch_pack_filters(w, wp, d.K, Cg, d.kH, d.kW, d.groups, d.flip, 1, ldw, d.dtype, c->stream));
  }
  if (need_zero) CU_OK(c, cudaMemsetAsync(dx, 0, dx_bytes, c->stream));
  FwdLikeArgs a;
  a.act = gin; a.Hs = d.Ho; a.Ws = d.Wo; a.Cin_g = Kg; a.Cp_in = Kp;
  a.wpacked = wp; a.ld_w = ldw; a.nmats = d.kH * d.kW * d.groups;
  a.n_out = Cg; a.groups = d.groups; a.N = d.N; a.dtype = d.dtype;
  a.view_sH = 1; a.view_sW = 1;
  std::vector<std::pair<int, int>> parity(1, {0, 0});
  for (const Cls& k : classes) {
    if (k.taps.empty()) continue;
    long long sn, sc, sh, sw, off;
    if (out_nhwc) {
      sn = 1LL * d.H * d.W * Cp; sc = 1; sh = 1LL * d.sH * d.W * Cp; sw = 1LL * d.sW * Cp;
      off = (1LL * k.h0 * d.W + k.w0) * Cp;
    } else {
      sn = 1LL * d.C * d.H * d.W; sc = 1LL * d.H * d.W; sh = 1LL * d.sH * d.W; sw = d.sW;
      off = 1LL * k.h0 * d.W + k.w0;
    }
    rc = run_conv_umma(c, a, k.taps, parity, k.Wt, k.Ht, dx, sn, sc, sh, sw, off, nullptr, 0,
                       !(flags & B200CONV_NO_SLAB));
    if (rc) return rc == 1 ? fail(c, B200CONV_E_CUDA, "internal: empty gradient view") : rc;
  }
  c->last_algo = "umma";
  return 0;
}

// Number of split-K slices of a gradWeights launch.  The items (base_items x slices) are spread
// over num_sms persistent CTAs; the launch lasts as long as its busiest CTA: ceil(items / SMs)
// items of ceil(pix_tiles / slices) pixel tiles each, plus `fixed` tiles' worth of per-item
// overhead (pipeline fill, accumulator read-out).  Pick the count that makes that smallest;
// among equals the smallest count (fewer partial slabs to add up).
static long long balanced_splits(long long pix_tiles, long long base_items, int sms, long long cap,
                                 long long fixed) {
  base_items = std::max(1LL, base_items);
  cap = std::max(1LL, std::min(cap, pix_tiles));
  const long long hi = std::min(cap, std::max(1LL, cdiv(3LL * sms, base_items)));
  long long best = 1, best_cost = -1;
  for (long long s = 1; s <= hi; ++s) {
    const long long per = cdiv(pix_tiles, s);
    if (cdiv(pix_tiles, per) != s) continue;
    const long long cost = cdiv(base_items * s, sms) * (per + fixed);
    if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
  }
  return best;
}

int wgrad_device(b200conv_ctx* c, const b200conv_desc& d, const void* x, const void* dy, void* dw,
                 int flags);

// A slice count the kernels can use near `s`: they cut the pixel tiles into ceil(tiles / s) per slice, and
// every slice must get at least one tile.
int valid_splits(long long pix_tiles, long long s) {
  s = std::max(1LL, std::min(s, pix_tiles));
  return (int)cdiv(pix_tiles, cdiv(pix_tiles, s));
}

// The slice count of a gradWeights launch.  The model's choice `s0` is right about the busiest SM's
// work but knows nothing of the reduction kernel's cost or of L2 effects, so with timing-based
// selection on, the first call of a geometry also times half and twice that count (main kernel plus
// reduction, second of two runs each) and the context remembers the fastest; the role the reference's
// GPU back end gives its meta-optimizer (theano/gpuarray/opt.py:2144-2222).  `run(splits, scratch)`
// enqueues the launch.  Returns the count, or a negative error code.
template <class Run>
int pick_splits(b200conv_ctx* c, const std::string& key, long long pix_tiles, long long cap, int s0, Run run) {
  cap = std::max(1LL, std::min(cap, pix_tiles));
  if (c->force_splits > 0) return valid_splits(pix_tiles, std::min<long long>(c->force_splits, cap));
  if (!c->autotune) return s0;
  auto it = c->split_cache.find(key);
  if (it != c->split_cache.end()) return it->second;
  if (c->capturing) return s0;
  int cand[3] = {s0, valid_splits(pix_tiles, std::min<long long>(cap, std::max(1, s0 / 2))),
                 valid_splits(pix_tiles, std::min<long long>(cap, 2LL * s0))};
  if (!c->ev_tune0) {
    if (cudaEventCreate(&c->ev_tune0) != cudaSuccess || cudaEventCreate(&c->ev_tune1) != cudaSuccess)
      return fail(c, B200CONV_E_CUDA, "event creation failed");
  }
  int best = s0;
  float best_ms = -1.f;
  for (int i = 0; i < 3; ++i) {
    if (i > 0 && (cand[i] == cand[0] || (i == 2 && cand[2] == cand[1]))) continue;
    float ms = 0.f;
    for (int rep = 0; rep < 2; ++rep) {
      Scratch trial(c);
      cudaEventRecord(c->ev_tune0, c->stream);
      int rc = run(cand[i], trial);
      if (rc) return rc < 0 ? rc : -rc;
      cudaEventRecord(c->ev_tune1, c->stream);
      if (cudaStreamSynchronize(c->stream) != cudaSuccess) return fail(c, B200CONV_E_CUDA, "synchronisation failed while tuning");
      cudaEventElapsedTime(&ms, c->ev_tune0, c->ev_tune1);
    }
    if (best_ms < 0.f || ms < best_ms) { best_ms = ms; best = cand[i]; }
  }
  c->split_cache[key] = best;
  return best;
}

// gradWeights with tap groups (wgrad_group.cu).  Returns 0 when launched, 2 when the geometry is
// left to the one-tap-per-item kernel (no two taps share a row offset, or the column span of the
// taps is too wide), or an error code.
int wgrad_grouped(b200conv_ctx* c, const b200conv_desc& d, const void* xin, const void* gin, void* dw,
                  int flags, Scratch& tmp) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);
  const int atom = d.dtype == B200CONV_F16 ? 64 : 32;
  const bool swz32 = d.dtype == B200CONV_F32;
  struct T { int view, dh, dw, wmat; };
  std::vector<T> taps;
  std::vector<std::pair<int, int>> parity;
  std::vector<int> slot;   // parity index -> tensor map slot or -1 (empty view)
  int nviews = 0;
  bool dropped = false;
  for (int i = 0; i < d.kH; ++i)
    for (int j = 0; j < d.kW; ++j) {
      const int ah = i * d.dilH - d.padH_l, aw = j * d.dilW - d.padW_l;
      const int rh = pymod(ah, d.sH), rw = pymod(aw, d.sW);
      int v = -1;
      for (size_t q = 0; q < parity.size(); ++q)
        if (parity[q].first == rh && parity[q].second == rw) v = (int)q;
      if (v < 0) {
        v = (int)parity.size();
        parity.push_back({rh, rw});
        slot.push_back((rh < d.H && rw < d.W) ? nviews++ : -1);
      }
      if (slot[v] < 0) { dropped = true; continue; }
      const int wi = d.flip ? d.kH - 1 - i : i, wj = d.flip ? d.kW - 1 - j : j;
      taps.push_back({slot[v], floordiv(ah, d.sH), floordiv(aw, d.sW), wi * d.kW + wj});
    }
  if (taps.empty() || (int)taps.size() > kMaxTaps) return 2;
  // column span per view
  int dwmin[kMaxViews], dwmax[kMaxViews];
  for (int v = 0; v < nviews; ++v) { dwmin[v] = 1 << 20; dwmax[v] = -(1 << 20); }
  for (const T& t : taps) {
    dwmin[t.view] = std::min(dwmin[t.view], t.dw);
    dwmax[t.view] = std::max(dwmax[t.view], t.dw);
  }
  int Ew = 0;
  for (int v = 0; v < nviews; ++v) Ew = std::max(Ew, dwmax[v] - dwmin[v]);
  if (Ew > 15 || Ew == 0) return 2;
  std::sort(taps.begin(), taps.end(), [](const T& a, const T& b) {
    if (a.view != b.view) return a.view < b.view;
    if (a.dh != b.dh) return a.dh < b.dh;
    return a.dw < b.dw;
  });
  GroupWgradParams p;
  memset(&p, 0, sizeof p);
  for (size_t i = 0; i < taps.size();) {
    size_t j = i;
    while (j < taps.size() && j - i < 4 && taps[j].view == taps[i].view && taps[j].dh == taps[i].dh) ++j;
    if (p.ngroups >= kMaxTapGroups) return 2;
    p.grp_view[p.ngroups] = (int16_t)taps[i].view;
    p.grp_dh[p.ngroups] = (int16_t)taps[i].dh;
    p.grp_first[p.ngroups] = (int16_t)i;
    p.grp_n[p.ngroups] = (int16_t)(j - i);
    ++p.ngroups;
    i = j;
  }
  for (size_t i = 0; i < taps.size(); ++i) {
    p.tap_off[i] = (int16_t)(taps[i].dw - dwmin[taps[i].view]);
    p.tap_wmat[i] = (int16_t)taps[i].wmat;
  }
  for (int v = 0; v < nviews; ++v) p.view_dwmin[v] = (int16_t)dwmin[v];
  // float16 layers with at most 64 channels: a tap group becomes one MMA whose column groups are the taps, if the
  // taps of every group are evenly spaced (stride and dilation decide the spacing; 1 for a plain 3x3 filter)
  if (d.dtype == B200CONV_F16 && Cg <= 64 && c->stack_taps) {
    int step = 0;
    bool even = true;
    for (int gi = 0; gi < p.ngroups && even; ++gi)
      for (int q = 1; q < p.grp_n[gi]; ++q) {
        const int dd = p.tap_off[p.grp_first[gi] + q] - p.tap_off[p.grp_first[gi] + q - 1];
        if (dd <= 0 || (step && dd != step)) even = false;
        step = dd;
      }
    if (even && step > 0) p.stack_step = step;
  }
  // pixel box of a stage
  const int kWgradPix = wgrad_pix(d.dtype);
  if ((d.Wo + Ew) * 2 <= kWgradPix || d.Wo + Ew <= kWgradPix) {
    p.Wa = p.Wb = d.Wo + Ew;                       // whole padded rows
    p.wt = d.Wo;
    p.th = std::max(1, std::min(d.Ho, kWgradPix / p.Wa));
    p.nb = p.th == d.Ho ? std::max(1, std::min(d.N, kWgradPix / (p.Wa * p.th))) : 1;
  } else {
    p.th = 1; p.nb = 1;                            // a segment of one output row
    const int parts = (int)cdiv(d.Wo, kWgradPix - Ew);
    p.wt = (int)cdiv(d.Wo, parts);
    p.Wa = p.wt; p.Wb = p.wt + Ew;
  }
  p.rows_a = p.Wa * p.th * p.nb; p.rows_b = p.Wb * p.th * p.nb;
  p.tiles_w = (int)cdiv(d.Wo, p.wt); p.tiles_h = (int)cdiv(d.Ho, p.th); p.tiles_n = (int)cdiv(d.N, p.nb);
  int rc = make_view(c, &p.dy_map, gin, d.dtype, Kg, d.groups, Kp, d.Wo, d.Ho, d.N, 0, 0, 1, 1, atom, p.Wa,
                     p.th, p.nb, swz32);
  if (rc) return rc;
  for (size_t v = 0; v < parity.size(); ++v) {
    if (slot[v] < 0) continue;
    rc = make_view(c, &p.x_views[slot[v]], xin, d.dtype, Cg, d.groups, Cp, d.W, d.H, d.N, parity[v].first,
                   parity[v].second, d.sH, d.sW, atom, p.Wb, p.th, p.nb, swz32);
    if (rc) return rc;
  }
  for (int v = nviews; v < kMaxViews; ++v) p.x_views[v] = p.x_views[0];
  p.groups = d.groups; p.Kg = Kg; p.Cg = Cg;
  p.Wo = d.Wo; p.Ho = d.Ho; p.Nimg = d.N;
  p.ktiles = (int)cdiv(Kg, 128); p.ctiles = (int)cdiv(Cg, 128);
  p.taps_total = d.kH * d.kW;
  const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
  const long long base_items = 1LL * p.ktiles * p.ctiles * d.groups * p.ngroups;
  // accumulators are not double buffered: aim at one item per SM
  const int s0 = (int)balanced_splits(pix_tiles, base_items, c->num_sms, pix_tiles, 6);
  p.atomic = (flags & B200CONV_ATOMIC_SPLITK) ? 1 : 0;
  p.status = c->d_status;
  p.wait_clocks = c->wait_clocks;
  p.trace = c->trace;
  const size_t slab_elems = (size_t)p.taps_total * d.K * Cg;
  auto run = [&](int splits, Scratch& sc) -> int {
    p.splits = splits;
    const int slabs = p.atomic ? 1 : p.splits;
    float* partial;
    int r = sc.get(sizeof(float) * slab_elems * slabs, reinterpret_cast<void**>(&partial));
    if (r) return r;
    if (p.atomic || dropped)
      CU_OK(c, cudaMemsetAsync(partial, 0, sizeof(float) * slab_elems * slabs, c->stream));
    p.partial = partial;
    p.partial_elems = (long long)slab_elems * slabs;
    KLAUNCH(c, kKWgradUmma, launch_wgrad_group(p, d.dtype, c->num_sms, c->stream));
    KLAUNCH(c, kKWgradReduce, launch_wgrad_reduce(partial, dw, slabs, p.taps_total, d.K, Cg,
                                                  (flags & B200CONV_DW_F32) ? B200CONV_F32 : d.dtype, c->stream));
    return 0;
  };
  char skey[220];
  snprintf(skey, sizeof skey, "sg.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d", d.dtype, d.N, d.C, d.H, d.W, d.K, d.kH,
           d.kW, d.sH, d.sW, d.dilH, d.dilW, d.padH_l, d.padW_l, d.groups, flags & (B200CONV_ATOMIC_SPLITK | B200CONV_DW_F32));
  const int splits = pick_splits(c, skey, pix_tiles, pix_tiles, s0, run);
  if (splits < 0) return splits;
  if ((rc = run(splits, tmp))) return rc;
  c->last_algo = "umma";
  return 0;
}

int wgrad_device(b200conv_ctx* c, const b200conv_desc& d, const void* x, const void* dy, void* dw,
                 int flags) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const size_t es = elem_size(d.dtype);
  const bool x_nhwc = flags & B200CONV_IN_NHWC, dy_nhwc = flags & B200CONV_IN2_NHWC;
  const size_t dw_elems = (size_t)d.K * Cg * d.kH * d.kW;
  // the gradient is accumulated in float32 whatever the data type; B200CONV_DW_F32 also stores it so
  const int odt = (flags & B200CONV_DW_F32) ? B200CONV_F32 : d.dtype;
  const size_t oes = elem_size(odt);
  if (dw_elems == 0) return 0;
  if (d.N == 0) {
    CU_OK(c, cudaMemsetAsync(dw, 0, oes * dw_elems, c->stream));
    return 0;
  }
  b200conv_desc flat;
  if (!(flags & B200CONV_FORCE_DIRECT) && flatten_1x1(d, x_nhwc && dy_nhwc, &flat))
    return wgrad_device(c, flat, x, dy, dw, flags);
  const int mg = (flags & B200CONV_FORCE_DIRECT) ? 1 : merge_factor(d);
  if (mg > 1) {
    b200conv_desc dm = d;
    dm.groups = d.groups / mg;
    if (umma_ok(dm)) {
      // gradient of the block-diagonal filters, then keep the diagonal blocks
      Scratch tm(c);
      void* dwm;
      int rc = tm.get(oes * dw_elems * mg, &dwm);
      if (rc) return rc;
      if ((rc = wgrad_device(c, dm, x, dy, dwm, flags))) return rc;
      KLAUNCH(c, kKPack, launch_merge_groups(dwm, dw, d.K, Cg, Kg, mg, d.kH * d.kW, 1, odt, c->stream));
      return 0;
    }
  }
  const bool use_umma = !(flags & B200CONV_FORCE_DIRECT) && umma_ok(d);
  if (!use_umma) {
    if (flags & B200CONV_FORCE_UMMA) return fail(c, B200CONV_E_UNSUPPORTED, "geometry not covered by the tensor-core kernel");
    if (x_nhwc || dy_nhwc) return fail(c, B200CONV_E_UNSUPPORTED, "direct kernels take NCHW tensors only");
    if (odt != d.dtype) return fail(c, B200CONV_E_UNSUPPORTED, "direct kernels store the gradient in the data type");
    KLAUNCH(c, kKDirect, launch_direct_wgrad(d, x, dy, dw, c->stream));
    c->last_algo = "direct";
    return 0;
  }
  Scratch tmp(c);
  const void* xin = x;
  const void* gin = dy;
  int rc;
  int s2_t0 = 0, s2_nt = 0, s2_q0 = 0;
  if (!(flags & (B200CONV_NO_S2D | B200CONV_ATOMIC_SPLITK)) && s2d_ok(d, &s2_t0, &s2_nt, &s2_q0)) {
    // stride 2 with very few channels: the x operand is the image with 2 x 2 pixel blocks as
    // channels, kS2dPixels consecutive blocks per reduction pixel; the taps are the block rows a
    // filter touches, and the reduction puts the result back into filter order
    if (!dy_nhwc && (rc = to_nhwc(c, tmp, dy, d.N, d.K, d.Ho, d.Wo, d.dtype, &gin))) return rc;
    const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
    const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);
    const int win = kS2dPixels * kS2dChannels;
    const int H2 = (d.H + 1) / 2, Wq = d.Wo + kS2dPixels - 1;
    void* xs;
    if ((rc = tmp.get(es * (size_t)d.N * H2 * Wq * kS2dChannels, &xs))) return rc;
    KLAUNCH(c, kKTranspose, launch_pad_s2d(x, xs, d.N, d.C, d.H, d.W, Cp, H2, Wq, s2_q0, x_nhwc ? 1 : 0,
                                           d.dtype, c->stream));
    UmmaWgradParams p;
    memset(&p, 0, sizeof p);
    const int atom = kBK;
    choose_tile(d.Wo, d.Ho, d.N, wgrad_pix(d.dtype), d.dtype == B200CONV_F16 ? 16 : 8, &p.bw, &p.bh, &p.bn);
    const bool swz32 = d.dtype == B200CONV_F32;
    if ((rc = make_view(c, &p.dy_map, gin, d.dtype, d.K, 1, Kp, d.Wo, d.Ho, d.N, 0, 0, 1, 1, atom, p.bw, p.bh,
                        p.bn, swz32)))
      return rc;
    {
      const size_t pix = (size_t)kS2dChannels * es, row = (size_t)Wq * pix;
      cuuint64_t dims[5] = {(cuuint64_t)win, 1, (cuuint64_t)d.Wo, (cuuint64_t)H2, (cuuint64_t)d.N};
      cuuint64_t strides[4] = {row, pix, row, (cuuint64_t)H2 * row};
      cuuint32_t box[5] = {(cuuint32_t)atom, 1, (cuuint32_t)p.bw, (cuuint32_t)p.bh, (cuuint32_t)p.bn};
      cuuint32_t estr[5] = {1, 1, 1, 1, 1};
      CUresult r = c->encode(&p.x_views[0],
                             d.dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                             5, xs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             swz32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) return fail(c, B200CONV_E_CUDA, "cuTensorMapEncodeTiled(space-to-depth x) failed: %d", (int)r);
    }
    for (int v = 1; v < kMaxViews; ++v) p.x_views[v] = p.x_views[0];
    for (int t = 0; t < s2_nt; ++t) {
      ConvTap tp;
      tp.dh = (int16_t)(t + s2_t0); tp.dw = 0; tp.view = 0; tp.wmat = (int16_t)t;
      p.taps[p.ntaps++] = tp;
    }
    p.groups = 1; p.Kg = d.K; p.Cg = win;
    p.Wo = d.Wo; p.Ho = d.Ho; p.Nimg = d.N;
    p.tiles_w = (int)cdiv(d.Wo, p.bw); p.tiles_h = (int)cdiv(d.Ho, p.bh); p.tiles_n = (int)cdiv(d.N, p.bn);
    p.ktiles = (int)cdiv(d.K, 128); p.ctiles = 1;
    p.taps_total = s2_nt;
    const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
    const long long base_items = 1LL * p.ktiles * p.ntaps;
    p.splits = (int)balanced_splits(pix_tiles, base_items, c->num_sms, pix_tiles / 4, 2);
    const size_t slab_elems = (size_t)s2_nt * d.K * win;
    float* partial;
    if ((rc = tmp.get(sizeof(float) * slab_elems * p.splits, reinterpret_cast<void**>(&partial)))) return rc;
    p.partial = partial;
    p.partial_elems = (long long)slab_elems * p.splits;
    p.status = c->d_status;
    p.wait_clocks = c->wait_clocks;
    p.trace = c->trace;
    KLAUNCH(c, kKWgradUmma, launch_wgrad_umma(p, d.dtype, 64, c->num_sms, c->stream));
    KLAUNCH(c, kKWgradReduce, launch_wgrad_reduce_s2d(partial, dw, p.splits, d.K, d.C, d.kH, d.kW, s2_nt, s2_t0,
                                                      s2_q0, d.padH_l, d.padW_l, win, d.flip, odt, c->stream));
    c->last_algo = "umma";
    return 0;
  }
  if (fold_ok(d) && !(flags & B200CONV_ATOMIC_SPLITK)) {
    // few input channels: the x operand is the row-folded image (kW pixels x Cp channels per
    // reduction pixel), the taps are the kH filter rows, and the reduction unfolds the result
    if (!dy_nhwc && (rc = to_nhwc(c, tmp, dy, d.N, d.K, d.Ho, d.Wo, d.dtype, &gin))) return rc;
    const int kBK = d.dtype == B200CONV_F16 ? 64 : 32;
    const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);
    const int Wp = fold_width(d);
    void* xp;
    if ((rc = tmp.get(es * (size_t)d.N * d.H * Wp * Cp, &xp))) return rc;
    KLAUNCH(c, kKTranspose, launch_pad_fold(x, xp, d.N, d.C, d.H, d.W, Cp, Wp, d.padW_l, x_nhwc ? 1 : 0,
                                            d.dtype, c->stream));
    FwdLikeArgs a;
    a.act = xp; a.Hs = d.H; a.Ws = d.Wo; a.Cin_g = kBK; a.Cp_in = Cp; a.N = d.N; a.dtype = d.dtype;
    a.groups = 1; a.view_sH = d.sH; a.view_sW = 1;
    a.fold = true; a.fold_Wp = Wp; a.fold_sW = d.sW;
    UmmaWgradParams p;
    memset(&p, 0, sizeof p);
    const int atom = kBK;
    choose_tile(d.Wo, d.Ho, d.N, wgrad_pix(d.dtype), d.dtype == B200CONV_F16 ? 16 : 8, &p.bw, &p.bh, &p.bn);
    const bool swz32 = d.dtype == B200CONV_F32;
    if ((rc = make_view(c, &p.dy_map, gin, d.dtype, d.K, 1, Kp, d.Wo, d.Ho, d.N, 0, 0, 1, 1, atom, p.bw, p.bh,
                        p.bn, swz32)))
      return rc;
    int nviews = 0, view_of_parity[kMaxViews];
    for (int q = 0; q < kMaxViews; ++q) view_of_parity[q] = -2;
    bool dropped = false;
    for (int i = 0; i < d.kH; ++i) {
      const int ah = i * d.dilH - d.padH_l, rh = pymod(ah, d.sH);
      if (view_of_parity[rh] == -2) {
        view_of_parity[rh] = -1;
        if (rh < d.H) {
          // the folded view with the 32-byte-atom swizzle gradWeights needs for tf32
          const size_t pix = (size_t)Cp * es, row = (size_t)Wp * pix;
          const int H2 = (d.H - rh + d.sH - 1) / d.sH;
          cuuint64_t dims[5] = {(cuuint64_t)kBK, 1, (cuuint64_t)d.Wo, (cuuint64_t)H2, (cuuint64_t)d.N};
          cuuint64_t strides[4] = {row, (cuuint64_t)d.sW * pix, (cuuint64_t)d.sH * row, (cuuint64_t)d.H * row};
          cuuint32_t box[5] = {(cuuint32_t)atom, 1, (cuuint32_t)p.bw, (cuuint32_t)p.bh, (cuuint32_t)p.bn};
          cuuint32_t estr[5] = {1, 1, 1, 1, 1};
          char* base = static_cast<char*>(xp) + (size_t)rh * row;
          CUresult r = c->encode(&p.x_views[nviews],
                                 d.dtype == B200CONV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                                 5, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swz32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
          if (r != CUDA_SUCCESS) return fail(c, B200CONV_E_CUDA, "cuTensorMapEncodeTiled(folded x) failed: %d", (int)r);
          view_of_parity[rh] = nviews++;
        }
      }
      if (view_of_parity[rh] < 0) { dropped = true; continue; }
      ConvTap t;
      t.dh = (int16_t)floordiv(ah, d.sH); t.dw = 0; t.view = (int16_t)view_of_parity[rh]; t.wmat = (int16_t)i;
      p.taps[p.ntaps++] = t;
    }
    for (int v = nviews; v < kMaxViews; ++v) p.x_views[v] = nviews ? p.x_views[0] : p.dy_map;
    p.groups = 1; p.Kg = d.K; p.Cg = kBK;
    p.Wo = d.Wo; p.Ho = d.Ho; p.Nimg = d.N;
    p.tiles_w = (int)cdiv(d.Wo, p.bw); p.tiles_h = (int)cdiv(d.Ho, p.bh); p.tiles_n = (int)cdiv(d.N, p.bn);
    p.ktiles = (int)cdiv(d.K, 128); p.ctiles = 1;
    p.taps_total = d.kH;
    const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
    const long long base_items = 1LL * p.ktiles * std::max(1, p.ntaps);
    p.splits = (int)balanced_splits(pix_tiles, base_items, c->num_sms, pix_tiles / 4, 2);
    const size_t slab_elems = (size_t)d.kH * d.K * kBK;
    float* partial;
    if ((rc = tmp.get(sizeof(float) * slab_elems * p.splits, reinterpret_cast<void**>(&partial)))) return rc;
    if (dropped || p.ntaps == 0)
      CU_OK(c, cudaMemsetAsync(partial, 0, sizeof(float) * slab_elems * p.splits, c->stream));
    p.partial = partial;
    p.partial_elems = (long long)slab_elems * p.splits;
    p.status = c->d_status;
    p.wait_clocks = c->wait_clocks;
    p.trace = c->trace;
    if (p.ntaps > 0) KLAUNCH(c, kKWgradUmma, launch_wgrad_umma(p, d.dtype, 64, c->num_sms, c->stream));
    KLAUNCH(c, kKWgradReduce, launch_wgrad_reduce_fold(partial, dw, p.splits, d.K, d.C, d.kH, d.kW, Cp, kBK,
                                                       d.flip, odt, c->stream));
    c->last_algo = "umma";
    return 0;
  }
  if (!x_nhwc && (rc = to_nhwc(c, tmp, x, d.N, d.C, d.H, d.W, d.dtype, &xin))) return rc;
  if (!dy_nhwc && (rc = to_nhwc(c, tmp, dy, d.N, d.K, d.Ho, d.Wo, d.dtype, &gin))) return rc;
  const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);

  // Two tensor-core kernels: tap groups sharing operands, or one tap per work item.  As for the
  // forward kernels the first call of a geometry times both and the context remembers the winner.
  bool try_group = !(flags & B200CONV_NO_GROUP);
  char key[200];
  snprintf(key, sizeof key, "w.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d", d.dtype, d.N, d.C, d.H, d.W,
           d.K, d.kH, d.kW, d.sH, d.sW, d.dilH, d.dilW, d.padH_l, d.padW_l, d.groups, flags & B200CONV_ATOMIC_SPLITK);
  // without timings: the one-tap kernel where it runs 256-column MMAs (their issue and TMA
  // budgets are comfortable), tap groups for narrower layers (they read the operands 3x less)
  if (try_group && !c->autotune && d.C / d.groups >= 256) try_group = false;
  if (try_group && c->autotune) {
    auto itc = c->algo_cache.find(key);
    if (itc != c->algo_cache.end()) {
      try_group = itc->second;
    } else if (!c->capturing) {
      if (!c->ev_tune0) {
        CU_OK(c, cudaEventCreate(&c->ev_tune0));
        CU_OK(c, cudaEventCreate(&c->ev_tune1));
      }
      float ms[2] = {0.f, 0.f};
      bool covered = true;
      for (int variant = 0; variant < 2 && covered; ++variant) {   // 0: one tap per item, 1: tap groups
        for (int rep = 0; rep < 2; ++rep) {
          CU_OK(c, cudaEventRecord(c->ev_tune0, c->stream));
          if (variant) {
            // own scratch, returned to the pool after each run: the second run then reuses the
            // first one's buffers and its timing holds no allocation
            Scratch trial(c);
            rc = wgrad_grouped(c, d, xin, gin, dw, flags, trial);
          } else {
            rc = wgrad_device(c, d, xin, gin, dw, flags | B200CONV_NO_GROUP | B200CONV_IN_NHWC | B200CONV_IN2_NHWC);
          }
          if (rc == 2) { covered = false; break; }
          if (rc) return rc;
          CU_OK(c, cudaEventRecord(c->ev_tune1, c->stream));
          CU_OK(c, cudaStreamSynchronize(c->stream));
          CU_OK(c, cudaEventElapsedTime(&ms[variant], c->ev_tune0, c->ev_tune1));
        }
      }
      try_group = covered && ms[1] <= ms[0];
      c->algo_cache[key] = try_group;
    }
  }
  if (try_group) {
    rc = wgrad_grouped(c, d, xin, gin, dw, flags, tmp);
    if (rc != 2) return rc;     // 2: geometry not covered, use the one-tap-per-item kernel
  }

  UmmaWgradParams p;
  memset(&p, 0, sizeof p);
  const int atom = d.dtype == B200CONV_F16 ? 64 : 32;
  const int kk = d.dtype == B200CONV_F16 ? 16 : 8;
  const int BN = Cg <= 64 ? 64 : Cg <= 128 ? 128 : 256;
  choose_tile(d.Wo, d.Ho, d.N, wgrad_pix(d.dtype, BN), kk, &p.bw, &p.bh, &p.bn);
  const bool swz32 = d.dtype == B200CONV_F32;  // MN-major tf32 operands need 32-byte swizzle atoms
  rc = make_view(c, &p.dy_map, gin, d.dtype, Kg, d.groups, Kp, d.Wo, d.Ho, d.N, 0, 0, 1, 1, atom,
                 p.bw, p.bh, p.bn, swz32);
  if (rc) return rc;
  std::vector<std::pair<int, int>> parity;
  std::vector<int> view_of;  // parity index -> tensor map index or -1
  int nviews = 0;
  bool dropped = false;
  for (int i = 0; i < d.kH; ++i)
    for (int j = 0; j < d.kW; ++j) {
      const int ah = i * d.dilH - d.padH_l, aw = j * d.dilW - d.padW_l;
      const int rh = pymod(ah, d.sH), rw = pymod(aw, d.sW);
      int v = -1;
      for (size_t q = 0; q < parity.size(); ++q)
        if (parity[q].first == rh && parity[q].second == rw) v = (int)q;
      if (v < 0) {
        v = (int)parity.size();
        parity.push_back({rh, rw});
        int slot = -1;
        if (rh < d.H && rw < d.W) {
          slot = nviews++;
          rc = make_view(c, &p.x_views[slot], xin, d.dtype, Cg, d.groups, Cp, d.W, d.H, d.N, rh, rw,
                         d.sH, d.sW, atom, p.bw, p.bh, p.bn, swz32);
          if (rc) return rc;
        }
        view_of.push_back(slot);
      }
      if (view_of[v] < 0) { dropped = true; continue; }
      ConvTap t;
      t.dh = (int16_t)floordiv(ah, d.sH); t.dw = (int16_t)floordiv(aw, d.sW);
      t.view = (int16_t)view_of[v];
      const int wi = d.flip ? d.kH - 1 - i : i, wj = d.flip ? d.kW - 1 - j : j;
      t.wmat = (int16_t)(wi * d.kW + wj);
      p.taps[p.ntaps++] = t;
    }
  for (int v = nviews; v < kMaxViews; ++v) p.x_views[v] = nviews ? p.x_views[0] : p.dy_map;
  p.groups = d.groups; p.Kg = Kg; p.Cg = Cg;
  p.Wo = d.Wo; p.Ho = d.Ho; p.Nimg = d.N;
  p.tiles_w = (int)cdiv(d.Wo, p.bw); p.tiles_h = (int)cdiv(d.Ho, p.bh); p.tiles_n = (int)cdiv(d.N, p.bn);
  // 256+ filters and 256+ channels in float16: pairs of CTAs compute 256 x 256 tiles and share the x tile
  const bool pair = c->use_pair && d.dtype == B200CONV_F16 && BN == 256 && Kg >= 256 && c->num_sms >= 2;
  p.ktiles = (int)cdiv(Kg, pair ? 256 : 128); p.ctiles = (int)cdiv(Cg, BN);
  p.taps_total = d.kH * d.kW;
  const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
  const long long base_items = 1LL * p.ktiles * p.ctiles * d.groups * std::max(1, p.ntaps);
  const int s0 = (int)balanced_splits(pix_tiles, base_items, pair ? c->num_sms / 2 : c->num_sms, pix_tiles / 4, 2);
  p.atomic = (flags & B200CONV_ATOMIC_SPLITK) ? 1 : 0;
  p.status = c->d_status;
  p.wait_clocks = c->wait_clocks;
  p.trace = c->trace;
  const size_t slab_elems = (size_t)p.taps_total * d.K * Cg;
  auto run = [&](int splits, Scratch& sc) -> int {
    p.splits = splits;
    const int slabs = p.atomic ? 1 : p.splits;
    float* partial;
    int r = sc.get(sizeof(float) * slab_elems * slabs, reinterpret_cast<void**>(&partial));
    if (r) return r;
    if (p.atomic || dropped || p.ntaps == 0)
      CU_OK(c, cudaMemsetAsync(partial, 0, sizeof(float) * slab_elems * slabs, c->stream));
    p.partial = partial;
    p.partial_elems = (long long)slab_elems * slabs;
    if (p.ntaps > 0) {
      if (pair) KLAUNCH(c, kKWgradUmma, launch_wgrad_pair(p, c->num_sms, c->stream));
      else KLAUNCH(c, kKWgradUmma, launch_wgrad_umma(p, d.dtype, BN, c->num_sms, c->stream));
    }
    KLAUNCH(c, kKWgradReduce, launch_wgrad_reduce(partial, dw, slabs, p.taps_total, d.K, Cg, odt, c->stream));
    return 0;
  };
  char skey[220];
  snprintf(skey, sizeof skey, pair ? "sp.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d" : "su.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d.%d", d.dtype, d.N, d.C, d.H, d.W, d.K, d.kH,
           d.kW, d.sH, d.sW, d.dilH, d.dilW, d.padH_l, d.padW_l, d.groups, flags & (B200CONV_ATOMIC_SPLITK | B200CONV_DW_F32));
  const int splits = pick_splits(c, skey, pix_tiles, std::max(1LL, pix_tiles / 4), s0, run);
  if (splits < 0) return splits;
  if ((rc = run(splits, tmp))) return rc;
  c->last_algo = "umma";
  return 0;
}

// ---- host-pointer wrappers: copy in, run, copy out, synchronise ---------------------------
int stage_setup(b200conv_ctx* c) {
  if (c->copy_pool) return 0;
  for (int i = 0; i < kStageBuffers; ++i) {
    cudaError_t e = cudaHostAlloc(&c->stage_buf[i], kStageChunk, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->stage_ev[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(c, B200CONV_E_NOMEM, "pinned staging buffers: %s", cudaGetErrorString(e));
    }
  }
  const char* env = getenv("B200CONV_COPY_THREADS");
  const int cores = (int)std::thread::hardware_concurrency();
  int n = env ? atoi(env) : std::min(8, std::max(2, cores / 2));   // 1.51 s -> 1.36 s per ResNet-50 step from 4 to 8 threads
  n = std::max(1, std::min(n, 16));
  c->copy_pool = new CopyPool(n);
  return 0;
}

// Host array -> device memory through the pinned buffers: while the DMA engine moves chunk i, the
// copy threads fill the other buffer with chunk i + 1.
int stage_upload(b200conv_ctx* c, void* d, const void* h, size_t bytes) {
  int rc = stage_setup(c);
  if (rc) return rc;
  int k = 0;
  for (size_t off = 0; off < bytes; off += kStageChunk, k ^= 1) {
    const size_t n = std::min(kStageChunk, bytes - off);
    if (c->stage_busy[k]) CU_OK(c, cudaEventSynchronize(c->stage_ev[k]));      // its previous transfer has left
    c->copy_pool->copy(c->stage_buf[k], static_cast<const char*>(h) + off, n);
    CU_OK(c, cudaMemcpyAsync(static_cast<char*>(d) + off, c->stage_buf[k], n, cudaMemcpyHostToDevice, c->stream));
    CU_OK(c, cudaEventRecord(c->stage_ev[k], c->stream));
    c->stage_busy[k] = true;
  }
  return 0;
}

// Device memory -> host array: chunk i + 1 travels into one buffer while the copy threads empty the
// other into the array.  Returns with everything in place (it waits for the stream).
int stage_download(b200conv_ctx* c, void* h, const void* d, size_t bytes) {
  int rc = stage_setup(c);
  if (rc) return rc;
  for (int k = 0; k < kStageBuffers; ++k)
    if (c->stage_busy[k]) { CU_OK(c, cudaEventSynchronize(c->stage_ev[k])); c->stage_busy[k] = false; }
  size_t prev_off = 0, prev_n = 0;
  int k = 0;
  for (size_t off = 0; off < bytes; off += kStageChunk, k ^= 1) {
    const size_t n = std::min(kStageChunk, bytes - off);
    CU_OK(c, cudaMemcpyAsync(c->stage_buf[k], static_cast<const char*>(d) + off, n, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(c, cudaEventRecord(c->stage_ev[k], c->stream));
    if (prev_n) {
      CU_OK(c, cudaEventSynchronize(c->stage_ev[k ^ 1]));
      c->copy_pool->copy(static_cast<char*>(h) + prev_off, c->stage_buf[k ^ 1], prev_n);
    }
    prev_off = off; prev_n = n;
  }
  if (prev_n) {
    CU_OK(c, cudaEventSynchronize(c->stage_ev[k ^ 1]));
    c->copy_pool->copy(static_cast<char*>(h) + prev_off, c->stage_buf[k ^ 1], prev_n);
  }
  return 0;
}

struct HostIO {
  b200conv_ctx* c;
  Scratch tmp;
  explicit HostIO(b200conv_ctx* ctx) : c(ctx), tmp(ctx) {}
  int in(const void* h, size_t bytes, void** d) {
    int rc = tmp.get(bytes, d);
    if (rc) return rc;
    if (bytes >= kStageMinBytes) return stage_upload(c, *d, h, bytes);
    if (bytes) CU_OK(c, cudaMemcpyAsync(*d, h, bytes, cudaMemcpyHostToDevice, c->stream));
    return 0;
  }
  int out(size_t bytes, void** d) { return tmp.get(bytes, d); }
  int back(void* h, const void* d, size_t bytes) {
    if (bytes >= kStageMinBytes) return stage_download(c, h, d, bytes);
    if (bytes) CU_OK(c, cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, c->stream));
    return 0;
  }
};

}  // namespace

// ======================================================================================
// exported functions
// ======================================================================================
extern "C" {

const char* b200conv_version(void) { return "b200conv 0.1 (sm_100a)"; }

int b200conv_create_error(char* buf, size_t n) {
  std::lock_guard<std::mutex> g(g_create_mu);
  if (buf && n) {
    strncpy(buf, g_create_err.c_str(), n - 1);
    buf[n - 1] = 0;
  }
  return (int)g_create_err.size();
}

int b200conv_create(int device, b200conv_ctx** out) {
  std::lock_guard<std::mutex> g(g_create_mu);
  if (!out) return B200CONV_E_INVALID;
  *out = nullptr;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0) {
    g_create_err = std::string("no CUDA device: ") + cudaGetErrorString(e);
    cudaGetLastError();
    return B200CONV_E_CUDA;
  }
  if (device < 0 || device >= ndev) {
    g_create_err = "device index out of range";
    return B200CONV_E_INVALID;
  }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, device);
  if (prop.major != 10) {
    g_create_err = "device is not compute capability 10.x (this library is built for sm_100a only)";
    return B200CONV_E_UNSUPPORTED;
  }
  DeviceGuard dg(device);
  b200conv_ctx* c = new b200conv_ctx();
  c->device = device;
  c->num_sms = c->device_sms = prop.multiProcessorCount;
  bool ok = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess &&
            cudaMalloc(&c->d_status, sizeof(int)) == cudaSuccess &&
            cudaMemset(c->d_status, 0, sizeof(int)) == cudaSuccess &&
            cudaHostAlloc(&c->h_status, sizeof(int), cudaHostAllocDefault) == cudaSuccess &&
            cudaEventCreate(&c->ev0) == cudaSuccess && cudaEventCreate(&c->ev1) == cudaSuccess;
  if (ok) {
    *c->h_status = 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    ok = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess &&
         qr == cudaDriverEntryPointSuccess && fn;
    c->encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (!ok) {
    g_create_err = std::string("context setup failed: ") + cudaGetErrorString(cudaGetLastError());
    delete c;
    return B200CONV_E_CUDA;
  }
  *out = c;
  return 0;
}

void b200conv_destroy(b200conv_ctx* c) {
  if (!c) return;
  DeviceGuard dg(c->device);
  cudaStreamSynchronize(c->stream);
  b200conv_nccl_destroy(c);
  for (auto& kv : c->free_blocks) cudaFree(kv.second);
  for (auto& kv : c->live) cudaFree(kv.first);
  if (c->l2buf) cudaFree(c->l2buf);
  if (c->d_token) cudaFree(c->d_token);
  if (c->up_stream) {
    cudaStreamDestroy(c->up_stream);
    cudaStreamDestroy(c->down_stream);
    cudaEventDestroy(c->ev_up);
    cudaEventDestroy(c->ev_down);
  }
  if (c->comm_stream) {
    cudaStreamDestroy(c->comm_stream);
    cudaEventDestroy(c->ev_comm_ready);
    cudaEventDestroy(c->ev_comm_done);
  }
  delete c->copy_pool;
  for (int i = 0; i < kStageBuffers; ++i) {
    if (c->stage_buf[i]) cudaFreeHost(c->stage_buf[i]);
    if (c->stage_ev[i]) cudaEventDestroy(c->stage_ev[i]);
  }
  cudaFree(c->d_status);
  cudaFreeHost(c->h_status);
  for (auto& r : c->prof_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (auto& e : c->prof_pool) cudaEventDestroy(e);
  cudaEventDestroy(c->ev0);
  cudaEventDestroy(c->ev1);
  if (c->ev_tune0) { cudaEventDestroy(c->ev_tune0); cudaEventDestroy(c->ev_tune1); }
  cudaStreamDestroy(c->stream);
  delete c;
}

int b200conv_last_error(b200conv_ctx* c, char* buf, size_t n) {
  if (!c) return 0;
  std::lock_guard<std::mutex> g(c->mu);
  if (buf && n) {
    strncpy(buf, c->err.c_str(), n - 1);
    buf[n - 1] = 0;
  }
  return (int)c->err.size();
}

int b200conv_padded_channels(int C, int dtype) { return pad_channels(C, dtype); }

// Resets the context's forward epilogue when a call returns, whichever way.
struct EpilogueScope {
  b200conv_ctx* c;
  EpilogueScope(b200conv_ctx* ctx, const ConvEpilogue& e) : c(ctx) { c->epi = e; }
  ~EpilogueScope() { c->epi = default_epilogue(); }
};

static int fwd_call(b200conv_ctx* c, const b200conv_desc* d, const void* x, const void* w, const void* bias,
                    const void* residual, void* y, ConvEpilogue epi, int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = validate(c, d);
  if (rc) return rc;
  epi.pool = (flags & B200CONV_POOL2X2) ? 1 : 0;
  if (!(flags & B200CONV_HOST_PTRS)) {
    epi.residual = residual;
    EpilogueScope scope(c, epi);
    return fwd_device(c, *d, x, w, bias, y, flags);
  }
  if (epi.pool) return fail(c, B200CONV_E_UNSUPPORTED, "the pooling epilogue takes channels-last device tensors");
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "host-pointer calls cannot be captured in a graph");
  if (flags & (B200CONV_IN_NHWC | B200CONV_OUT_NHWC))
    return fail(c, B200CONV_E_INVALID, "host tensors are NCHW");
  const size_t es = elem_size(d->dtype);
  const size_t nx = es * (size_t)d->N * d->C * d->H * d->W, nw = es * (size_t)d->K * (d->C / d->groups) * d->kH * d->kW,
               ny = es * (size_t)d->N * d->K * d->Ho * d->Wo;
  HostIO io(c);
  void *dx_, *dw_, *db_ = nullptr, *dr_ = nullptr, *dy_;
  if ((rc = io.in(x, nx, &dx_)) || (rc = io.in(w, nw, &dw_)) || (rc = io.out(ny, &dy_))) return rc;
  if (bias && (rc = io.in(bias, es * d->K, &db_))) return rc;
  if (residual && (rc = io.in(residual, ny, &dr_))) return rc;
  epi.residual = dr_;
  {
    EpilogueScope scope(c, epi);
    if ((rc = fwd_device(c, *d, dx_, dw_, db_, dy_, flags & ~B200CONV_HOST_PTRS))) return rc;
  }
  if ((rc = io.back(y, dy_, ny))) return rc;
  return sync_and_check(c);
}

int b200conv_fwd(b200conv_ctx* c, const b200conv_desc* d, const void* x, const void* w,
                 const void* bias, void* y, int flags) {
  return fwd_call(c, d, x, w, bias, nullptr, y, default_epilogue(), flags);
}

int b200conv_fwd_epilogue(b200conv_ctx* c, const b200conv_desc* d, const void* x, const void* w,
                          const void* bias, const void* residual, void* y, float alpha, float beta,
                          float slope, int flags) {
  ConvEpilogue e = default_epilogue();
  e.alpha = alpha;
  e.beta = residual ? beta : 0.f;
  e.lin = 0.5f * (1.f + slope);
  e.abs = 0.5f * (1.f - slope);
  return fwd_call(c, d, x, w, bias, residual, y, e, flags);
}

int b200conv_dgrad(b200conv_ctx* c, const b200conv_desc* d, const void* w, const void* dy, void* dx,
                   int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = validate(c, d);
  if (rc) return rc;
  if (!(flags & B200CONV_HOST_PTRS)) return dgrad_device(c, *d, w, dy, dx, flags);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "host-pointer calls cannot be captured in a graph");
  if (flags & (B200CONV_IN_NHWC | B200CONV_OUT_NHWC))
    return fail(c, B200CONV_E_INVALID, "host tensors are NCHW");
  const size_t es = elem_size(d->dtype);
  const size_t nx = es * (size_t)d->N * d->C * d->H * d->W, nw = es * (size_t)d->K * (d->C / d->groups) * d->kH * d->kW,
               ny = es * (size_t)d->N * d->K * d->Ho * d->Wo;
  HostIO io(c);
  void *dw_, *dy_, *dx_;
  if ((rc = io.in(w, nw, &dw_)) || (rc = io.in(dy, ny, &dy_)) || (rc = io.out(nx, &dx_))) return rc;
  if ((rc = dgrad_device(c, *d, dw_, dy_, dx_, flags & ~B200CONV_HOST_PTRS))) return rc;
  if ((rc = io.back(dx, dx_, nx))) return rc;
  return sync_and_check(c);
}

int b200conv_wgrad(b200conv_ctx* c, const b200conv_desc* d, const void* x, const void* dy, void* dw,
                   int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = validate(c, d);
  if (rc) return rc;
  if (!(flags & B200CONV_HOST_PTRS)) return wgrad_device(c, *d, x, dy, dw, flags);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "host-pointer calls cannot be captured in a graph");
  if (flags & (B200CONV_IN_NHWC | B200CONV_IN2_NHWC))
    return fail(c, B200CONV_E_INVALID, "host tensors are NCHW");
  const size_t es = elem_size(d->dtype);
  const size_t nx = es * (size_t)d->N * d->C * d->H * d->W, nw = es * (size_t)d->K * (d->C / d->groups) * d->kH * d->kW,
               ny = es * (size_t)d->N * d->K * d->Ho * d->Wo;
  HostIO io(c);
  void *dx_, *dy_, *dw_;
  const size_t nw_out = (flags & B200CONV_DW_F32) ? nw / es * sizeof(float) : nw;
  if ((rc = io.in(x, nx, &dx_)) || (rc = io.in(dy, ny, &dy_)) || (rc = io.out(nw_out, &dw_))) return rc;
  if ((rc = wgrad_device(c, *d, dx_, dy_, dw_, flags & ~B200CONV_HOST_PTRS))) return rc;
  if ((rc = io.back(dw, dw_, nw_out))) return rc;
  return sync_and_check(c);
}

int b200conv_maxpool2x2(b200conv_ctx* c, const void* x, void* y, int N, int C, int H, int W,
                        int dtype, int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (N < 0 || C < 0 || H < 2 || W < 2) return fail(c, B200CONV_E_INVALID, "pool needs H, W >= 2");
  const size_t es = elem_size(dtype);
  const int nhwc = (flags & B200CONV_IN_NHWC) ? 1 : 0, Cp = pad_channels(C, dtype);
  if (!(flags & B200CONV_HOST_PTRS)) {
    KLAUNCH(c, kKPool, launch_maxpool2x2(x, y, N, C, H, W, nhwc, Cp, dtype, c->stream));
    return 0;
  }
  if (nhwc) return fail(c, B200CONV_E_INVALID, "host tensors are NCHW");
  HostIO io(c);
  void *dx_, *dy_;
  int rc;
  const size_t nx = es * (size_t)N * C * H * W, ny = es * (size_t)N * C * (H / 2) * (W / 2);
  if ((rc = io.in(x, nx, &dx_)) || (rc = io.out(ny, &dy_))) return rc;
  KLAUNCH(c, kKPool, launch_maxpool2x2(dx_, dy_, N, C, H, W, 0, Cp, dtype, c->stream));
  if ((rc = io.back(y, dy_, ny))) return rc;
  return sync_and_check(c);
}

int b200conv_maxpool2x2_grad(b200conv_ctx* c, const void* x, const void* y, const void* gy, void* gx,
                             int N, int C, int H, int W, int dtype, int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (N < 0 || C < 0 || H < 2 || W < 2) return fail(c, B200CONV_E_INVALID, "pool needs H, W >= 2");
  const size_t es = elem_size(dtype);
  const int nhwc = (flags & B200CONV_IN_NHWC) ? 1 : 0, Cp = pad_channels(C, dtype);
  if (!(flags & B200CONV_HOST_PTRS)) {
    KLAUNCH(c, kKPool, launch_maxpool2x2_grad(x, y, gy, gx, N, C, H, W, nhwc, Cp, dtype, c->stream));
    return 0;
  }
  if (nhwc) return fail(c, B200CONV_E_INVALID, "host tensors are NCHW");
  HostIO io(c);
  void *dx_, *dy_, *dgy_, *dgx_;
  int rc;
  const size_t nx = es * (size_t)N * C * H * W, ny = es * (size_t)N * C * (H / 2) * (W / 2);
  if ((rc = io.in(x, nx, &dx_)) || (rc = io.in(y, ny, &dy_)) || (rc = io.in(gy, ny, &dgy_)) ||
      (rc = io.out(nx, &dgx_)))
    return rc;
  KLAUNCH(c, kKPool, launch_maxpool2x2_grad(dx_, dy_, dgy_, dgx_, N, C, H, W, 0, Cp, dtype, c->stream));
  if ((rc = io.back(gx, dgx_, nx))) return rc;
  return sync_and_check(c);
}

int b200conv_elementwise(b200conv_ctx* c, int op, const void* a, const void* b, void* out, long long pixels, int C,
                         int b_kind, float scalar, int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (op < 0 || op >= kEwCount || b_kind < 0 || b_kind > 3 || pixels < 0 || C < 0 ||
      (dtype != B200CONV_F32 && dtype != B200CONV_F16))
    return fail(c, B200CONV_E_INVALID, "bad element-wise operation");
  if ((b_kind == 0 || b_kind == 2) && !b) return fail(c, B200CONV_E_INVALID, "second operand missing");
  if (pixels == 0 || C == 0) return 0;
  const int Cp = pad_channels(C, dtype);
  Scratch tmp(c);
  float* chan = nullptr;
  if (b_kind == 2) {                       // the per-channel operand as Cp float32 values
    int rc = tmp.get(sizeof(float) * Cp, reinterpret_cast<void**>(&chan));
    if (rc) return rc;
    CU_OK(c, cudaMemsetAsync(chan, 0, sizeof(float) * Cp, c->stream));
    KLAUNCH(c, kKPack, launch_convert_bias(b, chan, C, dtype, c->stream));
  }
  KLAUNCH(c, kKTranspose, launch_elementwise(a, b_kind == 0 ? b : nullptr, chan, out, pixels * Cp, C, Cp, op, b_kind,
                                             scalar, dtype, c->stream));
  return 0;
}

int b200conv_channel_sum(b200conv_ctx* c, const void* x, void* out, long long pixels, int C, int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (pixels < 0 || C <= 0 || (dtype != B200CONV_F32 && dtype != B200CONV_F16))
    return fail(c, B200CONV_E_INVALID, "bad channel sum");
  const int Cp = pad_channels(C, dtype);
  Scratch tmp(c);
  float *partial = nullptr, *sums = nullptr;
  int rc = tmp.get(sizeof(float) * Cp * channel_sum_blocks(pixels), reinterpret_cast<void**>(&partial));
  if (rc || (rc = tmp.get(sizeof(float) * Cp, reinterpret_cast<void**>(&sums)))) return rc;
  KLAUNCH(c, kKTranspose, launch_channel_sum(x, partial, sums, pixels, C, Cp, dtype, c->stream));
  if (dtype == B200CONV_F32) {
    CU_OK(c, cudaMemcpyAsync(out, sums, sizeof(float) * C, cudaMemcpyDeviceToDevice, c->stream));
  } else {                                  // float32 sums -> float16 values
    KLAUNCH(c, kKPack, launch_convert_to_half(sums, out, C, c->stream));
  }
  return 0;
}

int b200conv_malloc(b200conv_ctx* c, size_t bytes, void** dptr) {
  if (!c || !dptr) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  return pool_alloc(c, bytes, dptr);
}
int b200conv_free(b200conv_ctx* c, void* dptr) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  return pool_free(c, dptr);
}
int b200conv_host_alloc(b200conv_ctx* c, size_t bytes, void** hptr) {
  if (!c || !hptr) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  cudaError_t e = cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(c, B200CONV_E_NOMEM, "pinned allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  }
  return 0;
}
int b200conv_host_free(b200conv_ctx* c, void* hptr) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  CU_OK(c, cudaFreeHost(hptr));
  return 0;
}
int b200conv_memcpy_h2d(b200conv_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (bytes) CU_OK(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
  return 0;
}
int b200conv_memcpy_d2h(b200conv_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (bytes) CU_OK(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
  return 0;
}
int b200conv_memset(b200conv_ctx* c, void* dst, int value, size_t bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (bytes) CU_OK(c, cudaMemsetAsync(dst, value, bytes, c->stream));
  return 0;
}
static int copy_streams(b200conv_ctx* c) {
  if (!c->up_stream) {
    CU_OK(c, cudaStreamCreateWithFlags(&c->up_stream, cudaStreamNonBlocking));
    CU_OK(c, cudaStreamCreateWithFlags(&c->down_stream, cudaStreamNonBlocking));
    CU_OK(c, cudaEventCreateWithFlags(&c->ev_up, cudaEventDisableTiming));
    CU_OK(c, cudaEventCreateWithFlags(&c->ev_down, cudaEventDisableTiming));
  }
  return 0;
}

int b200conv_memcpy_h2d_bg(b200conv_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  int rc = copy_streams(c);
  if (rc) return rc;
  if (bytes) CU_OK(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->up_stream));
  return 0;
}

int b200conv_join_uploads(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  if (!c->up_stream) return 0;
  CU_OK(c, cudaEventRecord(c->ev_up, c->up_stream));
  CU_OK(c, cudaStreamWaitEvent(c->stream, c->ev_up, 0));
  return 0;
}

int b200conv_memcpy_d2h_bg(b200conv_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  int rc = copy_streams(c);
  if (rc) return rc;
  CU_OK(c, cudaEventRecord(c->ev_down, c->stream));
  CU_OK(c, cudaStreamWaitEvent(c->down_stream, c->ev_down, 0));
  if (bytes) CU_OK(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->down_stream));
  c->down_pending = true;
  return 0;
}

int b200conv_sync(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  return sync_and_check(c);
}

int b200conv_nchw_to_nhwc(b200conv_ctx* c, const void* src, void* dst, int N, int C, int H, int W,
                          int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  KLAUNCH(c, kKTranspose, launch_transpose(src, dst, N, C, H * W, H * W, pad_channels(C, dtype), dtype, c->stream));
  return 0;
}
int b200conv_nhwc_to_nchw(b200conv_ctx* c, const void* src, void* dst, int N, int C, int H, int W,
                          int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  KLAUNCH(c, kKTranspose, launch_transpose(src, dst, N, H * W, C, pad_channels(C, dtype), H * W, dtype, c->stream));
  return 0;
}

int b200conv_timer_start(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  CU_OK(c, cudaEventRecord(c->ev0, c->stream));
  return 0;
}
int b200conv_timer_stop(b200conv_ctx* c, float* ms) {
  if (!c || !ms) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = join_comm(c);
  if (rc) return rc;
  CU_OK(c, cudaEventRecord(c->ev1, c->stream));
  rc = sync_and_check(c);
  if (rc) return rc;
  CU_OK(c, cudaEventElapsedTime(ms, c->ev0, c->ev1));
  return 0;
}
long long b200conv_launch_count(b200conv_ctx* c) { return c ? c->launches : 0; }

// ---- CUDA graphs: record a sequence of device-pointer calls once, replay it with one launch ---
int b200conv_graph_begin(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "a graph is already being captured");
  int rc = join_comm(c);
  if (rc) return rc;
  CU_OK(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed));
  c->capturing = new b200conv_graph();
  return 0;
}

int b200conv_graph_end(b200conv_ctx* c, b200conv_graph** out) {
  if (!c || !out) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (!c->capturing) return fail(c, B200CONV_E_INVALID, "no graph is being captured");
  b200conv_graph* gr = c->capturing;
  int rc = join_comm(c);      // a collective started inside the capture joins before it ends
  c->capturing = nullptr;
  cudaError_t e = cudaStreamEndCapture(c->stream, &gr->graph);
  if (e == cudaSuccess && rc == 0) e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
  if (e != cudaSuccess || rc) {
    cudaGetLastError();
    for (void* p : gr->retained) pool_free(c, p);
    if (gr->graph) cudaGraphDestroy(gr->graph);
    delete gr;
    return rc ? rc : fail(c, B200CONV_E_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  }
  *out = gr;
  return 0;
}

int b200conv_graph_launch(b200conv_ctx* c, b200conv_graph* gr) {
  if (!c || !gr || !gr->exec) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  CU_OK(c, cudaGraphLaunch(gr->exec, c->stream));
  c->launches += gr->launches;
  return 0;
}

int b200conv_graph_destroy(b200conv_ctx* c, b200conv_graph* gr) {
  if (!c || !gr) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  cudaStreamSynchronize(c->stream);
  if (gr->exec) cudaGraphExecDestroy(gr->exec);
  if (gr->graph) cudaGraphDestroy(gr->graph);
  for (void* p : gr->retained) pool_free(c, p);
  delete gr;
  return 0;
}

int b200conv_prepack(b200conv_ctx* c, int count, const b200conv_desc* descs, const void* const* filters,
                     int directions) {
  if (!c || count < 0 || (count && (!descs || !filters))) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  PackBatch batch[2];                       // one per data type
  int nblocks[2] = {0, 0};
  batch[0].njobs = batch[1].njobs = 0;
  auto flush = [&](int t) -> int {
    if (batch[t].njobs) KLAUNCH(c, kKPack, launch_pack_filters_batch(batch[t], nblocks[t], t, c->stream));
    batch[t].njobs = 0;
    nblocks[t] = 0;
    return 0;
  };
  for (int i = 0; i < count; ++i) {
    int rc = validate(c, &descs[i]);
    if (rc) return rc;
    b200conv_desc d = descs[i];
    if (!filters[i] || d.N == 0 || d.C == 0 || d.K == 0) continue;
    b200conv_desc flat;
    if (flatten_1x1(d, true, &flat)) d = flat;         // the geometry the channels-last calls will see
    const int Cg = d.C / d.groups, Kg = d.K / d.groups;
    for (int mode = 0; mode < 2; ++mode) {
      int ldc = 0;
      if (!(directions & (1 << mode)) || !plain_pack(d, mode, &ldc)) continue;
      const std::string key = pack_key(filters[i], d.K, Cg, d.kH, d.kW, d.groups, d.flip, mode, ldc, d.dtype);
      const size_t rows = mode == 0 ? (size_t)d.K : (size_t)d.C;
      const size_t bytes = elem_size(d.dtype) * (size_t)d.kH * d.kW * rows * ldc;
      auto it = c->packed.find(key);
      if (it == c->packed.end()) {
        void* p = nullptr;
        if ((rc = pool_alloc(c, bytes, &p))) return rc;
        it = c->packed.insert({key, b200conv_ctx::Packed{p, bytes, false, filters[i]}}).first;
      }
      const int t = d.dtype == B200CONV_F16 ? 1 : 0;
      if (batch[t].njobs == kPackBatchJobs && (rc = flush(t))) return rc;
      PackJob& j = batch[t].jobs[batch[t].njobs++];
      int gz = 1;
      j.src = filters[i]; j.dst = it->second.ptr;
      j.K = d.K; j.Cg = Cg; j.kH = d.kH; j.kW = d.kW; j.groups = d.groups; j.flip = d.flip; j.mode = mode; j.ldc = ldc;
      pack_filters_grid(Kg, Cg, d.groups, mode, ldc, d.kH * d.kW, &j.gx, &j.gy, &gz);
      j.first_block = nblocks[t];
      nblocks[t] += j.gx * j.gy * gz;
      it->second.valid = true;
    }
  }
  int rc = flush(0);
  if (rc) return rc;
  return flush(1);
}

int b200conv_filters_changed(b200conv_ctx* c, const void* w) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  for (auto& kv : c->packed)
    if (!w || kv.second.src == w) kv.second.valid = false;
  return 0;
}

int b200conv_set_autotune(b200conv_ctx* c, int enable) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  c->autotune = enable != 0;
  return 0;
}

int b200conv_memory_info(b200conv_ctx* c, size_t* pool_bytes, size_t* device_free_bytes) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (pool_bytes) *pool_bytes = c->pool_bytes;
  if (device_free_bytes) {
    size_t total = 0;
    CU_OK(c, cudaMemGetInfo(device_free_bytes, &total));
  }
  return 0;
}

int b200conv_set_wait_limit(b200conv_ctx* c, long long clocks) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  if (clocks < 1000) return fail(c, B200CONV_E_INVALID, "wait limit must be at least 1000 clocks");
  c->wait_clocks = clocks;
  return 0;
}

int b200conv_selftest_wait(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (c->capturing) return fail(c, B200CONV_E_INVALID, "not allowed while a graph is being captured");
  CU_OK(c, launch_wait_selftest(c->d_status, c->wait_clocks, c->stream));
  return sync_and_check(c);
}

int b200conv_set_pair_kernels(b200conv_ctx* c, int enable) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  c->use_pair = enable != 0;
  c->algo_cache.clear();
  return 0;
}

int b200conv_set_stacked_taps(b200conv_ctx* c, int enable) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  c->stack_taps = enable != 0;
  c->algo_cache.clear();
  c->split_cache.clear();
  return 0;
}

int b200conv_set_splits(b200conv_ctx* c, int splits) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  if (splits < 0) return fail(c, B200CONV_E_INVALID, "slice count must be >= 0 (0 = chosen by the library)");
  c->force_splits = splits;
  return 0;
}

// The tuning file: a header line naming the device the choices were timed on, then one line per
// choice.  Choices made on another device model or SM count are not loaded.
static std::string tuning_header(b200conv_ctx* c) {
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, c->device);
  std::string name = prop.name;
  for (char& ch : name)
    if (ch == ' ') ch = '_';
  return "b200conv-tuning 1 " + name + " " + std::to_string(c->num_sms);
}

int b200conv_tuning_save(b200conv_ctx* c, const char* path) {
  if (!c || !path) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  FILE* f = fopen(path, "w");
  if (!f) return fail(c, B200CONV_E_INVALID, "cannot write %s", path);
  fprintf(f, "%s\n", tuning_header(c).c_str());
  for (auto& kv : c->algo_cache) fprintf(f, "a %s %d\n", kv.first.c_str(), kv.second ? 1 : 0);
  for (auto& kv : c->split_cache) fprintf(f, "s %s %d\n", kv.first.c_str(), kv.second);
  fclose(f);
  return 0;
}

int b200conv_tuning_load(b200conv_ctx* c, const char* path, int* loaded) {
  if (!c || !path) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (loaded) *loaded = 0;
  FILE* f = fopen(path, "r");
  if (!f) return fail(c, B200CONV_E_INVALID, "cannot read %s", path);
  char line[512];
  int n = 0;
  bool ok = fgets(line, sizeof line, f) != nullptr;
  if (ok) {
    std::string head = line;
    while (!head.empty() && (head.back() == '\n' || head.back() == '\r')) head.pop_back();
    ok = head == tuning_header(c);
  }
  if (!ok) {
    fclose(f);
    return fail(c, B200CONV_E_INVALID, "%s was not written for this device and SM count", path);
  }
  while (fgets(line, sizeof line, f)) {
    char kind = 0, key[400];
    int val = 0;
    if (sscanf(line, "%c %399s %d", &kind, key, &val) != 3) continue;
    if (kind == 'a') { c->algo_cache[key] = val != 0; ++n; }
    else if (kind == 's' && val >= 1) { c->split_cache[key] = val; ++n; }
  }
  fclose(f);
  if (loaded) *loaded = n;
  return 0;
}

int b200conv_debug_trace(b200conv_ctx* c, void* dbuf) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  c->trace = static_cast<long long*>(dbuf);
  return 0;
}

int b200conv_kernel_timing(b200conv_ctx* c, int enable) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  CU_OK(c, cudaStreamSynchronize(c->stream));
  for (auto& r : c->prof_recs) {
    c->prof_pool.push_back(r.a);
    c->prof_pool.push_back(r.b);
  }
  c->prof_recs.clear();
  c->prof = enable != 0;
  return 0;
}

int b200conv_kernel_time(b200conv_ctx* c, const char* name, float* total_ms, int* launches) {
  if (!c || !name || !total_ms || !launches) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int kind = -1;
  for (int k = 0; k < kKCount; ++k)
    if (!strcmp(name, kKernelNames[k])) kind = k;
  if (kind < 0) return fail(c, B200CONV_E_INVALID, "unknown kernel family '%s'", name);
  CU_OK(c, cudaStreamSynchronize(c->stream));
  float sum = 0.f;
  int n = 0;
  for (auto& r : c->prof_recs) {
    if (r.kind != kind) continue;
    float ms = 0.f;
    CU_OK(c, cudaEventElapsedTime(&ms, r.a, r.b));
    sum += ms;
    ++n;
  }
  *total_ms = sum;
  *launches = n;
  return 0;
}
const char* b200conv_last_algo(b200conv_ctx* c) { return c ? c->last_algo : "none"; }

int b200conv_flush_l2(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (!c->l2buf) {
    c->l2bytes = 256u << 20;  // twice the 126 MB L2
    cudaError_t e = cudaMalloc(&c->l2buf, c->l2bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      c->l2buf = nullptr;
      return fail(c, B200CONV_E_NOMEM, "L2 flush buffer: %s", cudaGetErrorString(e));
    }
  }
  CU_OK(c, launch_fill_l2(c->l2buf, c->l2bytes, c->stream));
  return 0;
}

// ---- NCCL through dlopen: no link-time dependency, nothing loaded unless asked for ---------
typedef struct { char internal[128]; } nccl_uid;
typedef int (*nccl_get_uid_fn)(nccl_uid*);
typedef int (*nccl_init_rank_fn)(void**, int, nccl_uid, int);
typedef int (*nccl_allreduce_fn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*nccl_destroy_fn)(void*);
typedef const char* (*nccl_errstr_fn)(int);

static int nccl_load(b200conv_ctx* c) {
  if (c->nccl_lib) return 0;
  // B200CONV_NCCL_LIB names another library with NCCL's entry points (tests use a stand-in whose
  // collectives fail or stall on the host, so that the watchdog can be exercised without a fault)
  const char* names[] = {getenv("B200CONV_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n || !*n) continue;
    c->nccl_lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (c->nccl_lib) break;
  }
  if (!c->nccl_lib) return fail(c, B200CONV_E_NCCL, "cannot load libnccl.so.2: %s", dlerror());
  return 0;
}
static int nccl_fail(b200conv_ctx* c, const char* what, int code) {
  nccl_errstr_fn es = (nccl_errstr_fn)dlsym(c->nccl_lib, "ncclGetErrorString");
  return fail(c, B200CONV_E_NCCL, "%s failed: %s", what, es ? es(code) : "?");
}

int b200conv_nccl_unique_id(b200conv_ctx* c, void* id128) {
  if (!c || !id128) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  int rc = nccl_load(c);
  if (rc) return rc;
  nccl_get_uid_fn f = (nccl_get_uid_fn)dlsym(c->nccl_lib, "ncclGetUniqueId");
  if (!f) return fail(c, B200CONV_E_NCCL, "ncclGetUniqueId not found");
  int r = f(static_cast<nccl_uid*>(id128));
  return r ? nccl_fail(c, "ncclGetUniqueId", r) : 0;
}

int b200conv_nccl_init(b200conv_ctx* c, int nranks, int rank, const void* id128) {
  if (!c || !id128 || nranks < 1 || rank < 0 || rank >= nranks) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = nccl_load(c);
  if (rc) return rc;
  nccl_init_rank_fn f = (nccl_init_rank_fn)dlsym(c->nccl_lib, "ncclCommInitRank");
  if (!f) return fail(c, B200CONV_E_NCCL, "ncclCommInitRank not found");
  nccl_uid id;
  memcpy(&id, id128, sizeof id);
  int r = f(&c->comm, nranks, id, rank);
  if (r) return nccl_fail(c, "ncclCommInitRank", r);
  c->nranks = nranks;
  c->rank = rank;
  if (!c->d_token) CU_OK(c, cudaMalloc(&c->d_token, sizeof(float)));
  CU_OK(c, cudaMemsetAsync(c->d_token, 0, sizeof(float), c->stream));
  return 0;
}

int b200conv_allreduce_sum(b200conv_ctx* c, void* dbuf, size_t count, int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (!c->comm) return c->nranks == 1 ? 0 : fail(c, B200CONV_E_NCCL, "communicator not initialised (or aborted)");
  nccl_allreduce_fn f = (nccl_allreduce_fn)dlsym(c->nccl_lib, "ncclAllReduce");
  if (!f) return fail(c, B200CONV_E_NCCL, "ncclAllReduce not found");
  // ncclFloat16 = 6, ncclFloat32 = 7, ncclSum = 0
  int r = f(dbuf, dbuf, count, dtype == B200CONV_F16 ? 6 : 7, 0, c->comm, c->stream);
  return r ? nccl_fail(c, "ncclAllReduce", r) : 0;
}

int b200conv_allreduce_sum_async(b200conv_ctx* c, void* dbuf, size_t count, int dtype) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  if (!c->comm) return c->nranks == 1 ? 0 : fail(c, B200CONV_E_NCCL, "communicator not initialised (or aborted)");
  nccl_allreduce_fn f = (nccl_allreduce_fn)dlsym(c->nccl_lib, "ncclAllReduce");
  if (!f) return fail(c, B200CONV_E_NCCL, "ncclAllReduce not found");
  if (!c->comm_stream) {
    CU_OK(c, cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking));
    CU_OK(c, cudaEventCreateWithFlags(&c->ev_comm_ready, cudaEventDisableTiming));
    CU_OK(c, cudaEventCreateWithFlags(&c->ev_comm_done, cudaEventDisableTiming));
  }
  // Collectives queue up on the communication stream in the order they are issued; the main
  // stream only joins the last of them (b200conv_comm_wait and friends).
  CU_OK(c, cudaEventRecord(c->ev_comm_ready, c->stream));
  CU_OK(c, cudaStreamWaitEvent(c->comm_stream, c->ev_comm_ready, 0));
  int r = f(dbuf, dbuf, count, dtype == B200CONV_F16 ? 6 : 7, 0, c->comm, c->comm_stream);
  if (r) return nccl_fail(c, "ncclAllReduce", r);
  CU_OK(c, cudaEventRecord(c->ev_comm_done, c->comm_stream));
  c->comm_pending = true;
  return 0;
}

int b200conv_set_sm_count(b200conv_ctx* c, int sms) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  if (sms < 1 || sms > c->device_sms)
    return fail(c, B200CONV_E_INVALID, "SM count must be between 1 and %d", c->device_sms);
  c->num_sms = sms;
  c->algo_cache.clear();            // kernel choices were timed for another SM count
  c->split_cache.clear();
  return 0;
}

int b200conv_set_comm_timeout(b200conv_ctx* c, int milliseconds) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  if (milliseconds < 1) return fail(c, B200CONV_E_INVALID, "timeout must be at least 1 ms");
  c->comm_timeout_ms = milliseconds;
  return 0;
}

int b200conv_comm_wait(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  return join_comm(c);
}

int b200conv_barrier(b200conv_ctx* c) {
  if (!c) return B200CONV_E_INVALID;
  if (c->comm) {
    int rc = b200conv_allreduce_sum(c, c->d_token, 1, B200CONV_F32);
    if (rc) return rc;
  }
  return b200conv_sync(c);
}

int b200conv_nccl_destroy(b200conv_ctx* c) {
  if (!c || !c->comm) return 0;
  nccl_destroy_fn f = (nccl_destroy_fn)dlsym(c->nccl_lib, "ncclCommDestroy");
  if (f) f(c->comm);
  c->comm = nullptr;
  c->nranks = 1;
  return 0;
}

}  // extern "C"

// ======================================================================================
// gradWeights for callers that must not allocate
// ======================================================================================
// The split-K slabs of the filter gradient normally come from the context's pooled device
// memory, which may call cudaMalloc.  This variant keeps them in a fixed array that is part
// of the library image instead, so the call itself allocates nothing.
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;   // 32 MiB, resident on every GPU that loads the library
static __device__ __align__(256) unsigned char g_wgrad_scratch[kStaticScratchBytes];

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mu;
void* g_static_scratch_addr[kMaxStaticDevices];  // device address of g_wgrad_scratch, per device

// In host code `g_wgrad_scratch` is only a handle for the runtime, not a device address; the
// address on the current device has to be asked for.  Done once per device.
int static_scratch_address(b200conv_ctx* c, float** out) {
  std::lock_guard<std::mutex> g(g_static_mu);
  if (c->device < 0 || c->device >= kMaxStaticDevices)
    return fail(c, B200CONV_E_UNSUPPORTED, "device index %d beyond the static scratch table", c->device);
  if (!g_static_scratch_addr[c->device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_wgrad_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(c, B200CONV_E_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    }
    g_static_scratch_addr[c->device] = p;
  }
  *out = static_cast<float*>(g_static_scratch_addr[c->device]);
  return 0;
}

}  // namespace

extern "C" int b200conv_wgrad_static(b200conv_ctx* c, const b200conv_desc* dp, const void* x,
                                     const void* dy, void* dw, int flags) {
  if (!c) return B200CONV_E_INVALID;
  std::lock_guard<std::mutex> g(c->mu);
  DeviceGuard dg(c->device);
  int rc = validate(c, dp);
  if (rc) return rc;
  const b200conv_desc& d = *dp;
  if (flags & (B200CONV_HOST_PTRS | B200CONV_FORCE_DIRECT))
    return fail(c, B200CONV_E_INVALID, "wgrad_static takes channels-last device tensors only");
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const size_t es = elem_size(d.dtype);
  const size_t dw_elems = (size_t)d.K * Cg * d.kH * d.kW;
  if (dw_elems == 0) return 0;
  if (d.N == 0) {
    CU_OK(c, cudaMemsetAsync(dw, 0, es * dw_elems, c->stream));
    return 0;
  }
  if (!umma_ok(d))
    return fail(c, B200CONV_E_UNSUPPORTED, "wgrad_static covers the tensor-core geometries only");
  const size_t slab_bytes = sizeof(float) * (size_t)d.kH * d.kW * d.K * Cg;
  if (slab_bytes > kStaticScratchBytes)
    return fail(c, B200CONV_E_INVALID,
                "filter gradient needs %zu bytes of scratch per split-K slice; the static scratch "
                "holds %zu bytes (use b200conv_wgrad)", slab_bytes, kStaticScratchBytes);
  float* scratch = nullptr;
  if ((rc = static_scratch_address(c, &scratch))) return rc;

  const int Cp = pad_channels(d.C, d.dtype), Kp = pad_channels(d.K, d.dtype);
  UmmaWgradParams p;
  memset(&p, 0, sizeof p);
  const int atom = d.dtype == B200CONV_F16 ? 64 : 32;
  const int kk = d.dtype == B200CONV_F16 ? 16 : 8;
  const bool swz32 = d.dtype == B200CONV_F32;
  const int BN = Cg <= 64 ? 64 : Cg <= 128 ? 128 : 256;
  choose_tile(d.Wo, d.Ho, d.N, wgrad_pix(d.dtype, BN), kk, &p.bw, &p.bh, &p.bn);
  if ((rc = make_view(c, &p.dy_map, dy, d.dtype, Kg, d.groups, Kp, d.Wo, d.Ho, d.N, 0, 0, 1, 1, atom,
                      p.bw, p.bh, p.bn, swz32)))
    return rc;
  int nviews = 0;
  int view_slot[kMaxViews];
  int par_h[kMaxViews], par_w[kMaxViews], npar = 0;
  bool dropped = false;
  for (int i = 0; i < d.kH; ++i)
    for (int j = 0; j < d.kW; ++j) {
      const int ah = i * d.dilH - d.padH_l, aw = j * d.dilW - d.padW_l;
      const int rh = pymod(ah, d.sH), rw = pymod(aw, d.sW);
      int v = -1;
      for (int q = 0; q < npar; ++q)
        if (par_h[q] == rh && par_w[q] == rw) v = q;
      if (v < 0) {
        v = npar++;
        par_h[v] = rh; par_w[v] = rw;
        view_slot[v] = -1;
        if (rh < d.H && rw < d.W) {
          view_slot[v] = nviews++;
          if ((rc = make_view(c, &p.x_views[view_slot[v]], x, d.dtype, Cg, d.groups, Cp, d.W, d.H, d.N,
                              rh, rw, d.sH, d.sW, atom, p.bw, p.bh, p.bn, swz32)))
            return rc;
        }
      }
      if (view_slot[v] < 0) { dropped = true; continue; }
      ConvTap t;
      t.dh = (int16_t)floordiv(ah, d.sH); t.dw = (int16_t)floordiv(aw, d.sW);
      t.view = (int16_t)view_slot[v];
      const int wi = d.flip ? d.kH - 1 - i : i, wj = d.flip ? d.kW - 1 - j : j;
      t.wmat = (int16_t)(wi * d.kW + wj);
      p.taps[p.ntaps++] = t;
    }
  for (int v = nviews; v < kMaxViews; ++v) p.x_views[v] = nviews ? p.x_views[0] : p.dy_map;
  p.groups = d.groups; p.Kg = Kg; p.Cg = Cg;
  p.Wo = d.Wo; p.Ho = d.Ho; p.Nimg = d.N;
  p.tiles_w = (int)cdiv(d.Wo, p.bw); p.tiles_h = (int)cdiv(d.Ho, p.bh); p.tiles_n = (int)cdiv(d.N, p.bn);
  p.ktiles = (int)cdiv(Kg, 128); p.ctiles = (int)cdiv(Cg, BN);
  p.taps_total = d.kH * d.kW;
  const long long pix_tiles = 1LL * p.tiles_w * p.tiles_h * p.tiles_n;
  const long long base_items = 1LL * p.ktiles * p.ctiles * d.groups * std::max(1, p.ntaps);
  p.splits = (int)balanced_splits(pix_tiles, base_items, c->num_sms,
                                  std::min<long long>(pix_tiles / 4, (long long)(kStaticScratchBytes / slab_bytes)), 2);
  p.atomic = (flags & B200CONV_ATOMIC_SPLITK) ? 1 : 0;
  const int slabs = p.atomic ? 1 : p.splits;
  // the array keeps whatever the previous call left: clear what this call adds into or skips
  if (p.atomic || dropped || p.ntaps == 0)
    CU_OK(c, cudaMemsetAsync(scratch, 0, slab_bytes * slabs, c->stream));
  p.partial = scratch;
  p.partial_elems = (long long)(slab_bytes / sizeof(float)) * slabs;
  p.status = c->d_status;
  p.wait_clocks = c->wait_clocks;
  if (p.ntaps > 0) KLAUNCH(c, kKWgradUmma, launch_wgrad_umma(p, d.dtype, BN, c->num_sms, c->stream));
  KLAUNCH(c, kKWgradReduce, launch_wgrad_reduce(scratch, dw, slabs, p.taps_total, d.K, Cg,
                                                (flags & B200CONV_DW_F32) ? B200CONV_F32 : d.dtype, c->stream));
  c->last_algo = "umma";
  return 0;
}
