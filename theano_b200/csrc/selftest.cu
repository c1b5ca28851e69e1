// Self-test of the bounded device-side wait: a kernel that waits on a barrier nobody arrives on.
// It exercises the path every tensor-core kernel takes when a wait runs out (status word written,
// kernel returns, the context stays usable) without faulting or hanging anything.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {
namespace {

struct Bars {
  uint64_t never;
  volatile int abort;
};

__global__ void __launch_bounds__(64, 1) wait_selftest_kernel(int* status, long long limit) {
  __shared__ Bars bars;
  if (threadIdx.x == 0) {
    mbar_init(&bars.never, 1);
    bars.abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int warp = uniform_warp_index();
  bool ok;
  if (warp == 0) {
    ok = uniform_wait(&bars.never, 0, &bars, limit);                               // the issuers' wait
    if (!ok && elect_one()) atomicExch(status, kStatusTimeout);
  } else {
    ok = warp_wait_or_abort(&bars.never, 0, &bars, threadIdx.x & 31, limit);       // the epilogue warps' wait
    if (!ok && (threadIdx.x & 31) == 0) atomicExch(status, kStatusTimeout);
  }
  __syncthreads();
  if (bars.abort) abort_grace(limit);
}

}  // namespace

cudaError_t launch_wait_selftest(int* status, long long limit, cudaStream_t s) {
  wait_selftest_kernel<<<1, 64, 0, s>>>(status, limit);
  return cudaGetLastError();
}

}  // namespace b200
