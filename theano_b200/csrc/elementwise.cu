// Element-wise kernels on channels-last device tensors, and the per-channel sum.
//
// In compiled Theano graphs the convolution ops are separated by small Elemwise nodes (the bias
// add of a training graph, relu = 0.5 * (v + |v|), its gradient 0.5 * g + 0.5 * g * sgn(v), a
// residual add, a scale) and by the bias gradient Sum{axis=[0, 2, 3]}.  The reference's GPU
// back end keeps them on the device (theano/gpuarray/elemwise.py:86); these kernels do the same
// for tensors that live in HBM between two convolution ops, so that no activation travels to
// the host and back for a few arithmetic operations.  All of them are HBM bound.
#include "internal.h"

namespace b200 {
namespace {

template <typename T> struct Vec;                 // 16 bytes of T
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__half> { static constexpr int n = 8; };

template <typename T> __device__ __forceinline__ void load16(const T* p, float (&f)[Vec<T>::n]);
template <> __device__ __forceinline__ void load16<float>(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load16<__half>(const __half* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
template <typename T> __device__ __forceinline__ void store16(T* p, const float (&f)[Vec<T>::n]);
template <> __device__ __forceinline__ void store16<float>(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store16<__half>(__half* p, const float (&f)[8]) {
  uint4 v;
  __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

__device__ __forceinline__ float apply(int op, float a, float b) {
  switch (op) {
    case kEwAdd: return a + b;
    case kEwMul: return a * b;
    case kEwSub: return a - b;
    case kEwRSub: return b - a;
    case kEwDiv: return a / b;
    case kEwRDiv: return b / a;
    case kEwMax: return fmaxf(a, b);
    case kEwAbs: return fabsf(a);
    case kEwSgn: return a > 0.f ? 1.f : (a < 0.f ? -1.f : 0.f);
    case kEwNeg: return -a;
    default: return a;
  }
}

// out = op(a, b); b is a tensor of a's shape (b_kind 0), the scalar `s` (1), a float32 vector with
// one value per stored channel (2: element i belongs to channel i % Cp) or absent (3).  Pad
// channels are written as 0 so that the tensor stays a valid channels-last operand.
template <typename T>
__global__ void __launch_bounds__(256) elementwise_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          const float* __restrict__ chan, T* __restrict__ out,
                                                          long long nvec, int C, int Cp, int op, int b_kind, float s) {
  constexpr int V = Vec<T>::n;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
    float fa[V], fb[V], fo[V];
    load16<T>(a + i * V, fa);
    const int c0 = static_cast<int>((i * V) % Cp);
    if (b_kind == 0) load16<T>(b + i * V, fb);
#pragma unroll
    for (int q = 0; q < V; ++q) {
      const float bv = b_kind == 0 ? fb[q] : b_kind == 1 ? s : b_kind == 2 ? chan[c0 + q] : 0.f;
      fo[q] = c0 + q < C ? apply(op, fa[q], bv) : 0.f;
    }
    store16<T>(out + i * V, fo);
  }
}

// Stage 1 of the per-channel sum: block b adds the pixels p = b, b + gridDim.x, ... of every
// channel into partial[b][Cp] (float32); thread t owns channels t, t + 256, ...
template <typename T>
__global__ void __launch_bounds__(256) channel_sum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial,
                                                                  long long pixels, int Cp) {
  for (int c = threadIdx.x; c < Cp; c += 256) {
    float acc = 0.f;
    for (long long p = blockIdx.x; p < pixels; p += gridDim.x) acc += static_cast<float>(x[p * Cp + c]);
    partial[1LL * blockIdx.x * Cp + c] = acc;
  }
}
// Stage 2: out[c] = sum over blocks, in block order (the same result on every run).
__global__ void channel_sum_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int blocks, int C,
                                         int Cp) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float acc = 0.f;
  for (int b = 0; b < blocks; ++b) acc += partial[1LL * b * Cp + c];
  out[c] = acc;
}

}  // namespace

cudaError_t launch_elementwise(const void* a, const void* b, const float* chan, void* out, long long elems, int C,
                               int Cp, int op, int b_kind, float s, int dtype, cudaStream_t st) {
  if (elems == 0) return cudaSuccess;
  const int V = dtype == B200CONV_F16 ? 8 : 4;
  const long long nvec = elems / V;              // Cp is a multiple of V, so elems is
  long long grid = (nvec + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (dtype == B200CONV_F16)
    elementwise_kernel<__half><<<static_cast<int>(grid), 256, 0, st>>>(
        static_cast<const __half*>(a), static_cast<const __half*>(b), chan, static_cast<__half*>(out), nvec, C, Cp, op,
        b_kind, s);
  else
    elementwise_kernel<float><<<static_cast<int>(grid), 256, 0, st>>>(
        static_cast<const float*>(a), static_cast<const float*>(b), chan, static_cast<float*>(out), nvec, C, Cp, op,
        b_kind, s);
  return cudaGetLastError();
}

int channel_sum_blocks(long long pixels) { return static_cast<int>(pixels < 148 * 8 ? (pixels < 1 ? 1 : pixels) : 148 * 8); }

cudaError_t launch_channel_sum(const void* x, float* partial, float* out, long long pixels, int C, int Cp, int dtype,
                               cudaStream_t st) {
  const int blocks = channel_sum_blocks(pixels);
  if (dtype == B200CONV_F16)
    channel_sum_partial_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(x), partial, pixels, Cp);
  else
    channel_sum_partial_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), partial, pixels, Cp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  channel_sum_final_kernel<<<(C + 127) / 128, 128, 0, st>>>(partial, out, blocks, C, Cp);
  return cudaGetLastError();
}

}  // namespace b200
