// CUDA-core direct convolution kernels on the reference's own layouts (NCHW / OIHW).
//
// They cover every geometry the reference accepts and serve two purposes: the path for
// shapes the tensor-core kernels decline (e.g. fewer than four channels per group), and an
// independent on-device cross-check of the tensor-core kernels at sizes where a CPU
// computation would take minutes.  Arithmetic: products and sums in float32, one rounding to
// the storage type at the end.
#include "internal.h"

namespace b200 {
namespace {

template <typename T> __device__ __forceinline__ float ld(const T* p) { return static_cast<float>(*p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ void st(T* p, float v) { *p = static_cast<T>(v); }
template <> __device__ __forceinline__ void st<__half>(__half* p, float v) { *p = __float2half_rn(v); }

// top[n,k,oh,ow] = sum_{c,i,j} bottom[n, g*Cg+c, oh*sH-pH+i*dilH, ow*sW-pW+j*dilW] * w[k,c,i',j']
// with (i',j') = (i,j), or (kH-1-i, kW-1-j) when flip.
template <typename T>
__global__ void direct_fwd_kernel(b200conv_desc d, const T* __restrict__ x, const T* __restrict__ w,
                                  const float* __restrict__ bias, T* __restrict__ y, int relu, ConvEpilogue epi) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const long long total = 1LL * d.N * d.K * d.Ho * d.Wo;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int ow = idx % d.Wo;
    const int oh = (idx / d.Wo) % d.Ho;
    const int k = (idx / (1LL * d.Wo * d.Ho)) % d.K;
    const int n = idx / (1LL * d.Wo * d.Ho * d.K);
    const int g = k / Kg;
    float acc = 0.f;
    for (int c = 0; c < Cg; ++c) {
      const T* xc = x + (1LL * n * d.C + g * Cg + c) * d.H * d.W;
      const T* wc = w + (1LL * k * Cg + c) * d.kH * d.kW;
      for (int i = 0; i < d.kH; ++i) {
        const int h = oh * d.sH - d.padH_l + i * d.dilH;
        if (h < 0 || h >= d.H) continue;
        const int wi = d.flip ? d.kH - 1 - i : i;
        for (int j = 0; j < d.kW; ++j) {
          const int ww = ow * d.sW - d.padW_l + j * d.dilW;
          if (ww < 0 || ww >= d.W) continue;
          const int wj = d.flip ? d.kW - 1 - j : j;
          acc += ld(xc + 1LL * h * d.W + ww) * ld(wc + wi * d.kW + wj);
        }
      }
    }
    acc *= epi.alpha;
    if (bias) acc += bias[k];
    if (epi.residual) acc += epi.beta * ld(static_cast<const T*>(epi.residual) + idx);
    if (relu) acc = epi.lin * acc + epi.abs * fabsf(acc);
    st(y + idx, acc);
  }
}

// bottom[n,c,h,w] = sum_{k in group, i, j : divisible} top[n,k,(h+pH-i*dilH)/sH,(w+pW-j*dilW)/sW] * w[k,c,i',j']
template <typename T>
__global__ void direct_dgrad_kernel(b200conv_desc d, const T* __restrict__ w,
                                    const T* __restrict__ dy, T* __restrict__ dx) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const long long total = 1LL * d.N * d.C * d.H * d.W;
  for (long long idx = blockIdx.x * 1LL * blockDim.x + threadIdx.x; idx < total;
       idx += 1LL * gridDim.x * blockDim.x) {
    const int ww = idx % d.W;
    const int h = (idx / d.W) % d.H;
    const int c = (idx / (1LL * d.W * d.H)) % d.C;
    const int n = idx / (1LL * d.W * d.H * d.C);
    const int g = c / Cg, cl = c % Cg;
    float acc = 0.f;
    for (int i = 0; i < d.kH; ++i) {
      const int th = h + d.padH_l - i * d.dilH;
      if (th < 0 || th % d.sH) continue;
      const int oh = th / d.sH;
      if (oh >= d.Ho) continue;
      const int wi = d.flip ? d.kH - 1 - i : i;
      for (int j = 0; j < d.kW; ++j) {
        const int tw = ww + d.padW_l - j * d.dilW;
        if (tw < 0 || tw % d.sW) continue;
        const int ow = tw / d.sW;
        if (ow >= d.Wo) continue;
        const int wj = d.flip ? d.kW - 1 - j : j;
        for (int kq = 0; kq < Kg; ++kq) {
          const int k = g * Kg + kq;
          acc += ld(dy + ((1LL * n * d.K + k) * d.Ho + oh) * d.Wo + ow) *
                 ld(w + ((1LL * k * Cg + cl) * d.kH + wi) * d.kW + wj);
        }
      }
    }
    st(dx + idx, acc);
  }
}

// dw[k,c,i',j'] = sum_{n,oh,ow} top[n,k,oh,ow] * bottom[n, g*Cg+c, oh*sH-pH+i*dilH, ow*sW-pW+j*dilW]
// One block per filter element; threads stride over (n, oh, ow); warp shuffles then shared
// memory combine the partial sums in a fixed order.
template <typename T>
__global__ void direct_wgrad_kernel(b200conv_desc d, const T* __restrict__ x,
                                    const T* __restrict__ dy, T* __restrict__ dw) {
  const int Cg = d.C / d.groups, Kg = d.K / d.groups;
  const long long e = blockIdx.x;  // flat index into dw[K][Cg][kH][kW] in *correlation* tap order
  const int j = e % d.kW;
  const int i = (e / d.kW) % d.kH;
  const int cl = (e / (d.kW * d.kH)) % Cg;
  const int k = e / (1LL * d.kW * d.kH * Cg);
  const int g = k / Kg;
  const long long red = 1LL * d.N * d.Ho * d.Wo;
  float acc = 0.f;
  for (long long r = threadIdx.x; r < red; r += blockDim.x) {
    const int ow = r % d.Wo;
    const int oh = (r / d.Wo) % d.Ho;
    const int n = r / (1LL * d.Wo * d.Ho);
    const int h = oh * d.sH - d.padH_l + i * d.dilH;
    const int ww = ow * d.sW - d.padW_l + j * d.dilW;
    if (h < 0 || h >= d.H || ww < 0 || ww >= d.W) continue;
    acc += ld(dy + ((1LL * n * d.K + k) * d.Ho + oh) * d.Wo + ow) *
           ld(x + ((1LL * n * d.C + g * Cg + cl) * d.H + h) * d.W + ww);
  }
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
  __shared__ float part[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) part[wid] = acc;
  __syncthreads();
  if (wid == 0) {
    acc = lane < (blockDim.x >> 5) ? part[lane] : 0.f;
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
    if (lane == 0) {
      const int wi = d.flip ? d.kH - 1 - i : i, wj = d.flip ? d.kW - 1 - j : j;
      st(dw + ((1LL * k * Cg + cl) * d.kH + wi) * d.kW + wj, acc);
    }
  }
}

int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = 148LL * 32;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

cudaError_t launch_direct_fwd(const b200conv_desc& d, const void* x, const void* w,
                              const float* bias, void* y, int relu, const ConvEpilogue& epi, cudaStream_t s) {
  const long long total = 1LL * d.N * d.K * d.Ho * d.Wo;
  if (total == 0) return cudaSuccess;
  if (d.dtype == B200CONV_F16)
    direct_fwd_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        d, static_cast<const __half*>(x), static_cast<const __half*>(w), bias,
        static_cast<__half*>(y), relu, epi);
  else
    direct_fwd_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        d, static_cast<const float*>(x), static_cast<const float*>(w), bias,
        static_cast<float*>(y), relu, epi);
  return cudaGetLastError();
}

cudaError_t launch_direct_dgrad(const b200conv_desc& d, const void* w, const void* dy, void* dx,
                                cudaStream_t s) {
  const long long total = 1LL * d.N * d.C * d.H * d.W;
  if (total == 0) return cudaSuccess;
  if (d.dtype == B200CONV_F16)
    direct_dgrad_kernel<__half><<<grid_for(total, 256), 256, 0, s>>>(
        d, static_cast<const __half*>(w), static_cast<const __half*>(dy), static_cast<__half*>(dx));
  else
    direct_dgrad_kernel<float><<<grid_for(total, 256), 256, 0, s>>>(
        d, static_cast<const float*>(w), static_cast<const float*>(dy), static_cast<float*>(dx));
  return cudaGetLastError();
}

cudaError_t launch_direct_wgrad(const b200conv_desc& d, const void* x, const void* dy, void* dw,
                                cudaStream_t s) {
  const long long total = 1LL * d.K * (d.C / d.groups) * d.kH * d.kW;
  if (total == 0) return cudaSuccess;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (d.dtype == B200CONV_F16)
    direct_wgrad_kernel<__half><<<static_cast<int>(total), 256, 0, s>>>(
        d, static_cast<const __half*>(x), static_cast<const __half*>(dy), static_cast<__half*>(dw));
  else
    direct_wgrad_kernel<float><<<static_cast<int>(total), 256, 0, s>>>(
        d, static_cast<const float*>(x), static_cast<const float*>(dy), static_cast<float*>(dw));
  return cudaGetLastError();
}

}  // namespace b200
