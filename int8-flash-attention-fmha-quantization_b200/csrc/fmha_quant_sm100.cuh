// Per-tensor symmetric int8 quantisation on the device: the step the reference project performs on
// the host before the attention call (abs_max + float_quant2_int8, inc/utils.hpp:23-39, driven by
// test_fmha_i8.cpp:95-110).  Two bandwidth-bound kernels over fixed chunks of the tensor:
//   1. quant_absmax_kernel  one CTA per 65536-element chunk -> max|x| of the chunk into partial[chunk]
//   2. quant_apply_kernel   every CTA first reduces partial[] to the tensor's amax (<= 4096 floats, L2
//                           resident), then writes q = clamp(floor(x * (127/amax) + 0.5), -127, 127)
// The partial maxima are scratch memory: global memory that is neither input nor output.
// Algorithmic traffic: 4 B read (pass 1) + 4 B read + 1 B written (pass 2) = 9 bytes per element.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace fmha {

constexpr int kQuantChunk = 65536;       // elements per CTA
constexpr int kQuantThreads = 256;

__global__ void __launch_bounds__(kQuantThreads)
quant_absmax_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  const long long base = static_cast<long long>(blockIdx.x) * kQuantChunk;
  const long long end = min(base + kQuantChunk, n);
  float m = 0.f;
  // 16-byte loads while a whole float4 fits, scalar tail
  const long long n4 = (end - base) / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x + base);
  for (long long i = threadIdx.x; i < n4; i += kQuantThreads) {
    const float4 v = __ldg(x4 + i);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  for (long long i = base + n4 * 4 + threadIdx.x; i < end; i += kQuantThreads) m = fmaxf(m, fabsf(x[i]));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, s));
  __shared__ float warp_max[kQuantThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = warp_max[0];
#pragma unroll
    for (int i = 1; i < kQuantThreads / 32; ++i) b = fmaxf(b, warp_max[i]);
    partial[blockIdx.x] = b;
  }
}

__device__ __forceinline__ int quant_one(float v, float scale) {
  // float_quant2_int8: floorf(x*scale + 0.5) with the sum rounded once to float, clamp to +-127
  const float f = floorf(__fadd_rn(__fmul_rn(v, scale), 0.5f));
  return static_cast<int>(fminf(fmaxf(f, -127.f), 127.f));
}

__global__ void __launch_bounds__(kQuantThreads)
quant_apply_kernel(const float* __restrict__ x, long long n, const float* __restrict__ partial, int n_chunks,
                   int8_t* __restrict__ out, float* __restrict__ amax_out) {
  float m = 0.f;
  for (int i = threadIdx.x; i < n_chunks; i += kQuantThreads) m = fmaxf(m, partial[i]);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, s));
  __shared__ float warp_max[kQuantThreads / 32];
  __shared__ float s_amax;
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = warp_max[0];
#pragma unroll
    for (int i = 1; i < kQuantThreads / 32; ++i) b = fmaxf(b, warp_max[i]);
    s_amax = b;
    if (blockIdx.x == 0 && amax_out) *amax_out = b;
  }
  __syncthreads();
  const float amax = s_amax;
  const float scale = (amax > 0.f) ? __fdiv_rn(127.0f, amax) : 0.f;     // an all-zero tensor quantises to zeros

  const long long base = static_cast<long long>(blockIdx.x) * kQuantChunk;
  const long long end = min(base + kQuantChunk, n);
  const long long n16 = (end - base) / 16;
  const float4* x4 = reinterpret_cast<const float4*>(x + base);
  uint4* o16 = reinterpret_cast<uint4*>(out + base);
  for (long long i = threadIdx.x; i < n16; i += kQuantThreads) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 v = __ldg(x4 + i * 4 + k);
      w[k] = (static_cast<uint32_t>(quant_one(v.x, scale)) & 0xFFu) | ((static_cast<uint32_t>(quant_one(v.y, scale)) & 0xFFu) << 8) |
             ((static_cast<uint32_t>(quant_one(v.z, scale)) & 0xFFu) << 16) | ((static_cast<uint32_t>(quant_one(v.w, scale)) & 0xFFu) << 24);
    }
    o16[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  for (long long i = base + n16 * 16 + threadIdx.x; i < end; i += kQuantThreads) out[i] = static_cast<int8_t>(quant_one(x[i], scale));
}

}  // namespace fmha
