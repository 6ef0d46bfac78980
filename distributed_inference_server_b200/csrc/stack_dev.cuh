// stack_dev.cuh -- device helpers shared by k_stack.cu and k_stack_mix.cu.
#pragma once
#include "stack.h"

namespace dis {

template <bool F32>
__device__ __forceinline__ float ld_el(const void *p, long long i) {
  if (F32) return reinterpret_cast<const float *>(p)[i];
  return bf16_bits_to_float(reinterpret_cast<const uint16_t *>(p)[i]);
}
template <bool F32>
__device__ __forceinline__ void st_el(void *p, long long i, float v) {
  if (F32) reinterpret_cast<float *>(p)[i] = v;
  else reinterpret_cast<uint16_t *>(p)[i] = float_to_bf16_bits(v);
}
__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + __expf(-v)); }
__device__ __forceinline__ float sigmoid_precise(float v) { return 1.f / (1.f + expf(-v)); }

__device__ __forceinline__ float block_sum(float v, float *sh) {  // sh: 32 floats; every thread gets the total
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; i++) t += sh[i];
  return t;
}

}  // namespace dis
