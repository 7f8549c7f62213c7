// Typed access to gradient buffers: fp32, bf16 or fp16 in memory, fp32 in registers.
// The element type is a run-time argument of the exchange kernels (one warp-uniform branch per
// 4-element access) rather than a template parameter: the kernels are already instantiated per
// codec / transport, and the branch costs nothing next to the memory access it guards.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "segments.cuh"

namespace grace {

enum GradType : int { kGradF32 = 0, kGradBF16 = 1, kGradF16 = 2 };

__device__ __forceinline__ float grad_to_float(unsigned short h, int dtype) {
  if (dtype == kGradBF16) return __uint_as_float((unsigned)h << 16);
  return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ unsigned short float_to_grad(float f, int dtype) {
  if (dtype == kGradBF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  return __half_as_ushort(__float2half_rn(f));
}

// v[0..4) = p[i..i+4) (elements beyond `valid` read as 0).  fp32: 16-byte access, i % 4 == 0 and a
// 16-byte aligned base; 16-bit types: 8-byte access, 8-byte aligned base.
__device__ __forceinline__ void load4g(const void* __restrict__ p, int dtype, long long i, int valid, float (&v)[4]) {
  if (dtype == kGradF32) {
    load4(static_cast<const float*>(p), i, valid, v);
    return;
  }
  const unsigned short* h = static_cast<const unsigned short*>(p) + i;
  if (valid == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(h);
    v[0] = grad_to_float((unsigned short)(raw.x & 0xffffu), dtype);
    v[1] = grad_to_float((unsigned short)(raw.x >> 16), dtype);
    v[2] = grad_to_float((unsigned short)(raw.y & 0xffffu), dtype);
    v[3] = grad_to_float((unsigned short)(raw.y >> 16), dtype);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = j < valid ? grad_to_float(h[j], dtype) : 0.f;
  }
}

__device__ __forceinline__ void store4g(void* __restrict__ p, int dtype, long long i, int valid, const float (&v)[4]) {
  if (dtype == kGradF32) {
    store4(static_cast<float*>(p), i, valid, v);
    return;
  }
  unsigned short* h = static_cast<unsigned short*>(p) + i;
  if (valid == 4) {
    uint2 raw;
    raw.x = (unsigned)float_to_grad(v[0], dtype) | ((unsigned)float_to_grad(v[1], dtype) << 16);
    raw.y = (unsigned)float_to_grad(v[2], dtype) | ((unsigned)float_to_grad(v[3], dtype) << 16);
    *reinterpret_cast<uint2*>(h) = raw;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) if (j < valid) h[j] = float_to_grad(v[j], dtype);
  }
}

__device__ __forceinline__ float load1g(const void* __restrict__ p, int dtype, long long i) {
  if (dtype == kGradF32) return static_cast<const float*>(p)[i];
  return grad_to_float(static_cast<const unsigned short*>(p)[i], dtype);
}

}  // namespace grace
