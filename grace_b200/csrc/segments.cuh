// Helpers to walk a flat buffer made of 128-element-aligned segments with
// 16-byte vector accesses.
#pragma once
#include "exchange.h"

namespace grace {

// Visit the part of every segment that lies inside [lo, hi).
template <class F>
__device__ __forceinline__ void for_each_segment_range(const Segment* __restrict__ segs, int nseg, long long lo,
                                                       long long hi, F&& f) {
  int a = 0, b = nseg;
  while (a < b) {
    const int m = (a + b) >> 1;
    if (segs[m].offset + segs[m].numel > lo) b = m; else a = m + 1;
  }
  for (int s = a; s < nseg; ++s) {
    const long long sb = segs[s].offset;
    if (sb >= hi) break;
    const long long se = sb + segs[s].numel;
    const long long b0 = sb > lo ? sb : lo;
    const long long e0 = se < hi ? se : hi;
    if (b0 < e0) f(s, b0, e0);
  }
}

__device__ __forceinline__ void load4(const float* __restrict__ p, long long i, int valid, float (&v)[4]) {
  if (valid == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p + i);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = j < valid ? p[i + j] : 0.f;
  }
}
__device__ __forceinline__ void store4(float* __restrict__ p, long long i, int valid, const float (&v)[4]) {
  if (valid == 4) {
    *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) if (j < valid) p[i + j] = v[j];
  }
}


}  // namespace grace
