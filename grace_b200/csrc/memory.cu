// Stand-alone error-feedback kernels for the library path, where a user (or the
// Communicator base class) calls memory.compensate() and memory.update() one
// by one on CUDA tensors instead of going through a fused exchange:
//   residual_compensate   acc = beta * residual + gamma * g
//   residual_update       residual = acc - decompressed
//   sparse_update         residual = acc with the transmitted positions zeroed
//                         (TopK / Threshold / DGC payloads: no dense decompress)
//   dgc_compensate        u = m * u + clamp(g), v += u      (momentum correction)
//   dgc_mask              u, v zeroed where the mask is set
//   sum_squares           sum g^2 in fp64, fixed-order two-level reduction
// Each is one streaming pass with 16-byte accesses; gradients may be fp32, bf16
// or fp16 (converted on load), state is fp32.
//
// Replaces the chains of eager ops in the reference's memory classes:
// grace_dl/dist/memory/residual.py:10-20, memory/efsignsgd.py:11-19,
// memory/dgc.py:15-39 and torch/memory/dgc.py:16-19.
#include "common.cuh"
#include "exchange.h"
#include "gradio.cuh"

namespace grace {

namespace {

constexpr int kBlock = 256;
constexpr int kSumBlocks = 1024;   // partial sums of sum_squares (one per CTA, added in order by the second kernel)

__device__ __forceinline__ int valid4(long long i, long long n) { return i + 4 <= n ? 4 : (i < n ? (int)(n - i) : 0); }

__global__ void __launch_bounds__(kBlock) residual_compensate_kernel(const void* __restrict__ g, int g_dtype,
                                                                    const float* __restrict__ r, float* __restrict__ out,
                                                                    long long n, float beta, float gamma) {
  for (long long i = ((long long)blockIdx.x * kBlock + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * kBlock * 4) {
    const int valid = valid4(i, n);
    float gv[4], rv[4] = {0.f, 0.f, 0.f, 0.f}, ov[4];
    load4g(g, g_dtype, i, valid, gv);
    if (r) load4(r, i, valid, rv);
#pragma unroll
    for (int j = 0; j < 4; ++j) ov[j] = __fadd_rn(__fmul_rn(beta, rv[j]), __fmul_rn(gamma, gv[j]));   // rounded like the eager ops it replaces
    store4(out, i, valid, ov);
  }
}

__global__ void __launch_bounds__(kBlock) residual_update_kernel(const float* __restrict__ acc, const float* __restrict__ dec,
                                                                float* __restrict__ r, long long n) {
  for (long long i = ((long long)blockIdx.x * kBlock + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * kBlock * 4) {
    const int valid = valid4(i, n);
    float av[4], dv[4], ov[4];
    load4(acc, i, valid, av);
    load4(dec, i, valid, dv);
#pragma unroll
    for (int j = 0; j < 4; ++j) ov[j] = av[j] - dv[j];
    store4(r, i, valid, ov);
  }
}

// positions: int32 or int64 indices of the transmitted elements
__global__ void __launch_bounds__(kBlock) zero_at_kernel(float* __restrict__ a, float* __restrict__ b, const void* __restrict__ idx,
                                                        int idx64, long long k, long long n) {
  for (long long e = (long long)blockIdx.x * kBlock + threadIdx.x; e < k; e += (long long)gridDim.x * kBlock) {
    const long long p = idx64 ? static_cast<const long long*>(idx)[e] : (long long)static_cast<const int*>(idx)[e];
    if (p >= 0 && p < n) {   // a corrupt index is skipped, never dereferenced
      a[p] = 0.f;
      if (b) b[p] = 0.f;
    }
  }
}

__global__ void __launch_bounds__(kBlock) dgc_compensate_kernel(const void* __restrict__ g, int g_dtype, float* __restrict__ u,
                                                               float* __restrict__ v, long long n, float momentum,
                                                               float bound, int first) {
  for (long long i = ((long long)blockIdx.x * kBlock + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * kBlock * 4) {
    const int valid = valid4(i, n);
    float gv[4], uv[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f};
    load4g(g, g_dtype, i, valid, gv);
    if (!first) { load4(u, i, valid, uv); load4(v, i, valid, vv); }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float c = fminf(fmaxf(gv[j], -bound), bound);
      uv[j] = __fadd_rn(__fmul_rn(momentum, uv[j]), c);
      vv[j] = vv[j] + uv[j];
    }
    store4(u, i, valid, uv);
    store4(v, i, valid, vv);
  }
}

__global__ void __launch_bounds__(kBlock) dgc_mask_kernel(float* __restrict__ u, float* __restrict__ v,
                                                         const unsigned char* __restrict__ mask, long long n) {
  for (long long i = (long long)blockIdx.x * kBlock + threadIdx.x; i < n; i += (long long)gridDim.x * kBlock)
    if (mask[i]) { u[i] = 0.f; v[i] = 0.f; }
}

__global__ void __launch_bounds__(kBlock) sum_squares_partial_kernel(const void* __restrict__ g, int g_dtype, long long n,
                                                                    double* __restrict__ partial) {
  __shared__ double s_w[kBlock / 32];
  double acc = 0.0;
  for (long long i = ((long long)blockIdx.x * kBlock + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * kBlock * 4) {
    float gv[4];
    load4g(g, g_dtype, i, valid4(i, n), gv);
    acc += (double)(gv[0] * gv[0] + gv[1] * gv[1]) + (double)(gv[2] * gv[2] + gv[3] * gv[3]);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kBlock / 32; ++w) t += s_w[w];
    partial[blockIdx.x] = t;
  }
}

__global__ void sum_squares_final_kernel(const double* __restrict__ partial, int blocks, double* __restrict__ out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double t = 0.0;
    for (int b = 0; b < blocks; ++b) t += partial[b];   // fixed order: the same bits on every run
    *out = t;
  }
}

int grid_for(long long n, int per_thread) {
  long long need = (n + (long long)kBlock * per_thread - 1) / ((long long)kBlock * per_thread);
  if (need < 1) need = 1;
  return (int)(need < 148 * 8 ? need : 148 * 8);
}

}  // namespace

cudaError_t launch_residual_compensate(const void* g, int g_dtype, const float* r, float* out, long long n, float beta,
                                       float gamma, cudaStream_t stream) {
  residual_compensate_kernel<<<grid_for(n, 4), kBlock, 0, stream>>>(g, g_dtype, r, out, n, beta, gamma);
  return cudaGetLastError();
}
cudaError_t launch_residual_update(const float* acc, const float* dec, float* r, long long n, cudaStream_t stream) {
  residual_update_kernel<<<grid_for(n, 4), kBlock, 0, stream>>>(acc, dec, r, n);
  return cudaGetLastError();
}
cudaError_t launch_zero_at(float* a, float* b, const void* idx, int idx64, long long k, long long n, cudaStream_t stream) {
  if (k <= 0) return cudaSuccess;
  zero_at_kernel<<<grid_for(k, 1), kBlock, 0, stream>>>(a, b, idx, idx64, k, n);
  return cudaGetLastError();
}
cudaError_t launch_dgc_compensate(const void* g, int g_dtype, float* u, float* v, long long n, float momentum, float bound,
                                  int first, cudaStream_t stream) {
  dgc_compensate_kernel<<<grid_for(n, 4), kBlock, 0, stream>>>(g, g_dtype, u, v, n, momentum, bound, first);
  return cudaGetLastError();
}
cudaError_t launch_dgc_mask(float* u, float* v, const unsigned char* mask, long long n, cudaStream_t stream) {
  dgc_mask_kernel<<<grid_for(n, 1), kBlock, 0, stream>>>(u, v, mask, n);
  return cudaGetLastError();
}
int sum_squares_scratch_doubles() { return kSumBlocks + 1; }
cudaError_t launch_sum_squares(const void* g, int g_dtype, long long n, double* scratch, cudaStream_t stream) {
  int blocks = grid_for(n, 4);
  if (blocks > kSumBlocks) blocks = kSumBlocks;
  sum_squares_partial_kernel<<<blocks, kBlock, 0, stream>>>(g, g_dtype, n, scratch + 1);
  sum_squares_final_kernel<<<1, 32, 0, stream>>>(scratch + 1, blocks, scratch);
  return cudaGetLastError();
}

}  // namespace grace
