// Fused SGD(momentum, nesterov, weight decay) for sm_100a.
//
// Two entry points with torch.optim.SGD semantics:
//  * launch_fused_sgd: parameters, gradients and momentum buffers are three
//    flat fp32 buffers with the same layout, one streaming pass (16 B/elem
//    read, 8-12 B/elem written), optionally zeroing the gradient buffer for the
//    next backward pass and applying a gradient scale.
//  * launch_multi_sgd: a table of (param, grad, buf, numel) for tensors that do
//    not live in a flat buffer; one launch for the whole model.
// Replaces the foreach torch.optim.SGD step used by the reference's examples
// (examples/dist/CIFAR10-dawndist/torch_backend.py:159-162).
#include "exchange.h"

namespace grace {
namespace {

struct SgdHyper {
  float lr, momentum, dampening, weight_decay, grad_scale;
  int nesterov, first_step, zero_grad;
};

__device__ __forceinline__ void sgd_elem(float& p, float& g, float& b, const SgdHyper& h) {
  float d = g * h.grad_scale + h.weight_decay * p;
  if (h.momentum != 0.f) {
    b = h.first_step ? d : h.momentum * b + (1.f - h.dampening) * d;
    d = h.nesterov ? d + h.momentum * b : b;
  }
  p -= h.lr * d;
  if (h.zero_grad) g = 0.f;
}

__global__ void __launch_bounds__(256) fused_sgd_flat_kernel(float* __restrict__ p, float* __restrict__ g,
                                                             float* __restrict__ buf, long long n4, long long n,
                                                             SgdHyper h) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (h.momentum != 0.f && !h.first_step) bv = reinterpret_cast<float4*>(buf)[i];
    sgd_elem(pv.x, gv.x, bv.x, h); sgd_elem(pv.y, gv.y, bv.y, h);
    sgd_elem(pv.z, gv.z, bv.z, h); sgd_elem(pv.w, gv.w, bv.w, h);
    reinterpret_cast<float4*>(p)[i] = pv;
    if (h.momentum != 0.f) reinterpret_cast<float4*>(buf)[i] = bv;
    if (h.zero_grad) reinterpret_cast<float4*>(g)[i] = gv;
  }
  // tail (n not a multiple of 4)
  const long long t = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) {
    float pv = p[t], gv = g[t], bv = (h.momentum != 0.f && !h.first_step) ? buf[t] : 0.f;
    sgd_elem(pv, gv, bv, h);
    p[t] = pv;
    if (h.momentum != 0.f) buf[t] = bv;
    if (h.zero_grad) g[t] = gv;
  }
}

constexpr int kChunk = 256 * 4 * 4;  // elements per CTA in the table kernel

__global__ void __launch_bounds__(256) fused_sgd_table_kernel(const SgdTensor* __restrict__ table,
                                                              const int2* __restrict__ blocks, SgdHyper h) {
  const int2 blk = blocks[blockIdx.x];
  const SgdTensor t = table[blk.x];
  const int begin = blk.y * kChunk;
  const int end = min(begin + kChunk, t.numel);
  for (int i = begin + threadIdx.x; i < end; i += 256) {
    float pv = t.p[i], gv = t.g[i], bv = (h.momentum != 0.f && !h.first_step) ? t.buf[i] : 0.f;
    sgd_elem(pv, gv, bv, h);
    t.p[i] = pv;
    if (h.momentum != 0.f) t.buf[i] = bv;
    if (h.zero_grad) const_cast<float*>(t.g)[i] = gv;
  }
}

}  // namespace

cudaError_t launch_fused_sgd(float* p, float* g, float* buf, long long numel, float lr, float momentum, float dampening,
                             float weight_decay, int nesterov, int first_step, int zero_grad, float grad_scale,
                             cudaStream_t stream) {
  if (numel <= 0) return cudaSuccess;
  SgdHyper h{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_step, zero_grad};
  const long long n4 = numel / 4;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  fused_sgd_flat_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p, g, buf, n4, numel, h);
  return cudaGetLastError();
}

int sgd_table_chunk() { return kChunk; }

cudaError_t launch_multi_sgd(const SgdTensor* table, const int* blocks_xy, int nblocks, float lr, float momentum,
                             float dampening, float weight_decay, int nesterov, int first_step, int zero_grad,
                             float grad_scale, cudaStream_t stream) {
  if (nblocks <= 0) return cudaSuccess;
  SgdHyper h{lr, momentum, dampening, weight_decay, grad_scale, nesterov, first_step, zero_grad};
  fused_sgd_table_kernel<<<nblocks, 256, 0, stream>>>(table, reinterpret_cast<const int2*>(blocks_xy), h);
  return cudaGetLastError();
}

}  // namespace grace
