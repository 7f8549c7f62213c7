// Dense all-reduce through the NVSwitch multicast address of a symmetric buffer
// ("two-shot" in one kernel): every rank reduces its own 1/W slice with
// multimem.ld_reduce (the switch pulls the slice from all W GPUs and adds in
// flight) and broadcasts the scaled sum with multimem.st (the switch writes it
// into all W copies).  Per GPU and direction this moves (1 + 1/W)*N*4 bytes (a
// multimem load fetches the requester's own copy through the switch too), against
// 2*(W-1)/W*N*4 for a ring or a two-phase peer-load exchange and (W-1)*N*4 for a
// one-shot gather: it wins from four ranks on and loses at two.
//
//   P0  copy the local gradient into the symmetric buffer (skipped when the
//       caller's tensor already lives there)
//   P1  cross-GPU barrier: "my copy of the buffer is complete"
//   P2  slice reduce + broadcast over the multicast mapping
//   P3  cross-GPU barrier: "my slice has been written everywhere"
//   P4  copy the reduced buffer to the caller's output (skipped when in place)
//
// The reference sends uncompressed tensors through one library all-reduce per
// tensor (grace_dl/dist/communicator/allreduce.py:6-13); this kernel is the
// uncompressed path of the fused design.  Flags live on the symmetric heap and
// every wait is bounded, as in the other exchange kernels.
#include "common.cuh"
#include "exchange.h"

namespace grace {
namespace {

constexpr int kBlock = 512;
constexpr int kInFlight = 4;   // multimem loads issued per thread before the first is consumed

__device__ __forceinline__ float4 multimem_ld_reduce_add(const float4* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float4* mc, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// One cross-GPU rendezvous: CTA 0 raises this rank's flag on every peer, then
// every CTA waits (bounded) until all W flags in local memory reached `seq`.
__device__ __forceinline__ bool rendezvous(const DenseArgs& a, unsigned long long pad_off, bool ok, const Status& status,
                                           unsigned code) {
  const int tid = threadIdx.x;
  if (ok && blockIdx.x == 0 && tid < a.peers.world) {
    uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + pad_off) + a.peers.rank;
    st_release_sys(flag, a.peers.seq);
  }
  if (ok && tid < a.peers.world) {
    const uint64_t* mine = reinterpret_cast<const uint64_t*>(a.peers.heap[a.peers.rank] + pad_off) + tid;
    wait_flag_ge(mine, a.peers.seq, a.peers.timeout_ns, status, code, tid);
  }
  __syncthreads();
  return !status.failed();
}

__global__ void __launch_bounds__(kBlock, 1) dense_allreduce_kernel(const DenseArgs a) {
  const Status status{a.status};
  GridBarrier bar{a.barrier, 0u, a.peers.timeout_ns, status};
  const int tid = threadIdx.x;
  const long long gtid = (long long)blockIdx.x * kBlock + tid, gstride = (long long)gridDim.x * kBlock;
  const long long n4 = a.total / 4;
  float4* symm4 = reinterpret_cast<float4*>(a.symm);
  float4* mc4 = reinterpret_cast<float4*>(a.mc);

  // P0: stage the local gradient
  if (a.g != a.symm) {
    const float4* g4 = reinterpret_cast<const float4*>(a.g);
    for (long long i0 = gtid; i0 < n4; i0 += gstride * kInFlight) {   // kInFlight loads ahead of the stores
      float4 t[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) if (i0 + u * gstride < n4) t[u] = __ldcs(g4 + i0 + u * gstride);
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) if (i0 + u * gstride < n4) symm4[i0 + u * gstride] = t[u];
    }
  }
  bool ok = bar.sync();
  // P1
  ok = rendezvous(a, a.peers.ready_off, ok, status, kTimeoutPeerReady);
  // P2: this rank's slice, kInFlight vectors per thread at a time
  if (ok) {
    const long long chunk4 = (n4 + a.peers.world - 1) / a.peers.world;
    const long long lo = chunk4 * a.peers.rank;
    const long long hi = lo + chunk4 < n4 ? lo + chunk4 : n4;
    // software pipeline: the loads of the next batch are in flight while this batch is scaled and stored
    const long long step = gstride * kInFlight;
    float4 v[kInFlight];
    auto issue = [&](long long i0, float4 (&dst)[kInFlight]) {
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const long long i = i0 + u * gstride;
        if (i < hi) dst[u] = multimem_ld_reduce_add(mc4 + i);
      }
    };
    long long i0 = lo + gtid;
    if (i0 < hi) issue(i0, v);
    for (; i0 < hi; i0 += step) {
      float4 nv[kInFlight];
      if (i0 + step < hi) issue(i0 + step, nv);
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const long long i = i0 + u * gstride;
        if (i < hi) {
          v[u].x *= a.scale; v[u].y *= a.scale; v[u].z *= a.scale; v[u].w *= a.scale;
          multimem_st(mc4 + i, v[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) v[u] = nv[u];
    }
  }
  __threadfence_system();   // the multicast stores are ordered before the flag that follows the barrier
  ok = bar.sync();
  // P3
  ok = rendezvous(a, a.ready2_off, ok, status, kTimeoutPeerAck);
  // P4: hand the result to the caller (L1 is not coherent with the switch's writes: read through L2)
  if (ok && a.out != a.symm) {
    float4* out4 = reinterpret_cast<float4*>(a.out);
    for (long long i0 = gtid; i0 < n4; i0 += gstride * kInFlight) {
      uint4 t[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) if (i0 + u * gstride < n4) t[u] = ld_cg_u4(symm4 + i0 + u * gstride);
#pragma unroll
      for (int u = 0; u < kInFlight; ++u)
        if (i0 + u * gstride < n4)
          out4[i0 + u * gstride] = make_float4(__uint_as_float(t[u].x), __uint_as_float(t[u].y), __uint_as_float(t[u].z),
                                               __uint_as_float(t[u].w));
    }
  }
}

}  // namespace

int dense_max_grid(int device, int sm_limit) {
  int per_sm = 0, sms = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dense_allreduce_kernel, kBlock, 0);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  return per_sm * sms;
}

cudaError_t launch_dense_allreduce(const DenseArgs& a, int grid, cudaStream_t stream) {
  if (a.total % 4 != 0 || a.peers.world < 1 || a.peers.world > kMaxWorld || !a.symm || !a.mc) return cudaErrorInvalidValue;
  cudaError_t err = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (err != cudaSuccess) return err;
  void* params[] = {const_cast<DenseArgs*>(&a)};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dense_allreduce_kernel), dim3(grid), dim3(kBlock), params, 0,
                                     stream);
}

}  // namespace grace
