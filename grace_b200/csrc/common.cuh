// Shared device-side primitives: status words, bounded waits, grid barrier,
// cross-GPU signal flags, warp reductions and cache-bypassing vector loads.
//
// Rules every kernel in this directory follows:
//  * no wait is unbounded: each spin has a %globaltimer deadline; on expiry the
//    waiter records {code, detail} in the status block and every later phase of
//    the kernel becomes a no-op, so the kernel always returns and the context
//    stays usable;
//  * cross-GPU data is read with plain ld.global.cg from the peer mapping and
//    published with st.release.sys flags (never TMA from peer memory).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace grace {

constexpr int kMaxWorld = 16;

enum StatusCode : unsigned {
  kOk = 0,
  kTimeoutGridBarrier = 1,
  kTimeoutPeerReady = 2,
  kTimeoutPeerAck = 3,
  kSlotOverflow = 4,
  kBadArgument = 5,
  kTimeoutMbarrier = 6,
  kCheckFailed = 7,   // checked build (-DGRACE_CHECKED): an index or offset was out of range; the access was skipped
};

// Kernel identifiers recorded with a failed check.
enum KernelId : unsigned { kKernelSparse = 1, kKernelQuant = 2, kKernelLowRank = 3, kKernelDense = 4, kKernelSgd = 5 };

// Status block layout (unsigned words): [0] code (first error wins), [1] detail
// (peer rank or barrier index; source line of a failed check), [2] sequence number,
// [3] dropped-element count, [4] kernel id and [5], [6] the offending index of a
// failed check (checked build only).
struct Status {
  unsigned* words;
  __device__ __forceinline__ bool failed() const {
    return *reinterpret_cast<volatile unsigned*>(words) != kOk;
  }
  __device__ __forceinline__ void fail(unsigned code, unsigned detail, unsigned seq) const {
    if (atomicCAS(words, kOk, code) == kOk) {
      words[1] = detail;
      words[2] = seq;
      __threadfence_system();
    }
  }
  __device__ __forceinline__ void fail_check(unsigned kernel, unsigned line, unsigned long long index) const {
    if (atomicCAS(words, kOk, kCheckFailed) == kOk) {
      words[1] = line;
      words[4] = kernel;
      words[5] = (unsigned)index;
      words[6] = (unsigned)(index >> 32);
      __threadfence_system();
    }
  }
};

// Checked build: GRACE_IN_RANGE(status, kernel, index, limit) is true when index < limit; otherwise it records
// (kernel, source line, index) in the status block and is false, and the caller skips the access - nothing traps,
// the kernel runs to its end and the host raises at its next poll.  Stands in for a memory checker on the small
// shapes of the test-suite.  In the normal build the macro is the constant `true` and costs nothing.
#ifdef GRACE_CHECKED
#define GRACE_IN_RANGE(status, kernel, index, limit)                                                       \
  ((unsigned long long)(index) < (unsigned long long)(limit)                                               \
       ? true                                                                                              \
       : ((status).fail_check((kernel), __LINE__, (unsigned long long)(index)), false))
#else
#define GRACE_IN_RANGE(status, kernel, index, limit) true
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// 128-bit / 32-bit loads that bypass L1 (L1 is not coherent with peer writes).
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned ld_cg_u32(const void* p) {
  unsigned v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const void* p) { return __uint_as_float(ld_cg_u32(p)); }

// Grid-wide barrier for kernels launched cooperatively (all CTAs resident).
// `counter` is zeroed by the host before the launch; the k-th barrier of a
// kernel waits for k * gridDim.x arrivals.  Returns false after a timeout or if
// another CTA already recorded a failure; callers then skip their work but keep
// calling the barrier so that no CTA is left waiting.
struct GridBarrier {
  unsigned* counter;
  unsigned epoch;  // number of barriers passed so far (per thread copy, uniform)
  uint64_t timeout_ns;
  Status status;
  __device__ __forceinline__ bool sync() {
    epoch += 1;
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();  // also orders slot writes before a later cross-GPU release
      atomicAdd(counter, 1u);
      const unsigned target = epoch * gridDim.x;
      const uint64_t t0 = globaltimer_ns();
      unsigned spins = 0;
      while (ld_acquire_gpu(counter) < target) {
        if ((++spins & 0x3ff) == 0) {
          if (status.failed()) break;
          if (globaltimer_ns() - t0 > timeout_ns) {
            status.fail(kTimeoutGridBarrier, epoch, 0);
            break;
          }
        }
      }
    }
    __syncthreads();
    return !status.failed();
  }
};

// Wait until a 64-bit flag in local memory (written by a peer with
// st.release.sys) reaches `want`.  One thread calls this.
__device__ __forceinline__ bool wait_flag_ge(const uint64_t* flag, uint64_t want, uint64_t timeout_ns,
                                             const Status& status, unsigned code, unsigned detail) {
  const uint64_t t0 = globaltimer_ns();
  unsigned spins = 0;
  while (ld_acquire_sys(flag) < want) {
    if ((++spins & 0xff) == 0) {
      if (status.failed()) return false;
      if (globaltimer_ns() - t0 > timeout_ns) {
        status.fail(code, detail, (unsigned)want);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace grace
