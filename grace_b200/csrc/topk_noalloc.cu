// Allocation-free exact top-k by magnitude: see topk_noalloc.h for the
// contract.  Same algorithm as the compress phase of sparse_exchange.cu
// (histogram of the top 12 key bits, radix select over 12 + 12 + 7 bits on the
// device, compaction), restated for one tensor with caller-provided outputs and
// with all scratch in a static device array.
#include "topk_noalloc.h"

#include "common.cuh"

namespace {

using namespace grace;

constexpr int kBlock = 512;
constexpr int kBins = 4096;
constexpr int kIter = kBlock * 4;
constexpr int kStage = 2048;

// Work area layout (unsigned words).
struct Scratch {
  unsigned hist[kBins];
  unsigned prefix, need, tie_taken, out_count;
  unsigned barrier;
  unsigned status[4];
  unsigned pad[55];
};
static_assert(sizeof(Scratch) == kGraceTopkNoallocScratchBytes, "documented scratch size");

// The one and only work area of this entry point on each device.
static __device__ __align__(256) unsigned char g_scratch[kGraceTopkNoallocScratchBytes];

__device__ __forceinline__ void load4(const float* p, long long i, long long n, float (&v)[4]) {
  if (i + 4 <= n) {
    const float4 t = *reinterpret_cast<const float4*>(p + i);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (i + j < n) ? p[i + j] : 0.f;
  }
}

__global__ void __launch_bounds__(kBlock) topk_noalloc_kernel(const float* __restrict__ x, long long n, unsigned k,
                                                               float* __restrict__ values, int* __restrict__ indices,
                                                               Scratch* sc, unsigned long long timeout_ns) {
  __shared__ unsigned s_hist[kBins];
  __shared__ float s_val[kStage];
  __shared__ int s_idx[kStage];
  __shared__ unsigned s_scan[kBlock / 32];
  __shared__ unsigned s_count, s_base;
  const Status status{sc->status};
  GridBarrier bar{&sc->barrier, 0u, timeout_ns, status};
  const int tid = threadIdx.x;
  long long chunk = (n + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + kIter - 1) / kIter * kIter;
  const long long lo = (long long)blockIdx.x * chunk;
  const long long hi = lo + chunk < n ? lo + chunk : n;

  for (int b = tid; b < kBins; b += kBlock) s_hist[b] = 0;
  __syncthreads();

  bool ok = true;
  for (int level = 0; level < 3; ++level) {
    const int shift_prefix = level == 1 ? 19 : 7;
    const int shift_digit = level == 0 ? 19 : (level == 1 ? 7 : 0);
    const unsigned mask = level == 2 ? 0x7fu : 0xfffu;
    const unsigned prefix = level ? sc->prefix : 0u;
    if (ok) {
      for (long long i = lo + 4ll * tid; i < hi; i += kIter) {
        float v[4];
        load4(x, i, hi, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const unsigned key = __float_as_uint(v[j]) & 0x7fffffffu;
          if (i + j < hi && (level == 0 || (key >> shift_prefix) == prefix))
            atomicAdd(&s_hist[(key >> shift_digit) & mask], 1u);
        }
      }
      __syncthreads();
      for (int b = tid; b < kBins; b += kBlock) {
        const unsigned c = s_hist[b];
        if (c) { atomicAdd(&sc->hist[b], c); s_hist[b] = 0; }
      }
    }
    ok = bar.sync();
    if (ok && blockIdx.x == 0) {
      // suffix scan over the 4096 bins, 8 per thread, find the bin of the need-th largest key
      const unsigned need = level ? sc->need : k;
      unsigned c[8], local = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = sc->hist[tid * 8 + j]; sc->hist[tid * 8 + j] = 0; local += c[j]; }
      const int lane = tid & 31, warp = tid >> 5;
      unsigned incl = local;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += t;
      }
      if (lane == 0) s_scan[warp] = incl;
      __syncthreads();
      unsigned above = incl - local;
      for (int w = warp + 1; w < kBlock / 32; ++w) above += s_scan[w];
      if (above < need && need <= above + local) {
        unsigned cum = above;
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          if (cum < need && need <= cum + c[j]) {
            sc->prefix = (prefix << (level == 2 ? 7 : 12)) | (unsigned)(tid * 8 + j);
            sc->need = need - cum;
          }
          cum += c[j];
        }
      }
      __syncthreads();
    }
    ok = bar.sync();
  }

  // compaction: keys above the pivot, plus `need` of the keys equal to it
  const unsigned pivot = sc->prefix, need = sc->need;
  if (tid == 0) s_count = 0;
  __syncthreads();
  auto flush = [&]() {
    __syncthreads();
    const unsigned cnt = s_count;
    if (tid == 0) s_base = cnt ? atomicAdd(&sc->out_count, cnt) : 0u;
    __syncthreads();
    for (unsigned e = tid; e < cnt; e += kBlock) {
      const unsigned pos = s_base + e;
      if (pos < k) { values[pos] = s_val[e]; indices[pos] = s_idx[e]; }
    }
    __syncthreads();
    if (tid == 0) s_count = 0;
    __syncthreads();
  };
  if (ok) {
    const long long iters = lo < hi ? (hi - lo + kIter - 1) / kIter : 0;
    for (long long it = 0; it < iters; ++it) {
      const long long i = lo + it * kIter + 4ll * tid;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (i < hi) load4(x, i, hi, v);
      unsigned m = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (i + j >= hi) continue;
        const unsigned key = __float_as_uint(v[j]) & 0x7fffffffu;
        bool sel = key > pivot;
        if (key == pivot) sel = atomicAdd(&sc->tie_taken, 1u) < need;
        if (sel) m |= 1u << j;
      }
      // at most kIter (2048) selections per iteration: exactly the staging capacity
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (m & (1u << j)) {
          const unsigned pos = atomicAdd(&s_count, 1u);
          s_val[pos] = v[j];
          s_idx[pos] = (int)(i + j);
        }
      flush();
    }
  }
}

struct DeviceSetup {
  bool ready;
  Scratch* scratch;
  int max_grid;
};
DeviceSetup g_setup[64] = {};

}  // namespace

extern "C" const char* grace_topk_noalloc_strerror(int code) {
  switch (code) {
    case GRACE_NOALLOC_OK: return "ok";
    case GRACE_NOALLOC_BAD_ARGUMENT: return "bad argument: need non-null x (16-byte aligned), values and indices, and 1 <= k <= n";
    case GRACE_NOALLOC_TOO_LARGE: return "input too large: n exceeds 2^31 - 1 elements";
    case GRACE_NOALLOC_SETUP_FAILED: return "set-up failed: could not resolve the device work area or the launch geometry";
    case GRACE_NOALLOC_LAUNCH_FAILED: return "launch failed: the memset or the kernel launch was refused";
  }
  return "unknown code";
}

extern "C" int grace_topk_select_noalloc(const float* x, long long n, int k, float* values, int* indices, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (n > kGraceTopkNoallocMaxElems) return GRACE_NOALLOC_TOO_LARGE;
  if (!x || !values || !indices || n < 1 || k < 1 || (long long)k > n || (reinterpret_cast<uintptr_t>(x) & 15))
    return GRACE_NOALLOC_BAD_ARGUMENT;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GRACE_NOALLOC_SETUP_FAILED;
  DeviceSetup& s = g_setup[dev];
  if (!s.ready) {
    // Once per device, with that device current: the name g_scratch is only a
    // host-side handle; kernels need the address it has on this device.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || p == nullptr) return GRACE_NOALLOC_SETUP_FAILED;
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, topk_noalloc_kernel, kBlock, 0) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1 || sms < 1)
      return GRACE_NOALLOC_SETUP_FAILED;
    s.scratch = static_cast<Scratch*>(p);
    s.max_grid = per_sm * sms;
    s.ready = true;
  }
  // The work area still holds the previous call's state: clear all of it.
  if (cudaMemsetAsync(s.scratch, 0, sizeof(Scratch), stream) != cudaSuccess) {
    cudaGetLastError();
    return GRACE_NOALLOC_LAUNCH_FAILED;
  }
  long long need = (n + kIter - 1) / kIter;
  int grid = (int)(need < (long long)s.max_grid ? need : (long long)s.max_grid);
  if (grid < 1) grid = 1;
  unsigned uk = (unsigned)k;
  Scratch* sc = s.scratch;
  unsigned long long timeout_ns = 10ull * 1000 * 1000 * 1000;
  void* params[] = {&x, &n, &uk, &values, &indices, &sc, &timeout_ns};
  if (cudaLaunchCooperativeKernel((const void*)topk_noalloc_kernel, dim3(grid), dim3(kBlock), params, 0, stream) !=
      cudaSuccess) {
    cudaGetLastError();   // the refusal is reported through the return code; do not leave it for the caller's next check
    return GRACE_NOALLOC_LAUNCH_FAILED;
  }
  return GRACE_NOALLOC_OK;
}

extern "C" int grace_topk_noalloc_status(unsigned out[4], void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int dev = 0;
  if (!out || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_setup[dev].ready)
    return GRACE_NOALLOC_SETUP_FAILED;
  // the address resolved at set-up; the host-side name g_scratch would be the wrong thing to copy from
  const Scratch* sc = g_setup[dev].scratch;
  if (cudaMemcpyAsync(out, sc->status, 4 * sizeof(unsigned), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    cudaGetLastError();
    return GRACE_NOALLOC_LAUNCH_FAILED;
  }
  return GRACE_NOALLOC_OK;
}
