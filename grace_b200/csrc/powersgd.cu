// Fused PowerSGD exchange on sm_100a: low-rank projections on the 5th-gen
// tensor cores (tcgen05.mma, TF32 operands, fp32 accumulators in TMEM), tiles
// staged by TMA, both all-reduces done inside the kernel by loading the peers'
// partial results over NVLink.
//
// For every matrix M (n x m, row-major slice of the flat gradient buffer) of a
// launch, with rank r <= 8 padded to 16 columns:
//   S1  M' = G + R (error feedback; added in shared memory on the swizzled
//       tiles and written back by a TMA store), P = M' * Q: A = M' tile
//       [128 x 32] K-major, B = Q^T tile [16 x 32] K-major, D in TMEM
//       (128 lanes x 16 columns); split-K partial sums are added into this
//       rank's P slot on the symmetric heap;
//   R1  publish; wait for every peer; P = mean over ranks of the W slots
//       (identical order on every rank, so the results are bit-identical);
//       Gram matrix P^T P accumulated on the way;
//   O   orthogonalise P: Cholesky factor of the Gram matrix in fp64, P R^-1
//       (what modified Gram-Schmidt computes in exact arithmetic), written
//       transposed for the next stage;
//   S2  Q = M'^T * P: TMA brings 32 rows x 128 columns of M' (four unswizzled
//       boxes); the CTA transposes them in shared memory into a K-major
//       128B-swizzled A tile [128 x 32] (the TF32 MMA returns zeros for an
//       MN-major A operand on this part, so the transpose is done by hand),
//       B = P^T tile [16 x 32] K-major, D [128 x 16] in TMEM;
//   R2  publish; wait; Q = mean over ranks; kept as next step's warm start;
//   S3  out = P Q^T (rank-r outer products on CUDA cores), R = M' - out.
//
// Every mbarrier / flag / grid-barrier wait is bounded; TMA loads never use
// cluster multicast and never read peer memory (peers are read with ld.cg).
//
// Replaces, in the reference: compressor/powersgd.py:21-65 (three cuBLAS
// SGEMMs, TorchScript Gram-Schmidt, two NCCL all-reduces) and
// memory/powersgd.py:12-37.
#include <cuda.h>

#include "common.cuh"
#include "exchange.h"

namespace grace {

namespace {

constexpr int kThreads = 256;
constexpr int kStages = 6;             // 6 x (16 + 16 + 2) KiB ring per CTA (one CTA per SM: the runtime reports one resident CTA for this kernel at any shared-memory size)
constexpr int kTileRows = 128;          // MMA M
constexpr int kTileK = 32;              // fp32 elements per 128-byte swizzle row
constexpr int kRankPad = 16;            // MMA N
constexpr int kATileBytes = kTileRows * kTileK * 4;   // 16 KiB
constexpr int kBTileBytes = kRankPad * kTileK * 4;    // 2 KiB
constexpr int kKTilesPerItem = 16;      // split-K granularity: 512 columns (S1) / 512 rows (S2)
constexpr unsigned kTmemCols = 32;
constexpr int kProducerThread = 32;      // lane 0 of warp 1: TMA loads and stores
constexpr int kMaxRank = 8;              // ranks 1..8 (buffers are padded to kRankPad columns)
constexpr int kS3Trip = 16;             // rows whose loads are in flight together in stage 3
constexpr int kS3Rows = 64;             // rows per stage-3 work item

// instruction descriptor: D=f32, A=B=tf32, N=16, M=128 (bit layout: c_format
// [4,6), a_format [7,10), b_format [10,13), a_major 15, b_major 16, N>>3
// [17,23), M>>4 [24,29))
constexpr uint32_t kIdescS1 = (1u << 4) | (2u << 7) | (2u << 10) | ((kRankPad >> 3) << 17) | ((kTileRows >> 4) << 24);

struct __align__(1024) SmemLayout {
  unsigned char a[kStages][kATileBytes];   // gradient tile, becomes the A operand
  unsigned char r[kStages][kATileBytes];   // stage 1: residual tile; stage 2: unswizzled M' boxes before the transpose
  unsigned char b[kStages][kBTileBytes];   // Q^T / P^T tile
  unsigned long long full[kStages];
  unsigned long long mma_done[kStages];
  unsigned long long item_done;
  unsigned tmem_base;
  int bail;
  double gram[kMaxRank][kMaxRank];
  double rinv[kMaxRank][kMaxRank];
  float prow[kS3Rows][kMaxRank];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; returns false (and records the failure) when the limit expires.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, uint64_t timeout_ns, const Status& status,
                                          unsigned detail) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3f) == 0) {
      if (status.failed()) return false;
      if (globaltimer_ns() - t0 > timeout_ns) {
        status.fail(kTimeoutMbarrier, detail, 0);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(src)) : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // start>>4 [0,14) | LBO>>4 [16,30) | SBO>>4 [32,46) | version 1 [46,48) | SWIZZLE_128B (2) [61,64)
  return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"((unsigned)accum) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Work item of a GEMM stage: (matrix, block of 128 output rows, K split).
struct Item {
  int mat, blk, kt0, kt1;
};
__device__ __forceinline__ bool decode_item(const LowRankArgs& a, int stage, int idx, Item& it) {
  const int total = stage == 1 ? a.items_s1 : a.items_s2;
  if (idx >= total) return false;
  int mat = 0;
  while (mat + 1 < a.nmat && (stage == 1 ? a.mats[mat + 1].item1_begin : a.mats[mat + 1].item2_begin) <= idx) ++mat;
  const LowRankMatrix& M = a.mats[mat];
  const int local = idx - (stage == 1 ? M.item1_begin : M.item2_begin);
  const int ktiles = ((stage == 1 ? M.m : M.n) + kTileK - 1) / kTileK;
  const int splits = (ktiles + kKTilesPerItem - 1) / kKTilesPerItem;
  it.mat = mat;
  it.blk = local / splits;
  it.kt0 = (local % splits) * kKTilesPerItem;
  it.kt1 = min(it.kt0 + kKTilesPerItem, ktiles);
  return true;
}

// One GEMM stage over this CTA's items.  STAGE 1: P += M' Q.  STAGE 2: Q += M'^T P.
template <int STAGE>
__device__ void gemm_stage(const LowRankArgs& a, SmemLayout& sm, const Status& status, float* __restrict__ dst_slot,
                           unsigned& step_counter, unsigned& item_counter) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool add_residual = STAGE == 1 && a.has_memory;
  const uint32_t tmem_d = sm.tmem_base;
  const unsigned tile_bytes = kATileBytes + kBTileBytes + (add_residual ? kATileBytes : 0);

  // producer cursor (thread 0) and consumer cursor (all threads) walk the same sequence of (item, k-tile)
  int p_item = blockIdx.x, c_item = blockIdx.x;
  Item pit, cit;
  bool p_valid = decode_item(a, STAGE, p_item, pit);
  bool c_valid = decode_item(a, STAGE, c_item, cit);
  int p_kt = p_valid ? pit.kt0 : 0, c_kt = c_valid ? cit.kt0 : 0;
  unsigned p_step = step_counter, c_step = step_counter;

  // Two single-thread roles run side by side after each CTA barrier: thread 0 issues the MMAs,
  // thread kProducerThread issues the TMA store of M' and refills the ring.
  auto produce = [&]() {  // producer thread only: issue the TMA loads of the next (item, k-tile)
    if (!p_valid) return;
    const unsigned slot = p_step % kStages;
    if (p_step >= kStages) {
      // the MMAs that read this slot kStages steps ago must have retired, and the
      // TMA store that read its A tile must be done reading
      if (!mbar_wait(&sm.mma_done[slot], ((p_step / kStages) - 1) & 1, a.peers.timeout_ns, status, 100 + slot)) {
        p_valid = false;
        return;
      }
      tma_wait_read1();  // all of this thread's stores except the newest one have read their tile
    }
    const LowRankMatrix& M = a.mats[pit.mat];
    const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(a.maps) + (size_t)pit.mat * kMapsPerMatrix;
    mbar_expect_tx(&sm.full[slot], tile_bytes);
    if (STAGE == 1) {
      tma_load_2d(sm.a[slot], maps + kMapG1, p_kt * kTileK, pit.blk * kTileRows, &sm.full[slot]);
      if (add_residual) tma_load_2d(sm.r[slot], maps + kMapA1, p_kt * kTileK, pit.blk * kTileRows, &sm.full[slot]);
      tma_load_2d(sm.b[slot], maps + kMapQt, p_kt * kTileK, 0, &sm.full[slot]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)  // four unswizzled boxes of 32 columns x 32 rows of M'
        tma_load_2d(sm.r[slot] + j * 4096, maps + kMapM2, pit.blk * kTileRows + j * 32, p_kt * kTileK, &sm.full[slot]);
      tma_load_2d(sm.b[slot], maps + kMapPt, p_kt * kTileK, 0, &sm.full[slot]);
    }
    (void)M;
    ++p_step;
    if (++p_kt >= pit.kt1) {
      p_item += gridDim.x;
      p_valid = decode_item(a, STAGE, p_item, pit);
      p_kt = p_valid ? pit.kt0 : 0;
    }
  };

  if (tid == kProducerThread) {
    for (int i = 0; i < kStages - 1; ++i) produce();
  }

  long long t_wait = 0, t_work = 0, t_sync = 0, t_issue = 0, t_fence = 0, t_commit = 0;
  const bool prof = (a.part & 0x100) && blockIdx.x == 0 && tid == 0;
  while (c_valid) {
    const unsigned slot = c_step % kStages;
    long long t0 = prof ? clock64() : 0;
    bool ok = mbar_wait(&sm.full[slot], (c_step / kStages) & 1, a.peers.timeout_ns, status, 200 + slot);
    if (prof) { const long long t1 = clock64(); t_wait += t1 - t0; t0 = t1; }
    if (add_residual && ok) {
      float4* pa = reinterpret_cast<float4*>(sm.a[slot]);
      const float4* pr = reinterpret_cast<const float4*>(sm.r[slot]);
#pragma unroll
      for (int i = 0; i < kATileBytes / 16 / kThreads; ++i) {
        float4 x = pa[tid + i * kThreads];
        const float4 y = pr[tid + i * kThreads];
        x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
        pa[tid + i * kThreads] = x;
      }
      fence_async_smem();  // generic-proxy writes -> visible to the TMA store and the MMA
    }
    if (STAGE == 2 && ok) {
      // transpose: staging[j][k][mi] (k = row of M', 32 per tile; m = 32*j + mi) -> A[m][k], K-major with the
      // 128-byte swizzle (16-byte chunk index XOR row % 8).  One 4 x 4 block per thread.
      // Thread -> block mapping chosen so that both sides are free of bank conflicts: the eight
      // lanes of a quarter warp read eight different 16-byte chunks of the staging rows, and their
      // swizzled destination chunks (kq ^ row % 8) are eight different values as well.
      const int l8 = tid & 7, rest = tid >> 3;
      const int mq = (rest & 3) * 8 + l8;             // m / 4
      const int kq = (l8 >> 1) ^ (rest >> 2);         // k / 4
      const int j = mq >> 3, mi4 = (mq & 7) * 4;
      const unsigned char* st = sm.r[slot] + j * 4096 + mi4 * 4;
      float4 rowv[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) rowv[kk] = *reinterpret_cast<const float4*>(st + (kq * 4 + kk) * 128);
      const float t[4][4] = {{rowv[0].x, rowv[1].x, rowv[2].x, rowv[3].x}, {rowv[0].y, rowv[1].y, rowv[2].y, rowv[3].y},
                             {rowv[0].z, rowv[1].z, rowv[2].z, rowv[3].z}, {rowv[0].w, rowv[1].w, rowv[2].w, rowv[3].w}};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int mrow = mq * 4 + e;
        *reinterpret_cast<float4*>(sm.a[slot] + mrow * 128 + ((kq ^ (mrow & 7)) << 4)) =
            make_float4(t[e][0], t[e][1], t[e][2], t[e][3]);
      }
      fence_async_smem();
    }
    if (!ok) sm.bail = 1;
    if (prof) { const long long t1 = clock64(); t_work += t1 - t0; t0 = t1; }
    __syncthreads();
    if (prof) { const long long t1 = clock64(); t_sync += t1 - t0; t0 = t1; }
    if (sm.bail) break;
    const bool last_kt = (c_kt + 1 >= cit.kt1);
    if (tid == kProducerThread) {
      if (add_residual) {  // M' goes back to the accumulator buffer
        const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(a.maps) + (size_t)cit.mat * kMapsPerMatrix;
        tma_store_2d(maps + kMapA1, c_kt * kTileK, cit.blk * kTileRows, sm.a[slot]);
        tma_commit();
      }
      // refill the slot used one step ago: its MMAs were issued a whole iteration earlier, so the
      // wait inside produce() rarely stalls
      produce();
    }
    if (tid == 0) {
      tc_fence_after();
      if (prof) { const long long t1 = clock64(); t_fence += t1 - t0; t0 = t1; }
      const uint32_t a_addr = smem_u32(sm.a[slot]), b_addr = smem_u32(sm.b[slot]);
#pragma unroll
      for (int kk = 0; kk < kTileK / 8; ++kk) {
        const uint64_t adesc = smem_desc(a_addr + kk * 32, 16, 1024);   // K-major: 32 B per K step of 8
        const uint64_t bdesc = smem_desc(b_addr + kk * 32, 16, 1024);
        umma_tf32(tmem_d, adesc, bdesc, kIdescS1, !(c_kt == cit.kt0 && kk == 0));
      }
      if (prof) { const long long t1 = clock64(); t_issue += t1 - t0; t0 = t1; }
      umma_commit(&sm.mma_done[slot]);
      if (last_kt) umma_commit(&sm.item_done);
      if (prof) { const long long t1 = clock64(); t_commit += t1 - t0; t0 = t1; }
    }
    ++c_step;
    if (last_kt) {
      // ---- epilogue: TMEM -> registers -> red.add into this rank's slot ----
      ok = mbar_wait(&sm.item_done, item_counter & 1, a.peers.timeout_ns, status, 300);
      ++item_counter;
      if (!ok) sm.bail = 1;
      __syncthreads();
      if (sm.bail) break;
      tc_fence_after();
      if (warp < 4) {
        uint32_t v[16];
        const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const LowRankMatrix& M = a.mats[cit.mat];
        const int row = cit.blk * kTileRows + warp * 32 + lane;
        const int rows = STAGE == 1 ? M.n : M.m;
        if (row < rows) {
          float* dst = dst_slot + (STAGE == 1 ? M.p_off : M.q_off) + (size_t)row * kRankPad;
#pragma unroll
          for (int c = 0; c < kRankPad; ++c)
            if (c < a.rank) atomicAdd(dst + c, __uint_as_float(v[c]));
        }
      }
      tc_fence_before();
      __syncthreads();  // TMEM reads done before the next item's first MMA overwrites the accumulator
      c_item += gridDim.x;
      c_valid = decode_item(a, STAGE, c_item, cit);
      c_kt = c_valid ? cit.kt0 : 0;
      if (prof) { const long long t1 = clock64(); t_commit += t1 - t0; t0 = t1; }
    } else {
      ++c_kt;
    }
  }
  if (prof) {
    unsigned* w = a.status + 8 + (STAGE - 1) * 8;
    w[0] = (unsigned)(t_wait >> 4); w[1] = (unsigned)(t_work >> 4); w[2] = (unsigned)(t_sync >> 4);
    w[3] = (unsigned)(t_issue >> 4); w[4] = (unsigned)(t_fence >> 4); w[5] = (unsigned)(t_commit >> 4); w[6] = c_step;
  }
  // drain: every issued load must land and every store must finish before smem is reused
  if (tid == kProducerThread) {
    tma_wait_all0();
    while (c_step < p_step && !sm.bail) {  // loads issued ahead of a bail-out
      mbar_wait(&sm.full[c_step % kStages], (c_step / kStages) & 1, a.peers.timeout_ns, status, 400);
      ++c_step;
    }
  }
  __syncthreads();
  step_counter = c_step;  // uniform: every thread consumed the same steps
}

// Mean over ranks of a [rows x 16] region; optional Gram matrix per matrix.
__device__ void reduce_region(const LowRankArgs& a, size_t region_off, float* __restrict__ dst, size_t floats) {
  const int world = a.peers.world;
  const float inv = 1.f / (float)a.divisor;
  for (size_t i = ((size_t)blockIdx.x * kThreads + threadIdx.x) * 4; i < floats; i += (size_t)gridDim.x * kThreads * 4) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {
      const uint4 v = ld_cg_u4(a.peers.heap[p] + a.peers.slot_off + (region_off + i) * 4);
      s.x += __uint_as_float(v.x); s.y += __uint_as_float(v.y); s.z += __uint_as_float(v.z); s.w += __uint_as_float(v.w);
    }
    s.x *= inv; s.y *= inv; s.z *= inv; s.w *= inv;
    *reinterpret_cast<float4*>(dst + i) = s;
  }
}

__device__ bool publish_and_wait(const LowRankArgs& a, const Status& status, unsigned long long ready_off,
                                 bool do_publish, bool do_wait) {
  // called by all threads of all CTAs after a grid barrier
  __shared__ int s_ok;
  const int tid = threadIdx.x, rank = a.peers.rank, world = a.peers.world;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && tid < world && do_publish && !status.failed()) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint64_t*>(a.peers.heap[tid] + ready_off) + rank, a.peers.seq);
  }
  if (do_wait) {
    if (tid < world) {
      const uint64_t* flag = reinterpret_cast<const uint64_t*>(a.peers.heap[rank] + ready_off) + tid;
      if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(kThreads, 1) powersgd_kernel(const LowRankArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const Status status{a.status};
  GridBarrier bar{a.barrier, 0u, a.peers.timeout_ns, status};
  const int tid = threadIdx.x, warp = tid >> 5;
  const int rank = a.peers.rank, world = a.peers.world;
  float* const my_slot = reinterpret_cast<float*>(a.peers.heap[rank] + a.peers.slot_off);
  float* const slot_p = my_slot;                 // [p_floats]
  float* const slot_q = my_slot + a.p_floats;    // [q_floats]

  // ---- set-up: barriers, TMEM ----
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.mma_done[s], 1); }
    mbar_init(&sm.item_done, 1);
    sm.bail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  unsigned steps = 0, items = 0;

  // Phase groups (bit mask in a.phases, same meaning as the other exchanges):
  //   compress: S1 ... exchange happens twice inside; a single launch runs
  //   everything, the split launches of the one-GPU emulation run
  //   [S1 | publish P] [reduce P, O, S2 | publish Q] [reduce Q, S3] as three
  //   launches selected by a.part (0 = all, 1..3 = that part only).
  const int part = a.part & 0xff;   // bit 8 of a.part asks CTA 0 to record per-phase cycle counts in status[8..]: wait, smem work, barrier, MMA issue, fence, commit + epilogue, steps (units of 16 cycles)
  const bool part1 = part == 0 || part == 1;
  const bool part2 = part == 0 || part == 2;
  const bool part3 = part == 0 || part == 3;
  bool ok = true;

  if (part1) {
    if (tid < world && tid != rank && a.peers.seq > 2) {   // every CTA: none may zero the slot before the peers are done with it
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(a.peers.heap[rank] + a.peers.ack_off) + tid;
      wait_flag_ge(ack, a.peers.seq - 2, a.peers.timeout_ns, status, kTimeoutPeerAck, tid);
    }
    __syncthreads();
    // zero this rank's partial-sum slot (P and Q regions)
    const size_t nfl = (size_t)a.p_floats + a.q_floats;
    for (size_t i = ((size_t)blockIdx.x * kThreads + tid) * 4; i < nfl; i += (size_t)gridDim.x * kThreads * 4)
      *reinterpret_cast<float4*>(my_slot + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (blockIdx.x == 0)
      for (int i = tid; i < a.nmat * kRankPad * kRankPad; i += kThreads) a.gram[i] = 0.0;
    ok = bar.sync();
    if (ok) gemm_stage<1>(a, sm, status, slot_p, steps, items);
    fence_async_all();
    ok = bar.sync();
  }

  if (part1 || part2) {
    // publish P (part 1) / wait for the peers' P (part 2)
    ok = publish_and_wait(a, status, a.peers.ready_off, part1, part2) && ok && !status.failed();
  }

  if (part2) {
    if (ok) {
      // P = mean over ranks; Gram matrices
      reduce_region(a, 0, a.p_mean, a.p_floats);
    }
    ok = bar.sync() && ok;
    if (ok) {
      // Gram: one thread per row, shared-memory fp64 accumulation per matrix
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        for (int i = tid; i < kMaxRank * kMaxRank; i += kThreads) (&sm.gram[0][0])[i] = 0.0;
        __syncthreads();
        for (int row = blockIdx.x * kThreads + tid; row < M.n; row += gridDim.x * kThreads) {
          const float* pr = a.p_mean + M.p_off + (size_t)row * kRankPad;
          float v[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] = c < a.rank ? pr[c] : 0.f;
#pragma unroll
          for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int d = c; d < 8; ++d)
              if (d < a.rank) atomicAdd(&sm.gram[c][d], (double)v[c] * (double)v[d]);
        }
        __syncthreads();
        if (tid < kMaxRank * kMaxRank) {
          const int c = tid / kMaxRank, d = tid % kMaxRank;
          if (c <= d && d < a.rank && sm.gram[c][d] != 0.0)
            atomicAdd(&a.gram[(size_t)mat * 256 + c * kRankPad + d], sm.gram[c][d]);
        }
        __syncthreads();
      }
    }
    ok = bar.sync() && ok;
    if (ok) {
      // O: P_orth = P R^-1 with R^T R = Gram (upper Cholesky), written transposed [16][n]
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        if (tid == 0) {
          const int r = a.rank;
          double R[8][8] = {};
          const double* G = a.gram + (size_t)mat * 256;
          for (int j = 0; j < r; ++j) {
            for (int i = 0; i <= j; ++i) {
              double s = G[i * kRankPad + j];
              for (int k = 0; k < i; ++k) s -= R[k][i] * R[k][j];
              if (i == j) R[i][j] = s > 0.0 ? sqrt(s) : 0.0;
              else R[i][j] = R[i][i] > 0.0 ? s / R[i][i] : 0.0;
            }
          }
          // invert the upper-triangular R by back substitution
          for (int j = 0; j < r; ++j) {
            for (int i = 0; i < r; ++i) sm.rinv[i][j] = 0.0;
            if (R[j][j] > 0.0) sm.rinv[j][j] = 1.0 / R[j][j];
            for (int i = j - 1; i >= 0; --i) {
              double s = 0.0;
              for (int k = i + 1; k <= j; ++k) s += R[i][k] * sm.rinv[k][j];
              sm.rinv[i][j] = R[i][i] > 0.0 ? -s / R[i][i] : 0.0;
            }
          }
        }
        __syncthreads();
        for (int row = blockIdx.x * kThreads + tid; row < M.n; row += gridDim.x * kThreads) {
          const float* pr = a.p_mean + M.p_off + (size_t)row * kRankPad;
          float v[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] = c < a.rank ? pr[c] : 0.f;
          for (int c = 0; c < a.rank; ++c) {
            double s = 0.0;
            for (int k = 0; k <= c; ++k) s += (double)v[k] * sm.rinv[k][c];
            a.pt_orth[M.pt_off + (size_t)c * M.n + row] = (float)s;
          }
        }
        __syncthreads();
      }
    }
    fence_async_all();  // pt_orth is read by TMA next
    ok = bar.sync() && ok;
    if (ok) gemm_stage<2>(a, sm, status, slot_q, steps, items);
    ok = bar.sync() && ok;
  }

  if (part2 || part3) {
    ok = publish_and_wait(a, status, a.ready2_off, part2, part3) && ok && !status.failed();
  }

  if (part3) {
    if (ok) reduce_region(a, a.p_floats, a.q_mean, a.q_floats);
    ok = bar.sync() && ok;
    // acknowledge: both slot regions of this sequence have been read
    if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
      uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
      st_release_sys(ack, a.peers.seq);
    }
    if (ok) {
      // keep Q^T (warm start of the next step, B operand of S1)
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        for (int j = blockIdx.x * kThreads + tid; j < M.m; j += gridDim.x * kThreads) {
          const float* qr = a.q_mean + M.q_off + (size_t)j * kRankPad;
          for (int c = 0; c < a.rank; ++c) a.qt[M.qt_off + (size_t)c * M.m + j] = qr[c];
        }
      }
      // S3: out = P Q^T, residual = M' - out.  Item = kS3Rows rows x 1024 columns.
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        const float* __restrict__ src = a.has_memory ? a.acc : a.g;
        const int row_blocks = (M.n + kS3Rows - 1) / kS3Rows, col_blocks = (M.m + 1023) / 1024;
        for (int item = blockIdx.x; item < row_blocks * col_blocks; item += gridDim.x) {
          const int rb = item / col_blocks, cb = item % col_blocks;
          __syncthreads();
          for (int i = tid; i < kS3Rows * kMaxRank; i += kThreads) {
            const int rr = i / kMaxRank, c = i % kMaxRank, row = rb * kS3Rows + rr;
            sm.prow[rr][c] = (row < M.n && c < a.rank) ? a.pt_orth[M.pt_off + (size_t)c * M.n + row] : 0.f;
          }
          __syncthreads();
          const int col = cb * 1024 + tid * 4;
          if (col < M.m) {
            const int valid = min(4, M.m - col);
            float q[4][8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float4 lo4 = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo4;
              if (e < valid) {   // columns >= rank of q_mean are zero
                const float4* qp = reinterpret_cast<const float4*>(a.q_mean + M.q_off + (size_t)(col + e) * kRankPad);
                lo4 = qp[0];
                if (a.rank > 4) hi4 = qp[1];
              }
              q[e][0] = lo4.x; q[e][1] = lo4.y; q[e][2] = lo4.z; q[e][3] = lo4.w;
              q[e][4] = hi4.x; q[e][5] = hi4.y; q[e][6] = hi4.z; q[e][7] = hi4.w;
            }
            const int rows = min(kS3Rows, M.n - rb * kS3Rows);
            const bool vec = valid == 4 && (M.m & 3) == 0;
            for (int r0 = 0; r0 < rows; r0 += kS3Trip) {
              // kS3Trip rows per trip: issue the loads of M' first, then compute and store
              float4 mv[kS3Trip];
#pragma unroll
              for (int u = 0; u < kS3Trip; ++u) {
                mv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r0 + u < rows && a.has_memory && vec)
                  mv[u] = *reinterpret_cast<const float4*>(src + (size_t)M.g_off + (size_t)(rb * kS3Rows + r0 + u) * M.m + col);
              }
#pragma unroll
              for (int u = 0; u < kS3Trip; ++u) {
                const int rr = r0 + u;
                if (rr >= rows) break;
                const size_t base = (size_t)M.g_off + (size_t)(rb * kS3Rows + rr) * M.m + col;
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float s = 0.f;
#pragma unroll
                  for (int c = 0; c < 8; ++c) s += sm.prow[rr][c] * q[e][c];
                  o[e] = s;
                }
                if (vec) {
                  if (a.has_memory)
                    *reinterpret_cast<float4*>(a.acc + base) =
                        make_float4(mv[u].x - o[0], mv[u].y - o[1], mv[u].z - o[2], mv[u].w - o[3]);
                  *reinterpret_cast<float4*>(a.out + base) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
                  for (int e = 0; e < valid; ++e) {
                    const float m1 = src[base + e];
                    if (a.has_memory) a.acc[base + e] = m1 - o[e];
                    a.out[base + e] = o[e];
                  }
                }
              }
            }
          }
        }
      }
    }
  }

  // ---- teardown ----
  __syncthreads();
  if (tid == kProducerThread) tma_wait_all0();
  tc_fence_before();
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(kTmemCols) : "memory");
}

}  // namespace

size_t lowrank_smem_bytes() { return sizeof(SmemLayout) + 1024; }

int lowrank_max_grid(int device, int sm_limit) {
  static bool attr_set[64] = {};
  if (device >= 0 && device < 64 && !attr_set[device]) {
    cudaFuncSetAttribute(powersgd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lowrank_smem_bytes());
    attr_set[device] = true;
  }
  int per_sm = 0, sms = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, powersgd_kernel, kThreads, lowrank_smem_bytes());
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  if (per_sm > 1) per_sm = 1;
  return per_sm * sms;
}

// Resident CTAs per SM the runtime reports for a given dynamic shared-memory size (tuning aid).
int lowrank_occupancy(int dynamic_smem_bytes) {
  cudaFuncSetAttribute(powersgd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_smem_bytes);
  int per_sm = -1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, powersgd_kernel, kThreads, dynamic_smem_bytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return per_sm;
}

cudaError_t launch_powersgd(const LowRankArgs& a, int grid, cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (err != cudaSuccess) return err;
  LowRankArgs copy = a;
  void* params[] = {&copy};
  return cudaLaunchCooperativeKernel((const void*)powersgd_kernel, dim3(grid), dim3(kThreads), params,
                                     lowrank_smem_bytes(), stream);
}

// Host: encode the five tensor maps of one matrix.
//   G1 : gradient, box 32 x 128 (stage-1 A operand)
//   A1 : accumulator, box 32 x 128 (residual load, M' store)
//   M2 : M' (accumulator, or gradient without memory), box 32 x 32, not swizzled (transposed by the CTA in stage 2)
//   Qt : Q^T [16][m], box 32 x 16;  Pt : P^T [16][n], box 32 x 16
int lowrank_encode_maps(void* maps_out, const float* g, float* acc, const float* qt, const float* pt, int n, int m) {
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(maps_out);
  // The driver entry point is looked up at run time so that the extension does
  // not link against libcuda (it must import on machines without a driver).
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode_fn = nullptr;
  if (!encode_fn) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
      return -1;
    encode_fn = reinterpret_cast<EncodeFn>(fn);
  }
  EncodeFn cuTensorMapEncodeTiled_rt = encode_fn;
  auto enc = [cuTensorMapEncodeTiled_rt](CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                uint32_t box_outer, bool swizzle = true) -> CUresult {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 4};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return cuTensorMapEncodeTiled_rt(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r;
  if ((r = enc(maps + kMapG1, g, m, n, 32, 128)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapA1, acc ? acc : g, m, n, 32, 128)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapM2, acc ? acc : g, m, n, 32, 32, false)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapQt, qt, m, kRankPad, 32, 16)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapPt, pt, n, kRankPad, 32, 16)) != CUDA_SUCCESS) return (int)r;
  return 0;
}

}  // namespace grace
