// Fused PowerSGD exchange on sm_100a: low-rank projections on the 5th-gen
// tensor cores (tcgen05.mma, TF32 operands, fp32 accumulators in TMEM), tiles
// staged by TMA, both all-reduces done inside the kernel by loading the peers'
// partial results over NVLink.
//
// For every matrix M (n x m, row-major slice of the flat gradient buffer) of a
// launch, with rank r <= 16 padded to 16 columns:
//   S1  P = M' * Q with M' = G + R (error feedback): the gradient tile and the
//       residual tile [128 x 32, K-major] are both A operands of MMAs into the
//       same accumulator (P = G Q + R Q; B = Q^T tile [16 x 32] K-major, D in
//       TMEM: 128 lanes x 16 columns, two accumulators used alternately), while
//       other warps add the two tiles from shared memory and write M' to the
//       residual buffer for the later stages;
//   R1  publish; wait for every peer; P = mean over ranks of the W slots
//       (identical order on every rank, so the results are bit-identical);
//   O   orthogonalise P: Gram matrix P^T P and its Cholesky factor in fp64,
//       P R^-1 (what modified Gram-Schmidt computes in exact arithmetic),
//       written transposed for the next stage;
//   S2  Q = M'^T * P: TMA brings 32 rows x 128 columns of M' as four boxes of
//       32 x 32 in the "128-byte rows, 32-byte swizzle atoms" layout, which IS
//       the MN-major TF32 operand layout of the tensor core: the tile feeds
//       the MMA as it lands (A = M'^T [128 x 32] MN-major, B = P^T tile
//       [16 x 32] K-major); nothing is transposed by hand;
//   R2  publish; wait; Q = mean over ranks; kept as next step's warm start;
//   S3  out = P Q^T (rank-r outer products on CUDA cores), R = M' - out.
//
// The GEMM stages are warp specialised, with mbarriers between the roles and
// no CTA-wide barrier inside the loops:
//   warp 0     one thread issues the TMA loads of the operand ring;
//   warp 1     one thread issues the MMAs and commits them to the ring's
//              "empty" barriers and, at the end of a work item, to the
//              accumulator's "full" barrier;
//   warps 2, 3, 8  (S1 with error feedback) read the gradient and the residual
//              tile from shared memory, add them and store M' to global
//              memory (16 bytes per thread and access);
//   warps 4-7  epilogue: TMEM -> registers -> this item's partial result.
// A ring slot is free again when its MMAs have retired and the adder warps
// have read it.
// Split-K is deterministic: every work item (128 output rows x a K range)
// writes its partial sums to its own block of a scratch buffer; after the
// stage (and a grid barrier) the partials of a row block are added in split
// order into the slot.  The epilogue itself is a TMEM read and one store per
// row, so that many short items do not hold up the MMA thread.
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

constexpr int kThreads = 288;
constexpr int kTileRows = 128;          // MMA M
constexpr int kTileK = 32;              // fp32 elements per 128-byte row
constexpr int kRankPad = 16;            // MMA N
constexpr int kATileBytes = kTileRows * kTileK * 4;   // 16 KiB
constexpr int kBTileBytes = kRankPad * kTileK * 4;    // 2 KiB
// A DRAM page should be visited for more than one 128-byte tile row: a ring step of stage 1 therefore carries
// kS1Tiles K tiles side by side (256 contiguous bytes of every matrix row); a step of stage 2 has its four boxes of
// 32 columns side by side already (512 bytes).
constexpr int kS1Tiles = 2;
constexpr int kStagesR = 3;             // stage 1 with a residual tile: 3 steps of 2 x (16 + 16 + 2) KiB
constexpr int kStagesS1 = 5;            // stage 1 without: 5 steps of 2 x (16 + 2) KiB
constexpr int kStagesNoR = 11;          // stage 2: 11 steps of 16 + 2 KiB
constexpr int kRingBytes = kStagesR * kS1Tiles * (2 * kATileBytes + kBTileBytes);   // 204 KiB
static_assert(kStagesNoR * (kATileBytes + kBTileBytes) <= kRingBytes, "ring too small");
static_assert(kStagesS1 * kS1Tiles * (kATileBytes + kBTileBytes) <= kRingBytes, "ring too small");
constexpr unsigned kTmemCols = 32;      // two accumulators of 16 columns
constexpr int kMaxRank = 16;
constexpr int kS3Trip = 12;             // rows of one trip of stage 3 (the next trip's loads are already in flight)
constexpr int kS3Rows = 64;             // rows per stage-3 work item
constexpr int kS3Cols = kThreads * 4;   // columns per stage-3 work item
// warp roles of the GEMM stages
constexpr int kProducerWarp = 0, kMmaWarp = 1, kEpilogueWarp0 = 4;
constexpr int kAdderWarps = 3;          // warps 2, 3 and 8

// instruction descriptor: D=f32, A=B=tf32, N=16, M=128 (bit layout: c_format
// [4,6), a_format [7,10), b_format [10,13), a_major 15, b_major 16, N>>3
// [17,23), M>>4 [24,29)); bit 15 set = A is MN-major (stage 2)
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kRankPad >> 3) << 17) | ((kTileRows >> 4) << 24);
constexpr uint32_t kIdescAmn = kIdesc | (1u << 15);

struct __align__(1024) SmemLayout {
  unsigned char ring[kRingBytes];
  unsigned long long full[kStagesNoR];     // TMA landed
  unsigned long long empty[kStagesNoR];    // MMAs retired (and, in S1 with error feedback, the adder warps have read the tiles)
  unsigned long long acc_full[2];          // an item's MMAs retired
  unsigned long long acc_empty[2];         // the epilogue has read the accumulator
  unsigned tmem_base;
  int bars_valid;                          // the mbarriers above hold valid objects (a GEMM stage ran)
  int epi_ok;                              // epilogue: the accumulator arrived in time
  double gram[kMaxRank][kMaxRank];
  double rinv[kMaxRank][kMaxRank];
  float prow[kS3Rows][kMaxRank];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(void* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait; returns false (and records the failure) when the limit expires or another role already failed.
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
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Shared-memory matrix descriptor: start>>4 [0,14) | LBO>>4 [16,30) | SBO>>4 [32,46) | version 1 [46,48) |
// layout type [61,64): 2 = 128-byte swizzle of 16-byte chunks (K-major tiles), 1 = 128-byte rows swizzled in
// 32-byte atoms (the one layout the tensor core accepts for an MN-major TF32 operand).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
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
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Work item of a GEMM stage: (matrix, block of 128 output rows, K split).  Which K tiles a split takes, and how the
// items are numbered, is chosen so that CTAs running side by side read NEIGHBOURING pieces of the same matrix rows at
// about the same time (a tile row is only 128 bytes in stage 1 and 512 bytes in stage 2: taken alone they would
// open a DRAM page for very little):
//   stage 1  items of a row block are consecutive (split fastest) and split s takes the K tiles s, s + S, s + 2S, ...
//            so the S CTAs of a block walk the rows together, 128 bytes apart;
//   stage 2  blocks are fastest (item = split * blocks + block) and a split takes a contiguous K range, so
//            consecutive CTAs read adjacent 512-byte pieces of the same rows.
struct Item {
  int mat, blk;
  int kt0, kt_step, kt_count;   // K tiles kt0, kt0 + kt_step, ... (kt_count of them)
  int first, stride;            // split s of this row block is item first + s * stride
  int splits;
};
__device__ __forceinline__ bool decode_item(const LowRankArgs& a, int stage, int idx, Item& it) {
  const int total = stage == 1 ? a.items_s1 : a.items_s2;
  if (idx >= total) return false;
  int mat = 0;
  while (mat + 1 < a.nmat && (stage == 1 ? a.mats[mat + 1].item1_begin : a.mats[mat + 1].item2_begin) <= idx) ++mat;
  const LowRankMatrix& M = a.mats[mat];
  const int begin = stage == 1 ? M.item1_begin : M.item2_begin;
  const int local = idx - begin;
  const int ktiles = stage == 1 ? (M.m + kS1Tiles * kTileK - 1) / (kS1Tiles * kTileK) : (M.n + kTileK - 1) / kTileK;   // ring steps
  const int splits = stage == 1 ? M.splits1 : M.splits2;
  it.mat = mat;
  it.splits = splits;
  if (stage == 1) {
    const int sp = local % splits;
    it.blk = local / splits;
    it.first = begin + it.blk * splits;
    it.stride = 1;
    it.kt0 = sp;
    it.kt_step = splits;
    it.kt_count = (ktiles - sp + splits - 1) / splits;
  } else {
    const int blocks = (M.m + kTileRows - 1) / kTileRows;
    const int sp = local / blocks;
    it.blk = local % blocks;
    it.first = begin + it.blk;
    it.stride = blocks;
    it.kt0 = (int)((long long)sp * ktiles / splits);
    it.kt_step = 1;
    it.kt_count = (int)((long long)(sp + 1) * ktiles / splits) - it.kt0;
  }
  return true;
}

// One GEMM stage over this CTA's items.  STAGE 1: P = M' Q.  STAGE 2: Q = M'^T P.
// Every role walks the same sequence of (item, K tile) steps, which it derives from blockIdx by itself.
template <int STAGE>
__device__ void gemm_stage(const LowRankArgs& a, SmemLayout& sm, const Status& status) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool has_r = STAGE == 1 && a.has_memory;
  constexpr int T = STAGE == 1 ? kS1Tiles : 1;                    // K tiles per ring step
  const unsigned nstages = STAGE == 2 ? kStagesNoR : (has_r ? kStagesR : kStagesS1);
  // a step holds T gradient tiles, then (S1 with error feedback) T residual tiles, then T B tiles
  const unsigned off_r = T * kATileBytes, off_b = (has_r ? 2 : 1) * T * kATileBytes;
  const unsigned stage_bytes = off_b + T * kBTileBytes;
  const uint64_t tmo = a.peers.timeout_ns;
  if (tid == 0) {
    if (sm.bars_valid) {   // objects of the previous stage: all their phases are over (a CTA barrier lies behind us)
      for (int s = 0; s < kStagesNoR; ++s) { mbar_inval(&sm.full[s]); mbar_inval(&sm.empty[s]); }
      for (int b = 0; b < 2; ++b) { mbar_inval(&sm.acc_full[b]); mbar_inval(&sm.acc_empty[b]); }
    }
    for (int s = 0; s < kStagesNoR; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], has_r ? 1 + kAdderWarps : 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], 4); }
    sm.bars_valid = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kProducerWarp) {
    if (lane == 0) {
      unsigned step = 0;
      Item it;
      bool ok = true;
      for (int idx = blockIdx.x; ok && decode_item(a, STAGE, idx, it); idx += gridDim.x) {
        const CUtensorMap* maps = reinterpret_cast<const CUtensorMap*>(a.maps) + (size_t)it.mat * kMapsPerMatrix;
        for (int kj = 0, kt = it.kt0; kj < it.kt_count; ++kj, kt += it.kt_step, ++step) {
          const unsigned slot = step % nstages;
          if (step >= nstages) ok = mbar_wait(&sm.empty[slot], ((step / nstages) - 1) & 1, tmo, status, 100 + slot);
          if (!ok) break;
          unsigned char* base = sm.ring + (size_t)slot * stage_bytes;
          mbar_expect_tx(&sm.full[slot], stage_bytes);
          if (STAGE == 1) {
#pragma unroll
            for (int t = 0; t < T; ++t) {   // a tile past the last column is filled with zeros by the TMA unit
              const int x = (kt * T + t) * kTileK;
              tma_load_2d(base + t * kATileBytes, maps + kMapG1, x, it.blk * kTileRows, &sm.full[slot]);
              if (has_r) tma_load_2d(base + off_r + t * kATileBytes, maps + kMapA1, x, it.blk * kTileRows, &sm.full[slot]);
              tma_load_2d(base + off_b + t * kBTileBytes, maps + kMapQt, x, 0, &sm.full[slot]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)  // four boxes of 32 columns x 32 rows of M': the MN-major operand layout
              tma_load_2d(base + j * 4096, maps + kMapM2, it.blk * kTileRows + j * 32, kt * kTileK, &sm.full[slot]);
            tma_load_2d(base + off_b, maps + kMapPt, kt * kTileK, 0, &sm.full[slot]);
          }
        }
      }
      if (!ok || status.failed()) {
        // a consumer gave up: every load already issued must still land before the shared memory is let go
        for (unsigned s = step > nstages ? step - nstages : 0; s < step; ++s)
          mbar_wait(&sm.full[s % nstages], (s / nstages) & 1, tmo, status, 400);
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      unsigned step = 0, item = 0;
      Item it;
      bool ok = true;
      for (int idx = blockIdx.x; ok && decode_item(a, STAGE, idx, it); idx += gridDim.x, ++item) {
        const unsigned buf = item & 1, use = item >> 1;
        if (use >= 1) ok = mbar_wait(&sm.acc_empty[buf], (use - 1) & 1, tmo, status, 300 + buf);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = sm.tmem_base + buf * kRankPad;
        for (int kj = 0, kt = it.kt0; kj < it.kt_count; ++kj, kt += it.kt_step, ++step) {
          const unsigned slot = step % nstages;
          ok = mbar_wait(&sm.full[slot], (step / nstages) & 1, tmo, status, 200 + slot);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sm.ring + (size_t)slot * stage_bytes), b_addr = a_addr + off_b;
#pragma unroll
          for (int t = 0; t < T; ++t) {
#pragma unroll
            for (int kk = 0; kk < kTileK / 8; ++kk) {
              const uint64_t bdesc = smem_desc(b_addr + t * kBTileBytes + kk * 32, 16, 1024, 2);   // K-major: 32 B per K step of 8
              const uint64_t adesc = STAGE == 1
                                         ? smem_desc(a_addr + t * kATileBytes + kk * 32, 16, 1024, 2)
                                         // MN-major: a K step is 8 rows of 128 B (two atoms of 4 rows, 512 B apart);
                                         // the next 32 of the 128 M-columns sit one box (4096 B) further on
                                         : smem_desc(a_addr + kk * 1024, 4096, 512, 1);
              umma_tf32(tmem_d, adesc, bdesc, STAGE == 1 ? kIdesc : kIdescAmn, !(kj == 0 && t == 0 && kk == 0));
            }
            if (has_r) {   // the residual tile into the same accumulator: P = G Q + R Q
#pragma unroll
              for (int kk = 0; kk < kTileK / 8; ++kk)
                umma_tf32(tmem_d, smem_desc(a_addr + off_r + t * kATileBytes + kk * 32, 16, 1024, 2),
                          smem_desc(b_addr + t * kBTileBytes + kk * 32, 16, 1024, 2), kIdesc, true);
            }
          }
          umma_commit(&sm.empty[slot]);
        }
        if (!ok) break;
        umma_commit(&sm.acc_full[buf]);
      }
    }
  } else if (warp == 2 || warp == 3 || warp == 8) {
    if (has_r) {
      // M' = G + R for the later stages: both tiles are read from shared memory (they hold the same 128-byte
      // swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8)), added, and stored straight to global memory
      const int at = (warp == 8 ? 64 : (warp - 2) * 32) + lane;   // 0 .. 95
      constexpr int kAdders = kAdderWarps * 32;
      unsigned step = 0;
      Item it;
      bool ok = true;
      for (int idx = blockIdx.x; ok && decode_item(a, STAGE, idx, it); idx += gridDim.x) {
        const LowRankMatrix& M = a.mats[it.mat];
        float* const dst = a.acc + M.g_off;
        for (int kj = 0, kt = it.kt0; kj < it.kt_count; ++kj, kt += it.kt_step, ++step) {
          const unsigned slot = step % nstages;
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.full[slot], (step / nstages) & 1, tmo, status, 500 + slot));
          if (!ok) break;
          const unsigned char* base = sm.ring + (size_t)slot * stage_bytes;
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const float4* pa = reinterpret_cast<const float4*>(base + t * kATileBytes);
            const float4* pr = reinterpret_cast<const float4*>(base + off_r + t * kATileBytes);
#pragma unroll 4
            for (int i = at; i < kATileBytes / 16; i += kAdders) {
              float4 x = pa[i];
              const float4 y = pr[i];
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
              const int row = i >> 3, grow = it.blk * kTileRows + row;
              const int gcol = (kt * T + t) * kTileK + (((i & 7) ^ (row & 7)) << 2);
              if (grow < M.n && gcol < M.m)   // m is a multiple of 4: the four columns are inside together
                *reinterpret_cast<float4*>(dst + (size_t)grow * M.m + gcol) = x;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.empty[slot]);
        }
      }
    }
  } else {
    // ---- epilogue warps: TMEM -> registers -> this item's block of partial sums ----
    const int ew = warp - kEpilogueWarp0;                     // TMEM lane quarter of this warp (warp % 4)
    const int erow = ew * 32 + lane;                          // row of the 128-row block held by this thread
    const int rpad4 = (a.rank + 3) / 4;                       // float4 per row that carry data
    const size_t item_base = STAGE == 1 ? 0 : (size_t)a.items_s1;
    unsigned item = 0;
    Item it;
    for (int idx = blockIdx.x; decode_item(a, STAGE, idx, it); idx += gridDim.x, ++item) {
      const unsigned buf = item & 1, use = item >> 1;
      if (erow == 0) sm.epi_ok = mbar_wait(&sm.acc_full[buf], use & 1, tmo, status, 700 + buf) ? 1 : 0;
      named_bar_sync(1, 128);
      if (!sm.epi_ok) break;                                  // one decision for all four warps
      tc_fence_after();
      uint32_t v[16];
      const uint32_t taddr = sm.tmem_base + buf * kRankPad + ((uint32_t)(ew * 32) << 16);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);         // the MMA thread may start the item after next
      float4* part = reinterpret_cast<float4*>(a.partial + (item_base + idx) * (size_t)(kTileRows * kRankPad)) + erow * 4;
      for (int c4 = 0; c4 < rpad4; ++c4)
        part[c4] = make_float4(__uint_as_float(v[4 * c4]), __uint_as_float(v[4 * c4 + 1]), __uint_as_float(v[4 * c4 + 2]),
                               __uint_as_float(v[4 * c4 + 3]));
      named_bar_sync(1, 128);   // epi_ok is rewritten by the next item
    }
  }
  __syncthreads();
}

// Upper Cholesky factor R of sm.gram (R^T R = Gram) and its inverse into sm.rinv, by one thread.  RMAX bounds the
// loops at compile time so that, for small ranks, R lives in registers.  A non-positive pivot (a rank-deficient P)
// zeroes its row and column: the corresponding direction is dropped, as a projection onto nothing.
template <int RMAX>
__device__ void cholesky_inverse(SmemLayout& sm, int r) {
  double R[RMAX][RMAX];
#pragma unroll
  for (int j = 0; j < RMAX; ++j) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      R[i][j] = 0.0;
      if (i <= j && j < r) {
        double s = sm.gram[i][j];
#pragma unroll
        for (int k = 0; k < RMAX; ++k) if (k < i) s -= R[k][i] * R[k][j];
        if (i == j) R[i][j] = s > 0.0 ? sqrt(s) : 0.0;
        else R[i][j] = R[i][i] > 0.0 ? s / R[i][i] : 0.0;
      }
    }
  }
  // invert the upper-triangular R by back substitution
  double inv[RMAX][RMAX];
#pragma unroll
  for (int j = 0; j < RMAX; ++j) {
#pragma unroll
    for (int i = 0; i < RMAX; ++i) inv[i][j] = 0.0;
    if (j < r && R[j][j] > 0.0) inv[j][j] = 1.0 / R[j][j];
#pragma unroll
    for (int i = RMAX - 1; i >= 0; --i) {
      if (i < j && j < r) {
        double s = 0.0;
#pragma unroll
        for (int k = 0; k < RMAX; ++k) if (k > i && k <= j) s += R[i][k] * inv[k][j];
        inv[i][j] = R[i][i] > 0.0 ? -s / R[i][i] : 0.0;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RMAX; ++i)
#pragma unroll
    for (int j = 0; j < RMAX; ++j) sm.rinv[i][j] = inv[i][j];
}

// Same for ranks above 4, with the factor in shared memory (the operand ring is idle at that point).
__device__ void cholesky_inverse_large(SmemLayout& sm, int r) {
  double (*R)[kMaxRank] = reinterpret_cast<double (*)[kMaxRank]>(sm.ring);
  for (int j = 0; j < r; ++j) {
    for (int i = 0; i <= j; ++i) {
      double s = sm.gram[i][j];
      for (int k = 0; k < i; ++k) s -= R[k][i] * R[k][j];
      if (i == j) R[i][j] = s > 0.0 ? sqrt(s) : 0.0;
      else R[i][j] = R[i][i] > 0.0 ? s / R[i][i] : 0.0;
    }
  }
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

// Split-K reduction after a GEMM stage: row by row, the partial sums of the K splits are added in split order (the
// same order on every run and every rank) and stored to this rank's slot.  One thread per output row.
template <int STAGE>
__device__ void reduce_partials(const LowRankArgs& a, float* __restrict__ dst_slot) {
  const int rpad4 = (a.rank + 3) / 4;
  const size_t item_base = STAGE == 1 ? 0 : (size_t)a.items_s1;
  for (int mat = 0; mat < a.nmat; ++mat) {
    const LowRankMatrix& M = a.mats[mat];
    const int rows = STAGE == 1 ? M.n : M.m;
    const int splits = STAGE == 1 ? M.splits1 : M.splits2;
    const int blocks = (rows + kTileRows - 1) / kTileRows;
    const int begin = STAGE == 1 ? M.item1_begin : M.item2_begin;
    for (int row = blockIdx.x * kThreads + threadIdx.x; row < rows; row += gridDim.x * kThreads) {
      const int blk = row / kTileRows, erow = row % kTileRows;
      // numbering of decode_item: stage 1 split fastest, stage 2 block fastest
      const size_t first = item_base + begin + (STAGE == 1 ? (size_t)blk * splits : (size_t)blk);
      const size_t stride = STAGE == 1 ? 1 : (size_t)blocks;
      float4 sum[4];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) sum[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp = 0; sp < splits; ++sp) {
        const float4* src = reinterpret_cast<const float4*>(a.partial + (first + sp * stride) * (size_t)(kTileRows * kRankPad)) + erow * 4;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          if (c4 < rpad4) {
            const float4 t = __ldcg(src + c4);
            sum[c4].x += t.x; sum[c4].y += t.y; sum[c4].z += t.z; sum[c4].w += t.w;
          }
        }
      }
      float4* dst = reinterpret_cast<float4*>(dst_slot + (STAGE == 1 ? M.p_off : M.q_off) + (size_t)row * kRankPad);
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) dst[c4] = sum[c4];   // the padded columns are written too (zeros)
    }
  }
}

// Mean over ranks of a [rows x 16] region.
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

// S3 for one matrix: out = P Q^T, residual = M' - out.  Item = kS3Rows rows x kS3Cols columns; a thread owns four
// columns and walks the rows in trips of kS3Trip with the loads of the next trip already in flight.
template <int R4>   // R4 = ceil(rank / 4): how many groups of four rank columns take part
__device__ void stage3_matrix(const LowRankArgs& a, SmemLayout& sm, const LowRankMatrix& M) {
  const int tid = threadIdx.x;
  const float* __restrict__ src = a.has_memory ? a.acc : a.g;
  const int row_blocks = (M.n + kS3Rows - 1) / kS3Rows, col_blocks = (M.m + kS3Cols - 1) / kS3Cols;
  for (int item = blockIdx.x; item < row_blocks * col_blocks; item += gridDim.x) {
    const int rb = item / col_blocks, cb = item % col_blocks;
    __syncthreads();
    for (int i = tid; i < kS3Rows * kMaxRank; i += kThreads) {
      const int rr = i / kMaxRank, c = i % kMaxRank, row = rb * kS3Rows + rr;
      sm.prow[rr][c] = (row < M.n && c < a.rank) ? a.pt_orth[M.pt_off + (size_t)c * M.n + row] : 0.f;
    }
    __syncthreads();
    const int col = cb * kS3Cols + tid * 4;
    if (col >= M.m) continue;
    const int valid = min(4, M.m - col);
    float q[4][4 * R4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
#pragma unroll
      for (int h = 0; h < R4; ++h) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < valid && 4 * h < a.rank)   // columns >= rank of q_mean are zero
          t = reinterpret_cast<const float4*>(a.q_mean + M.q_off + (size_t)(col + e) * kRankPad)[h];
        q[e][4 * h] = t.x; q[e][4 * h + 1] = t.y; q[e][4 * h + 2] = t.z; q[e][4 * h + 3] = t.w;
      }
    }
    const int rows = min(kS3Rows, M.n - rb * kS3Rows);
    const bool vec = valid == 4 && (M.m & 3) == 0;
    const size_t base0 = (size_t)M.g_off + (size_t)(rb * kS3Rows) * M.m + col;
    auto fetch = [&](float4 (&mv)[kS3Trip], int r0) {
#pragma unroll
      for (int u = 0; u < kS3Trip; ++u) {
        mv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + u < rows && a.has_memory && vec)
          mv[u] = *reinterpret_cast<const float4*>(src + base0 + (size_t)(r0 + u) * M.m);
      }
    };
    float4 cur[kS3Trip], nxt[kS3Trip];
    fetch(cur, 0);
    for (int r0 = 0; r0 < rows; r0 += kS3Trip) {
      fetch(nxt, r0 + kS3Trip);   // rows past the item read nothing
#pragma unroll
      for (int u = 0; u < kS3Trip; ++u) {
        const int rr = r0 + u;
        if (rr >= rows) break;
        const size_t base = base0 + (size_t)rr * M.m;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4 * R4; ++c) {
          const float p = sm.prow[rr][c];
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] += p * q[e][c];
        }
        if (vec) {
          if (a.has_memory)
            *reinterpret_cast<float4*>(a.acc + base) =
                make_float4(cur[u].x - o[0], cur[u].y - o[1], cur[u].z - o[2], cur[u].w - o[3]);
          *reinterpret_cast<float4*>(a.out + base) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
          for (int e = 0; e < valid; ++e) {
            const float m1 = src[base + e];
            if (a.has_memory) a.acc[base + e] = m1 - o[e];
            a.out[base + e] = o[e];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kS3Trip; ++u) cur[u] = nxt[u];
    }
  }
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

  // ---- set-up: TMEM (the mbarriers are initialised by each GEMM stage) ----
  if (tid == 0) sm.bars_valid = 0;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // A single launch runs everything; the split launches of the one-GPU emulation run
  //   [S1 | publish P] [reduce P, O, S2 | publish Q] [reduce Q, S3]
  // as three launches selected by a.part (0 = all, 1..3 = that part only).
  const int part = a.part;
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
    ok = !status.failed();   // (the slot is written only by reduce_partials below, whole rows at a time)
    if (ok) gemm_stage<1>(a, sm, status);
    fence_async_all();
    ok = bar.sync();
    if (ok) reduce_partials<1>(a, slot_p);
    ok = bar.sync() && ok;
  }

  if (part1 || part2) {
    // publish P (part 1) / wait for the peers' P (part 2)
    ok = publish_and_wait(a, status, a.peers.ready_off, part1, part2) && ok && !status.failed();
  }

  if (part2) {
    if (ok) {
      // P = mean over ranks, one thread per row: the Gram pass below reads only the rows its own thread wrote
      // (same row -> thread mapping), so no grid barrier separates the two
      const float inv = 1.f / (float)a.divisor;
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        for (int row = blockIdx.x * kThreads + tid; row < M.n; row += gridDim.x * kThreads) {
          const size_t off = ((size_t)M.p_off + (size_t)row * kRankPad) * 4;
          float4 sum[4];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) sum[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p = 0; p < world; ++p) {
            const char* src = a.peers.heap[p] + a.peers.slot_off + off;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const uint4 v = ld_cg_u4(src + 16 * c4);
              sum[c4].x += __uint_as_float(v.x); sum[c4].y += __uint_as_float(v.y);
              sum[c4].z += __uint_as_float(v.z); sum[c4].w += __uint_as_float(v.w);
            }
          }
          float4* dst = reinterpret_cast<float4*>(a.p_mean + M.p_off + (size_t)row * kRankPad);
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4)
            dst[c4] = make_float4(sum[c4].x * inv, sum[c4].y * inv, sum[c4].z * inv, sum[c4].w * inv);
        }
      }
    }
    if (ok) {
      // Gram matrices P^T P in fp64, added in a fixed order at every level (lanes by shuffles, warps in warp order,
      // CTAs in CTA order) so that two runs give the same bits: a thread takes one row, a warp adds its rows'
      // products with shuffles, the CTA adds its warps and stores one partial matrix per CTA.
      double* const wpart = reinterpret_cast<double*>(sm.ring);           // [warp][256], the ring is idle here
      const int lane = tid & 31;
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        float v[kMaxRank];
#pragma unroll
        for (int c = 0; c < kMaxRank; ++c) v[c] = 0.f;
        double acc_cd[kMaxRank] = {};   // row c of the upper triangle, one c at a time (keeps the register count low)
        const int row0 = blockIdx.x * kThreads + tid;
        for (int c = 0; c < a.rank; ++c) {
#pragma unroll
          for (int d = 0; d < kMaxRank; ++d) acc_cd[d] = 0.0;
          for (int row = row0; row < M.n; row += gridDim.x * kThreads) {
            const float* pr = a.p_mean + M.p_off + (size_t)row * kRankPad;
#pragma unroll
            for (int d = 0; d < kMaxRank; ++d) v[d] = d < a.rank ? pr[d] : 0.f;
            const double vc = (double)pr[c];
#pragma unroll
            for (int d = 0; d < kMaxRank; ++d) acc_cd[d] += vc * (double)v[d];
          }
#pragma unroll
          for (int d = 0; d < kMaxRank; ++d) {
            if (d < c || d >= a.rank) continue;   // uniform over the CTA
            const double t = warp_sum(acc_cd[d]);
            if (lane == 0) wpart[warp * 256 + c * kRankPad + d] = t;
          }
        }
        __syncthreads();
        if (tid < kRankPad * kRankPad) {
          const int c = tid / kRankPad, d = tid % kRankPad;
          double t = 0.0;
          if (c <= d && d < a.rank)
            for (int w = 0; w < kThreads / 32; ++w) t += wpart[w * 256 + tid];
          a.gram_part[((size_t)blockIdx.x * a.nmat + mat) * 256 + tid] = t;
        }
        __syncthreads();
      }
    }
    ok = bar.sync() && ok;
    if (ok) {
      // O: P_orth = P R^-1 with R^T R = Gram (upper Cholesky), written transposed [16][n]
      for (int mat = 0; mat < a.nmat; ++mat) {
        const LowRankMatrix& M = a.mats[mat];
        {
          // the CTAs' partial matrices: one warp per entry of the upper triangle; a lane adds the partials of CTAs
          // lane, lane + 32, ... (in that order), the lanes are combined by the shuffle tree: a fixed order
          const int lane = tid & 31;
          const int entries = a.rank * (a.rank + 1) / 2;
          for (int e = warp; e < entries; e += kThreads / 32) {
            int c = 0, rem = e;
            while (rem >= a.rank - c) { rem -= a.rank - c; ++c; }
            const int d = c + rem;
            double t = 0.0;
            for (unsigned b = lane; b < gridDim.x; b += 32)
              t += __ldcg(a.gram_part + ((size_t)b * a.nmat + mat) * 256 + c * kRankPad + d);
            t = warp_sum(t);
            if (lane == 0) sm.gram[c][d] = t;
          }
        }
        __syncthreads();
        if (tid == 0) {
          if (a.rank <= 4) cholesky_inverse<4>(sm, a.rank);
          else cholesky_inverse_large(sm, a.rank);
        }
        __syncthreads();
        for (int row = blockIdx.x * kThreads + tid; row < M.n; row += gridDim.x * kThreads) {
          const float* pr = a.p_mean + M.p_off + (size_t)row * kRankPad;
          float v[kMaxRank];
#pragma unroll
          for (int c = 0; c < kMaxRank; ++c) v[c] = c < a.rank ? pr[c] : 0.f;
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
    if (ok) gemm_stage<2>(a, sm, status);
    ok = bar.sync() && ok;
    if (ok) reduce_partials<2>(a, slot_q);
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
      for (int mat = 0; mat < a.nmat; ++mat) {
        if (a.rank <= 4) stage3_matrix<1>(a, sm, a.mats[mat]);
        else if (a.rank <= 8) stage3_matrix<2>(a, sm, a.mats[mat]);
        else if (a.rank <= 12) stage3_matrix<3>(a, sm, a.mats[mat]);
        else stage3_matrix<4>(a, sm, a.mats[mat]);
      }
    }
  }

  // ---- teardown ----
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
//   M2 : M' (accumulator, or gradient without memory), box 32 x 32, 128-byte rows swizzled in 32-byte atoms: the
//        MN-major TF32 operand layout of stage 2
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
                uint32_t box_outer, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) -> CUresult {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 4};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return cuTensorMapEncodeTiled_rt(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r;
  if ((r = enc(maps + kMapG1, g, m, n, 32, 128)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapA1, acc ? acc : g, m, n, 32, 128)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapM2, acc ? acc : g, m, n, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapQt, qt, m, kRankPad, 32, 16)) != CUDA_SUCCESS) return (int)r;
  if ((r = enc(maps + kMapPt, pt, n, kRankPad, 32, 16)) != CUDA_SUCCESS) return (int)r;
  return 0;
}

}  // namespace grace
