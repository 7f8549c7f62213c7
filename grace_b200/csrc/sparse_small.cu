// Sparse exchange of ONE small tensor (up to 8192 elements) by a single CTA.
//
// The persistent kernel of sparse_exchange.cu is built for buckets of millions
// of elements: a cooperative launch, two memsets, 4096-bin histograms in
// global memory and several grid barriers, about 0.1 ms whatever the size.  A
// training loop that calls step(tensor, name) per parameter meets mostly tiny
// tensors (batch-norm scales and biases: a few hundred elements, k = 1 or 2),
// so this variant keeps everything of such a tensor on one SM:
//   * a thread holds 16 consecutive elements in registers (compensated value,
//     DGC momentum), nothing is re-read from global memory;
//   * the k-th largest magnitude comes from four radix passes (8 + 8 + 8 + 7
//     key bits) over 256-bin shared-memory histograms (one per warp, summed
//     and suffix-scanned by 256 threads); among equal keys the
//     lowest indices win, so exactly k entries travel and the list is in
//     index order whatever the timing;
//   * compaction by a block-wide prefix sum straight into the send slot, the
//     residual (and DGC u, v) zeroed at the picks in the same registers;
//   * publish / bounded waits / acknowledge exactly as the large kernel (same
//     flags, same slot header), then every rank's list is added, in rank
//     order, into a shared-memory copy of the output that is written once.
// One plain launch, no scratch memory, no memset.  Same arguments and phases
// as the large kernel; launch_sparse_exchange() picks the variant from the
// layout alone (one tensor, padded length <= 8192, not random-k, no clipping),
// so all ranks decide alike.
//
// Replaces, for such tensors, the same reference code as sparse_exchange.cu:
// compressor/topk.py:32-49, threshold.py:16-27, memory/residual.py:10-20,
// memory/dgc.py:21-39 and communicator/allgather.py:8-45.
#include "common.cuh"
#include "exchange.h"
#include "gradio.cuh"

namespace grace {

namespace {

constexpr int kSmallBlock = 512;
constexpr int kSmallPer = 16;                          // elements per thread
constexpr int kSmallMax = kSmallBlock * kSmallPer;     // 8192
constexpr unsigned kSmallHeaderBytes = 128;            // slot header of sparse_exchange.cu: [0] entries, [1] overflow

struct SmallSmem {
  float out[kSmallMax];        // the dense output while the ranks' lists are added; per-warp histograms before
  unsigned warp_tot[kSmallBlock / 32];
  float warp_max[kSmallBlock / 32];
  unsigned prefix, need, total;
  float bound;
  int ok;
};

// Exclusive prefix sum of v over the CTA in thread order; total in sm.total.
__device__ __forceinline__ unsigned block_excl_scan(SmallSmem& sm, unsigned v) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();   // warp_tot of an earlier scan has been read by everybody
  if (lane == 31) sm.warp_tot[warp] = incl;
  __syncthreads();
  unsigned before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kSmallBlock / 32; ++w) {
    const unsigned t = sm.warp_tot[w];
    if (w < warp) before += t;
    total += t;
  }
  if (tid == 0) sm.total = total;
  return before + incl - v;
}

__global__ void __launch_bounds__(kSmallBlock, 1) sparse_small_kernel(const SparseArgs a) {
  __shared__ SmallSmem sm;
  const Status status{a.status};
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = a.peers.rank, world = a.peers.world;
  char* const my_heap = a.peers.heap[rank];
  unsigned* const my_hdr = reinterpret_cast<unsigned*>(my_heap + a.peers.slot_off);
  float* const my_vals = reinterpret_cast<float*>(my_heap + a.peers.slot_off + kSmallHeaderBytes);
  int* const my_idx = reinterpret_cast<int*>(my_vals + a.cap);
  const Segment seg = a.segs[0];
  const long long off = seg.offset;
  const int n = seg.numel < kSmallMax ? seg.numel : kSmallMax;
  const int first = tid * kSmallPer;          // this thread's elements: [first, first + 16) of the tensor

  if (a.phases & kPhaseCompress) {
    // the slot of this parity was last used by sequence seq - 2: every peer must have read it
    if (tid < world && tid != rank && a.peers.seq > 2) {
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ack_off) + tid;
      wait_flag_ge(ack, a.peers.seq - 2, a.peers.timeout_ns, status, kTimeoutPeerAck, tid);
    }
    __syncthreads();
    if (tid == 0) sm.ok = status.failed() ? 0 : 1;
    __syncthreads();
    if (sm.ok) {
      // ---- compensate: everything of the tensor lives in registers from here on ----
      float av[kSmallPer], uv[kSmallPer];
      const bool read_acc = a.u || (a.acc && a.beta != 0.f);
#pragma unroll
      for (int q = 0; q < kSmallPer / 4; ++q) {
        const int i = first + 4 * q;
        const int valid = i < n ? (n - i >= 4 ? 4 : n - i) : 0;
        float gv[4] = {0.f, 0.f, 0.f, 0.f}, rv[4] = {0.f, 0.f, 0.f, 0.f}, mv[4] = {0.f, 0.f, 0.f, 0.f};
        if (valid) {
          load4g(a.g, a.g_dtype, off + i, valid, gv);
          if (read_acc) load4(a.acc, off + i, valid, rv);
          if (a.u) load4(a.u, off + i, valid, mv);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (a.u) {
            uv[4 * q + j] = a.momentum * mv[j] + gv[j];
            av[4 * q + j] = rv[j] + uv[4 * q + j];
          } else {
            uv[4 * q + j] = 0.f;
            av[4 * q + j] = a.beta * rv[j] + a.gamma * gv[j];
          }
        }
      }
      const int mine = first < n ? (n - first >= kSmallPer ? kSmallPer : n - first) : 0;   // valid elements here

      // ---- which elements travel ----
      unsigned sel_mask = 0;
      if (a.mode == kSparseTopK) {
        unsigned prefix = 0, need = (unsigned)(seg.k < 1 ? 1 : (seg.k > n ? n : seg.k));
        // one 256-bin histogram per warp (in the area of the output copy, idle until the exchange): keys of one
        // tensor share a few exponents, and a single histogram would serialise the whole CTA on those bins
        unsigned* const whist = reinterpret_cast<unsigned*>(sm.out);
        static_assert(sizeof(float) * kSmallMax >= sizeof(unsigned) * 256 * (kSmallBlock / 32), "warp histograms do not fit");
#pragma unroll 1
        for (int pass = 0; pass < 4; ++pass) {
          const int bits = pass == 3 ? 7 : 8;
          const int shift = pass == 3 ? 0 : 23 - 8 * pass;        // position of this pass's digit in the 31-bit key
          for (int b = tid; b < 256 * (kSmallBlock / 32); b += kSmallBlock) whist[b] = 0;
          __syncthreads();
#pragma unroll
          for (int e = 0; e < kSmallPer; ++e) {
            if (e < mine) {
              const unsigned key = __float_as_uint(av[e]) & 0x7fffffffu;
              if (pass == 0 || (key >> (shift + bits)) == prefix)
                atomicAdd(&whist[warp * 256 + ((key >> shift) & ((1u << bits) - 1u))], 1u);
            }
          }
          __syncthreads();
          // the digit holding the need-th largest key: thread d < 256 owns bin d and learns how many keys lie in
          // the bins above it (suffix sums over the lanes, then over the eight warps of bins)
          unsigned c = 0, incl = 0;
          if (tid < 256) {
#pragma unroll
            for (int w = 0; w < kSmallBlock / 32; ++w) c += whist[w * 256 + tid];
            incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const unsigned t = __shfl_down_sync(0xffffffffu, incl, o);
              if (lane + o < 32) incl += t;
            }
            if (lane == 0) sm.warp_tot[warp] = incl;
          }
          __syncthreads();
          if (tid < 256) {
            unsigned above = incl - c;
            for (int w = warp + 1; w < 8; ++w) above += sm.warp_tot[w];
            if (c && above < need && need <= above + c) {          // true for exactly one bin
              sm.prefix = (prefix << bits) | (unsigned)tid;
              sm.need = need - above;
            }
          }
          __syncthreads();
          prefix = sm.prefix;
          need = sm.need;
        }
        // keys above the pivot all travel; of the keys equal to it, the `need` lowest indices
        unsigned eq = 0;
#pragma unroll
        for (int e = 0; e < kSmallPer; ++e)
          if (e < mine && (__float_as_uint(av[e]) & 0x7fffffffu) == prefix) ++eq;
        unsigned eq_before = block_excl_scan(sm, eq);
#pragma unroll
        for (int e = 0; e < kSmallPer; ++e) {
          if (e >= mine) continue;
          const unsigned key = __float_as_uint(av[e]) & 0x7fffffffu;
          if (key > prefix) sel_mask |= 1u << e;
          else if (key == prefix) {
            if (eq_before < need) sel_mask |= 1u << e;
            ++eq_before;
          }
        }
      } else {
        float thr = a.threshold;
        if (!a.strict) {   // the torch.distributed flavour caps the threshold by max(x)
          float m = -INFINITY;
#pragma unroll
          for (int e = 0; e < kSmallPer; ++e) if (e < mine) m = fmaxf(m, av[e]);
          m = warp_max(m);
          if (lane == 0) sm.warp_max[warp] = m;
          __syncthreads();
          if (tid == 0) {
            float t = -INFINITY;
            for (int w = 0; w < kSmallBlock / 32; ++w) t = fmaxf(t, sm.warp_max[w]);
            sm.bound = t;
          }
          __syncthreads();
          thr = fminf(thr, sm.bound);
        }
#pragma unroll
        for (int e = 0; e < kSmallPer; ++e)
          if (e < mine && (a.strict ? fabsf(av[e]) > thr : fabsf(av[e]) >= thr)) sel_mask |= 1u << e;
      }

      // ---- compaction into the send slot (index order), error-feedback update in the registers ----
      unsigned pos = block_excl_scan(sm, (unsigned)__popc(sel_mask));
      __syncthreads();
      const unsigned total = sm.total;
      unsigned dropped = 0;
#pragma unroll
      for (int e = 0; e < kSmallPer; ++e) {
        if (!((sel_mask >> e) & 1u)) continue;
        if (pos < a.cap && GRACE_IN_RANGE(status, kKernelSparse, kSmallHeaderBytes + (size_t)a.cap * 8, a.peers.slot_bytes + 1)) {
          my_vals[pos] = av[e];
          my_idx[pos] = (int)(off + first + e);
          av[e] = 0.f;
          uv[e] = 0.f;
        } else {
          ++dropped;   // no room (threshold mode): the value stays in the residual
        }
        ++pos;
      }
      if (dropped) atomicAdd(&a.status[3], dropped);
      if (tid == 0) {
        my_hdr[0] = total < a.cap ? total : a.cap;
        my_hdr[1] = total < a.cap ? 0u : total - a.cap;
      }
      // new residual (and DGC momentum)
#pragma unroll
      for (int q = 0; q < kSmallPer / 4; ++q) {
        const int i = first + 4 * q;
        const int valid = i < n ? (n - i >= 4 ? 4 : n - i) : 0;
        if (!valid) continue;
        const float r4[4] = {av[4 * q], av[4 * q + 1], av[4 * q + 2], av[4 * q + 3]};
        const float u4[4] = {uv[4 * q], uv[4 * q + 1], uv[4 * q + 2], uv[4 * q + 3]};
        if (a.acc) store4(a.acc, off + i, valid, r4);
        if (a.u) store4(a.u, off + i, valid, u4);
      }
    }
    __syncthreads();
  }

  if (a.phases & kPhasePublish) {
    if (tid < world && !status.failed()) {
      __threadfence_system();   // the CTA barrier above ordered every thread's slot writes before this fence
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ready_off) + rank, a.peers.seq);
    }
  }

  if ((a.phases & kPhaseExchange) && a.out) {
    if (tid == 0) sm.ok = 1;
    __syncthreads();
    if (tid < world) {
      const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + tid;
      if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) sm.ok = 0;
    }
    for (int i = tid; i < kSmallMax; i += kSmallBlock) sm.out[i] = 0.f;
    __syncthreads();
    // one decision for the whole CTA (the loop below has CTA barriers): a status word that another launch of the
    // channel changes at this moment must not split the threads
    if (tid == 0 && status.failed()) sm.ok = 0;
    __syncthreads();
    if (sm.ok) {
      for (int p = 0; p < world; ++p) {   // rank order: the same sums, bit for bit, on every GPU
        const char* slot = a.peers.heap[p] + a.peers.slot_off;
        unsigned count = ld_cg_u32(slot);
        if (count > a.cap) count = a.cap;
        const char* vals = slot + kSmallHeaderBytes;
        const char* idxs = vals + (size_t)a.cap * 4;
        for (unsigned e = tid; e < count; e += kSmallBlock) {
          const float v = ld_cg_f32(vals + (size_t)e * 4);
          const long long idx = (long long)(int)ld_cg_u32(idxs + (size_t)e * 4) - off;
          if (idx < 0 || idx >= n) {   // a corrupt index is reported, never followed
            status.fail(kBadArgument, (unsigned)p, (unsigned)a.peers.seq);
            continue;
          }
          sm.out[idx] += v * a.scale;   // the indices of one list are distinct: no two threads meet
        }
        __syncthreads();
      }
      // every slot of this sequence has been read: the peers may reuse theirs
      if (tid < world && tid != rank)
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank, a.peers.seq);
#pragma unroll
      for (int q = 0; q < kSmallPer / 4; ++q) {
        const int i = first + 4 * q;
        const int valid = i < n ? (n - i >= 4 ? 4 : n - i) : 0;
        if (!valid) continue;
        const float o4[4] = {sm.out[i], sm.out[i + 1], sm.out[i + 2], sm.out[i + 3]};
        store4(a.out, off + i, valid, o4);
      }
    }
  }
}

}  // namespace

bool sparse_small_applies(const SparseArgs& a) {
  return a.nseg == 1 && a.total <= kSmallMax && a.mode != kSparseRandomK && !a.clip_off &&
         !(a.phases & kPhaseClip) && !a.tile_start;
}

cudaError_t launch_sparse_small(const SparseArgs& a, cudaStream_t stream) {
  sparse_small_kernel<<<1, kSmallBlock, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace grace
