// Fused sparse gradient exchange for TopK / DGC / Threshold on sm_100a.
//
// One persistent cooperative kernel does, for a flat buffer holding any number
// of named gradients (segments):
//   A   acc = beta*residual + gamma*g   (DGC: u = m*u + g, v += u, acc = v),
//       store acc as the new residual, zero the output, histogram the top 12
//       magnitude bits per segment (shared-memory histograms, one flush per
//       segment and CTA);
//   P1  per segment, the bin holding the k-th largest magnitude (device-side
//       suffix scan, no host round trip);
//   B   one more streaming pass: everything above the pivot bin goes straight
//       to this rank's send slot, the keys inside the pivot bin go to a small
//       candidate list; picks are staged per warp in shared memory and flushed
//       with one global atomic per flush; the residual (and DGC u, v) is zeroed
//       at the picked positions, which is the whole error-feedback update;
//   P2, P3  the remaining 12 + 7 key bits are resolved on the candidate list
//       only (if the pivot bins hold more keys than the list, the kernel falls
//       back to two more passes over the tensor); exactly k entries come out;
//   publish   st.release.sys of the sequence number into every peer's flag pad;
//   X   for every rank in rank order: bounded wait for its flag, stream its
//       list with ld.global.cg over NVLink and red.global.add.f32 into the
//       dense output scaled by 1/W (a grid barrier separates the lists when
//       W > 2 so that all replicas get bit-identical sums); then acknowledge
//       so the slot can be reused.
//   X'  tile-ordered variant (kTile instantiation, chosen by the host for large
//       tensors whose ranks together deliver a few percent of the elements):
//       before publishing, every rank orders its own picks by 8192-element
//       output tile (counting sort in local memory) and appends a directory of
//       tile offsets; a receiver then reads, for two tiles at a time, each
//       peer's range of the ordered list, adds the ranks in order 0..W-1 in
//       shared memory and writes the tiles once, densely: no global atomics,
//       no zero-fill of the output in pass A, the same bits as X.
// Threshold mode skips the select; random-k mode draws the positions from
// Philox so that only values travel.
//
// What it replaces in the reference: ATen topk / nonzero / scatter_, the
// rdxtopk extension with its three blocking copies per digit
// (radixtopk_cuda/rdxtopk_cuda.cu:459-529), the W dense decompressions of
// communicator/allgather.py:40-45, memory/residual.py:18-20 and
// memory/dgc.py:21-39.
#include <cstdlib>

#include "common.cuh"
#include "exchange.h"
#include "philox.cuh"
#include "segments.cuh"
#include "gradio.cuh"

namespace grace {

namespace {

constexpr int kBlock = 512;
constexpr int kBins = 4096;
constexpr int kStageCap = 8192;           // staged (value, index) pairs per CTA
constexpr int kIterElems = kBlock * 4;    // elements per CTA iteration
constexpr int kCandStage = 4096;          // staged pivot-bin candidates per CTA
constexpr int kWarpStage = kStageCap / (kBlock / 32);   // 512 staged picks per warp
constexpr int kWarpCand = kCandStage / (kBlock / 32);   // 256 staged candidates per warp
constexpr int kTileShift = 13;             // decode tiles of 8192 output elements (32 KiB of shared memory)
constexpr int kTileElems = 1 << kTileShift;
constexpr int kUnroll = 4;                // 16-byte loads in flight per thread and array
constexpr unsigned kSlotHeaderBytes = 128;

__device__ __forceinline__ unsigned ordered_bits(float f) {
  // monotone map float -> unsigned (for atomicMax on signed floats)
  unsigned b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(unsigned b) {
  return __uint_as_float((b & 0x80000000u) ? (b & 0x7fffffffu) : ~b);
}

template <bool B> struct Bool { static constexpr bool value = B; };

struct Smem {
  union {
    unsigned hist[kBins];
    struct {
      float val[kStageCap];
      int idx[kStageCap];
    } stage;
  };
  float cand_val[kCandStage];   // keys of the pivot bin awaiting refinement (fast path), kWarpCand per warp
  int cand_idx[kCandStage];
  unsigned wcnt[kBlock / 32];   // entries staged by each warp
  unsigned ccnt[kBlock / 32];
  unsigned scan[kBlock / 32 + 1];
};

__device__ __forceinline__ void flush_hist(unsigned* __restrict__ shist, unsigned* __restrict__ ghist) {
  __syncthreads();
  for (int b = threadIdx.x; b < kBins; b += kBlock) {
    const unsigned c = shist[b];
    if (c) {
      atomicAdd(ghist + b, c);
      shist[b] = 0;
    }
  }
  __syncthreads();
}
__device__ __forceinline__ void flush_hist(Smem& sm, unsigned* __restrict__ ghist) { flush_hist(sm.hist, ghist); }

// Suffix-scan one segment's histogram and pick the bin holding the `need`-th
// largest key.  All threads of the CTA take part; the histogram is left zero.
__device__ void pivot_segment(Smem& sm, unsigned* __restrict__ ghist, SparseState* __restrict__ st, unsigned need,
                              int bits) {
  constexpr int kPer = kBins / kBlock;  // 8 bins per thread
  const int t = threadIdx.x;
  unsigned c[kPer];
  unsigned local = 0;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    c[j] = ghist[t * kPer + j];
    ghist[t * kPer + j] = 0;
    local += c[j];
  }
  // inclusive scan of `local` over threads in *descending* thread order
  const int lane = t & 31, warp = t >> 5;
  unsigned incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned n = __shfl_down_sync(0xffffffffu, incl, o);
    if (lane + o < 32) incl += n;
  }
  if (lane == 0) sm.scan[warp] = incl;  // warp total
  __syncthreads();
  unsigned above_warps = 0;
  for (int w = warp + 1; w < kBlock / 32; ++w) above_warps += sm.scan[w];
  const unsigned above = above_warps + incl - local;  // keys in bins owned by higher threads
  if (above < need && need <= above + local) {
    unsigned cum = above;
#pragma unroll
    for (int j = kPer - 1; j >= 0; --j) {
      if (cum < need && need <= cum + c[j]) {
        st->prefix = (st->prefix << bits) | (unsigned)(t * kPer + j);
        st->need = need - cum;
        st->tie_taken = 0;
        st->pivot_count = c[j];
      }
      cum += c[j];
    }
  }
  __syncthreads();
}

// kTile selects the tile-ordered exchange (sender orders its list by output tile, receivers build dense
// tiles); it is a separate instantiation so that the scatter-add variant keeps its code and registers.
template <bool kTile>
__global__ void __launch_bounds__(kBlock, 2) sparse_exchange_kernel(const SparseArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const Status status{a.status};
  GridBarrier bar{a.barrier, 0u, a.peers.timeout_ns, status};
  const int tid = threadIdx.x;
  const int rank = a.peers.rank, world = a.peers.world;
  char* const my_heap = a.peers.heap[rank];
  unsigned* const my_hdr = reinterpret_cast<unsigned*>(my_heap + a.peers.slot_off);
  float* const my_vals = reinterpret_cast<float*>(my_heap + a.peers.slot_off + kSlotHeaderBytes);
  int* const my_idx = reinterpret_cast<int*>(my_vals + a.cap);

  // contiguous share of the flat buffer for this CTA
  long long chunk = (a.total + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + kIterElems - 1) / kIterElems * kIterElems;
  const long long lo = (long long)blockIdx.x * chunk;
  const long long hi = lo + chunk < a.total ? lo + chunk : a.total;
  const void* __restrict__ src = a.acc ? (const void*)a.acc : a.g;   // what the passes after A re-read
  const int src_dtype = a.acc ? (int)kGradF32 : a.g_dtype;
  const bool topk = a.mode == kSparseTopK;
  const bool randomk = a.mode == kSparseRandomK;
  const bool dense_decode = kTile && !randomk;  // tile-ordered lists and decode

  if (a.phases & (kPhaseCompress | kPhaseClip)) {
    // Before overwriting anything of parity (seq & 1) in this rank's heap (send slot, clipping sums): every peer
    // must have finished reading what sequence seq-2 put there.  Every CTA waits (the acknowledgement words are
    // local memory), so none of them can touch the slot early.
    if (tid < world && tid != rank && a.peers.seq > 2) {
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ack_off) + tid;
      wait_flag_ge(ack, a.peers.seq - 2, a.peers.timeout_ns, status, kTimeoutPeerAck, tid);
    }
    __syncthreads();
  }

  // ---- phase C (DGC gradient clipping): per tensor sum of g^2 on this rank, published to the peers; the clamp
  //      bound sqrt(mean over ranks of the sums) is then formed by every rank from the W published values, in rank
  //      order.  Replaces torch.sum(g*g) + all_reduce of grace_dl/torch/memory/dgc.py:16-19. ----
  double* const my_clip = reinterpret_cast<double*>(my_heap + a.clip_off) + (size_t)(a.peers.seq & 1) * a.nseg;
  if (a.phases & kPhaseClip) {
    __shared__ double s_sq[kBlock / 32];
    bool okc = !status.failed();
    if (okc && lo < hi) {
      for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
        double part = 0.0;
        for (long long base = b0 + 4ll * tid; base < e0; base += (long long)kUnroll * kIterElems) {
          float gv[kUnroll][4];
#pragma unroll
          for (int q = 0; q < kUnroll; ++q) {
            const long long i = base + (long long)q * kIterElems;
            const int valid = i < e0 ? ((e0 - i) >= 4 ? 4 : (int)(e0 - i)) : 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) gv[q][j] = 0.f;
            if (valid) load4g(a.g, a.g_dtype, i, valid, gv[q]);
          }
          float l = 0.f;
#pragma unroll
          for (int q = 0; q < kUnroll; ++q)
#pragma unroll
            for (int j = 0; j < 4; ++j) l += gv[q][j] * gv[q][j];
          part += (double)l;
        }
        part = warp_sum(part);
        if ((tid & 31) == 0) s_sq[tid >> 5] = part;
        __syncthreads();
        if (tid == 0) {
          double tot = 0.0;
          for (int w = 0; w < kBlock / 32; ++w) tot += s_sq[w];
          atomicAdd(&a.clip_sq[s], tot);
        }
        __syncthreads();
      });
    }
    okc = bar.sync();
    if (okc)
      for (int s = blockIdx.x * kBlock + tid; s < a.nseg; s += gridDim.x * kBlock) {
        my_clip[s] = __ldcg(&a.clip_sq[s]);
        a.clip_sq[s] = 0.0;   // left zero for the next launch
      }
    okc = bar.sync();
    if (blockIdx.x == 0 && tid < world && okc) {
      __threadfence_system();
      uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.clip_ready_off) + rank;
      st_release_sys(flag, a.peers.seq);
    }
  }

  if (a.phases & kPhaseCompress) {
    __shared__ float s_bound;
    if (a.clip_off) {   // the peers' sums must have arrived before the first clamp
      if (tid < world) {
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.clip_ready_off) + tid;
        wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid);
      }
      __syncthreads();
    }
    if (blockIdx.x == 0 && tid == 0) { my_hdr[0] = 0; my_hdr[1] = 0; }
    if (kTile && dense_decode) {   // tile counters of the ordering step; many grid barriers lie between here and their use
      const long long nb1 = ((a.total + kTileElems - 1) >> kTileShift) + 1;
      for (long long b = (long long)blockIdx.x * kBlock + tid; b < nb1; b += (long long)gridDim.x * kBlock) a.tile_start[b] = 0;
    }
    // Hinted second-level histogram: under error feedback the selection threshold moves little from step to step
    // while the accumulated values pile up just below it, so the first-level pivot bin holds a few percent of all
    // elements.  Keys that fall into the bin that was the pivot in the previous launch are therefore also counted by
    // their next 12 bits in this pass; when the pivot bin is the same again, 24 key bits are resolved before the
    // compaction pass and the candidate list shrinks by three orders of magnitude.  A wrong hint costs nothing but the
    // extra counting (the selection never depends on it).  The staging area of the candidates is free in this pass.
    static_assert(sizeof(float) * kCandStage >= sizeof(unsigned) * kBins, "second histogram does not fit");
    unsigned* const s_hist2 = reinterpret_cast<unsigned*>(sm.cand_val);
    const bool hinted = a.fine_hint && topk;
    auto g_hist2 = [&](int s) { return a.hist + ((size_t)a.nseg + s) * kBins; };   // second-level histogram of a segment
    auto g_hint = [&](int s) { return a.hist + 2 * (size_t)a.nseg * kBins + s; };   // its hint word
    for (int b = tid; b < kBins; b += kBlock) { sm.hist[b] = 0; s_hist2[b] = 0; }
    __syncthreads();

    // ---- phase A: compensate, store accumulator, zero output, histogram ----
    if (lo < hi) {
      for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
        float tmax = -INFINITY;
        const bool read_acc = a.u || (a.acc && a.beta != 0.f);
        const unsigned hint = hinted ? *g_hint(s) : 0xffffffffu;
        float clip = INFINITY;   // element-wise clamp of the incoming gradient
        if (a.clip_off) {
          __syncthreads();
          if (tid == 0) {
            double tot = 0.0;
            for (int p = 0; p < world; ++p) {   // rank order: the same bound, bit for bit, on every GPU
              const char* pc = a.peers.heap[p] + a.clip_off + ((size_t)(a.peers.seq & 1) * a.nseg + s) * 8;
              unsigned long long raw;
              asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(raw) : "l"(pc));
              tot += __longlong_as_double((long long)raw);
            }
            s_bound = (float)sqrt(tot / (double)world);
          }
          __syncthreads();
          clip = s_bound;
        }
        auto trip_a = [&](auto full_tag, long long base) {
          constexpr bool kFull = decltype(full_tag)::value;   // all kUnroll vectors fully inside the range
          // issue every load of the trip before the first dependent instruction
          int valid[kUnroll];
          float gv[kUnroll][4], rv[kUnroll][4], uv[kUnroll][4];
#pragma unroll
          for (int q = 0; q < kUnroll; ++q) {
            const long long i = base + (long long)q * kIterElems;
            valid[q] = kFull ? 4 : (i < e0 ? ((e0 - i) >= 4 ? 4 : (int)(e0 - i)) : 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) { rv[q][j] = 0.f; uv[q][j] = 0.f; gv[q][j] = 0.f; }
            if (valid[q]) {
              load4g(a.g, a.g_dtype, i, valid[q], gv[q]);
              if (read_acc) load4(a.acc, i, valid[q], rv[q]);
              if (a.u) load4(a.u, i, valid[q], uv[q]);
            }
          }
#pragma unroll
          for (int q = 0; q < kUnroll; ++q) {
            if (!valid[q]) continue;
            const long long i = base + (long long)q * kIterElems;
            float av[4];
            if (a.clip_off) {
#pragma unroll
              for (int j = 0; j < 4; ++j) gv[q][j] = fminf(fmaxf(gv[q][j], -clip), clip);
            }
            if (a.u) {
#pragma unroll
              for (int j = 0; j < 4; ++j) { uv[q][j] = a.momentum * uv[q][j] + gv[q][j]; av[j] = rv[q][j] + uv[q][j]; }
              store4(a.u, i, valid[q], uv[q]);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) av[j] = a.beta * rv[q][j] + a.gamma * gv[q][j];
            }
            if (a.acc) store4(a.acc, i, valid[q], av);
            if (a.out && !dense_decode) { const float z[4] = {0.f, 0.f, 0.f, 0.f}; store4(a.out, i, valid[q], z); }
            if (topk) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (kFull || j < valid[q]) {
                  const unsigned key = __float_as_uint(av[j]) & 0x7fffffffu;
                  atomicAdd(&sm.hist[key >> 19], 1u);
                  if ((key >> 19) == hint) atomicAdd(&s_hist2[(key >> 7) & 0xfffu], 1u);
                }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) if (kFull || j < valid[q]) tmax = fmaxf(tmax, av[j]);
            }
          }
        };
        {
          const long long trip_elems = (long long)kUnroll * kIterElems;
          long long base = b0 + 4ll * tid;
          for (; base + trip_elems - 4ll * tid <= e0; base += trip_elems) trip_a(Bool<true>{}, base);
          for (; base < e0; base += trip_elems) trip_a(Bool<false>{}, base);
        }
        if (topk) {
          flush_hist(sm, a.hist + (size_t)s * kBins);
          if (hint != 0xffffffffu) flush_hist(s_hist2, g_hist2(s));
        } else if (!randomk) {
          tmax = warp_max(tmax);
          if ((tid & 31) == 0 && tmax > -INFINITY) atomicMax(&a.state[s].max_bits, ordered_bits(tmax));
        }
      });
    }
    // zero the padding gaps of the output (between segments) is unnecessary:
    // nothing ever writes there.
    bool ok = bar.sync();
    bool fast = false;
    SparseState* const extra = a.state + a.nseg;  // [prefix] = candidate total, [need] = candidate cursor

    if (topk) {
      // ---- radix select: levels of 12, 12 and 7 key bits ----
      // Fast path (exact mode): when the pivot bins of the first level are small enough, the
      // compaction pass also collects their keys into a candidate list and the remaining two levels
      // run on that list only: two streaming passes over the tensor instead of four.
      const int nlevels = a.levels;
      for (int level = 0; level < nlevels; ++level) {
        const int bits = level == 2 ? 7 : 12;
        if (ok) {
          for (int s = blockIdx.x; s < a.nseg; s += gridDim.x) {
            if (level == 1 && a.state[s].fine) continue;   // its second level came with the first pass
            const unsigned need = level == 0 ? (unsigned)a.segs[s].k : a.state[s].need;
            pivot_segment(sm, a.hist + (size_t)s * kBins, &a.state[s], need, bits);
            if (level == 0) {
              if (hinted) {
                const unsigned hint = *g_hint(s), p0 = a.state[s].prefix;
                if (hint == p0) {
                  pivot_segment(sm, g_hist2(s), &a.state[s], a.state[s].need, 12);
                } else if (hint != 0xffffffffu) {
                  for (int b = tid; b < kBins; b += kBlock) g_hist2(s)[b] = 0;   // leave it zero
                }
                __syncthreads();   // every thread has read the hint word before thread 0 replaces it
                if (tid == 0) {
                  *g_hint(s) = p0;
                  a.state[s].fine = hint == p0 ? 1u : 0u;
                }
                __syncthreads();
              }
              if (tid == 0) atomicAdd(&extra->prefix, a.state[s].pivot_count);   // candidates of this segment
            }
          }
        }
        ok = bar.sync();
        if (level == 0 && nlevels == 3 && a.cand_cap) {
          // extra->prefix now holds the exact number of keys in the pivot bins of all segments
          fast = ld_acquire_gpu(&extra->prefix) <= a.cand_cap;
          if (fast) break;
        }
        if (level + 1 < nlevels) {
          // histogram of the next digit among keys that match the prefix
          const int shift_prefix = level == 0 ? 19 : 7;
          const int shift_digit = level == 0 ? 7 : 0;
          const unsigned digit_mask = level == 0 ? 0xfffu : 0x7fu;
          if (ok && lo < hi) {
            for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
              const unsigned prefix = a.state[s].prefix;
              if (level == 0 && a.state[s].fine) return;   // 24 bits are known already
              for (long long base = b0 + 4ll * tid; base < e0; base += (long long)kUnroll * kIterElems) {
                int valid[kUnroll];
                float av[kUnroll][4];
#pragma unroll
                for (int q = 0; q < kUnroll; ++q) {
                  const long long i = base + (long long)q * kIterElems;
                  valid[q] = i < e0 ? ((e0 - i) >= 4 ? 4 : (int)(e0 - i)) : 0;
                  if (valid[q]) load4g(src, src_dtype, i, valid[q], av[q]);
                }
#pragma unroll
                for (int q = 0; q < kUnroll; ++q) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (j >= valid[q]) continue;
                    const unsigned key = __float_as_uint(av[q][j]) & 0x7fffffffu;
                    if ((key >> shift_prefix) == prefix) atomicAdd(&sm.hist[(key >> shift_digit) & digit_mask], 1u);
                  }
                }
              }
              flush_hist(sm, a.hist + (size_t)s * kBins);
            });
          }
          ok = bar.sync();
        }
      }
    }

    // ---- phase B: compaction into the send slot + error-feedback update ----
    // Every warp stages its picks in its own slice of shared memory and flushes it by itself
    // (one global atomic per flush, coalesced copies): the streaming loop has no CTA barrier.
    __syncthreads();
    const int key_shift_all = topk ? (fast ? 19 : (a.levels == 3 ? 0 : (a.levels == 2 ? 7 : 19))) : 0;
    const int lane = tid & 31, warp = tid >> 5;
    const unsigned lane_lt = (1u << lane) - 1u;
    float* const w_val = sm.stage.val + warp * kWarpStage;
    int* const w_idx = sm.stage.idx + warp * kWarpStage;
    float* const c_val = sm.cand_val + warp * kWarpCand;
    int* const c_idx = sm.cand_idx + warp * kWarpCand;
    if (lane == 0) { sm.wcnt[warp] = 0; sm.ccnt[warp] = 0; }
    __syncwarp();
    auto flush_warp = [&]() {
      __syncwarp();
      const unsigned wcount = sm.wcnt[warp];
      unsigned base = 0;
      if (lane == 0 && wcount) base = atomicAdd(&my_hdr[0], wcount);
      base = __shfl_sync(0xffffffffu, base, 0);
      for (unsigned e = lane; e < wcount; e += 32) {
        const unsigned pos = base + e;
        if (pos < a.cap) {
          my_vals[pos] = w_val[e];
          my_idx[pos] = w_idx[e];
        } else {
          // no room: give the value back to the residual so nothing is lost
          if (a.acc) a.acc[w_idx[e]] = w_val[e];
          atomicAdd(&a.status[3], 1u);
        }
      }
      __syncwarp();
      if (lane == 0) sm.wcnt[warp] = 0;
      __syncwarp();
    };
    auto flush_warp_cand = [&]() {
      __syncwarp();
      const unsigned ccount = sm.ccnt[warp];
      unsigned base = 0;
      if (lane == 0 && ccount) base = atomicAdd(&extra->need, ccount);
      base = __shfl_sync(0xffffffffu, base, 0);
      for (unsigned e = lane; e < ccount; e += 32) {
        const unsigned pos = base + e;
        if (pos < a.cand_cap) { a.cand_val[pos] = c_val[e]; a.cand_idx[pos] = c_idx[e]; }
      }
      __syncwarp();
      if (lane == 0) sm.ccnt[warp] = 0;
      __syncwarp();
    };
    if (ok && randomk) {
      // ---- random-k: gather the agreed positions; the residual is zeroed there after a barrier
      //      (positions are drawn with replacement, duplicates must all read the same value) ----
      const int total_k = a.kprefix[a.nseg];
      auto locate = [&](int e, int& sgm) {
        int lo_s = 0, hi_s = a.nseg;
        while (lo_s + 1 < hi_s) {
          const int m = (lo_s + hi_s) >> 1;
          if (a.kprefix[m] <= e) lo_s = m; else hi_s = m;
        }
        sgm = lo_s;
      };
      for (int e = blockIdx.x * kBlock + tid; e < total_k; e += gridDim.x * kBlock) {
        int sgm;
        locate(e, sgm);
        const unsigned j = (unsigned)(e - a.kprefix[sgm]);
        const Philox4 r4 = philox_group((uint64_t)(j >> 2), a.rk_step, 7u, a.seg_seed[sgm]);
        const unsigned word = (j & 3) == 0 ? r4.x : ((j & 3) == 1 ? r4.y : ((j & 3) == 2 ? r4.z : r4.w));
        const long long idx = a.segs[sgm].offset + (long long)(word % (unsigned)a.segs[sgm].numel);
        my_vals[e] = load1g(src, src_dtype, idx);
        my_idx[e] = (int)idx;
      }
      ok = bar.sync();
      if (ok && a.acc)
        for (int e = blockIdx.x * kBlock + tid; e < total_k; e += gridDim.x * kBlock) a.acc[my_idx[e]] = 0.f;
      if (blockIdx.x == 0 && tid == 0) my_hdr[0] = (unsigned)total_k;
    }
    if (ok && lo < hi && !randomk) {
      for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
        const unsigned pivot = a.state[s].prefix;
        const unsigned need = a.state[s].need;
        // a hinted segment enters the candidate pass with 24 resolved key bits instead of 12
        const int key_shift = (topk && fast && a.state[s].fine) ? 7 : key_shift_all;
        float thr = a.threshold;
        if (!topk && !a.strict) thr = fminf(thr, from_ordered_bits(a.state[s].max_bits));   // dist flavour: capped by max(x)
        const bool strict = a.strict != 0;                                                  // Horovod flavour: |x| > threshold
        auto trip_b = [&](auto full_tag, long long base) {
          constexpr bool kFull = decltype(full_tag)::value;
          int valid[kUnroll];
          float avs[kUnroll][4];
#pragma unroll
          for (int q = 0; q < kUnroll; ++q) {
            const long long i = base + (long long)q * kIterElems;
            valid[q] = kFull ? 4 : (i < e0 ? ((e0 - i) >= 4 ? 4 : (int)(e0 - i)) : 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) avs[q][j] = 0.f;
            if (valid[q]) load4g(src, src_dtype, i, valid[q], avs[q]);
          }
#pragma unroll
          for (int q = 0; q < kUnroll; ++q) {
            const long long i = base + (long long)q * kIterElems;
            const float (&av)[4] = avs[q];
            // a warp adds at most 128 entries per step to either stage
            __syncwarp();
            if (sm.wcnt[warp] + 128 > kWarpStage) flush_warp();
            if (fast && sm.ccnt[warp] + 128 > kWarpCand) flush_warp_cand();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (!kFull && j >= valid[q]) continue;
              bool hit;  // rare: this element is picked or is a candidate
              unsigned kp = 0;
              if (topk) {
                kp = (__float_as_uint(av[j]) & 0x7fffffffu) >> key_shift;
                hit = kp >= pivot;
              } else {
                hit = strict ? fabsf(av[j]) > thr : fabsf(av[j]) >= thr;
              }
              if (hit) {
                bool sel = true;
                if (topk && kp == pivot) {
                  sel = false;
                  if (fast) {  // decided later, on the candidate list
                    const unsigned pos = atomicAdd(&sm.ccnt[warp], 1u);
                    c_val[pos] = av[j];
                    c_idx[pos] = (int)(i + j);
                  } else {
                    sel = atomicAdd(&a.state[s].tie_taken, 1u) < need;
                  }
                }
                if (sel) {
                  const unsigned pos = atomicAdd(&sm.wcnt[warp], 1u);
                  w_val[pos] = av[j];
                  w_idx[pos] = (int)(i + j);
                  if (GRACE_IN_RANGE(status, kKernelSparse, i + j, a.total)) {
                    if (a.acc) a.acc[i + j] = 0.f;
                    if (a.u) a.u[i + j] = 0.f;
                  }
                }
              }
            }
          }
        };
        const long long trip_elems = (long long)kUnroll * kIterElems;
        long long base = b0 + 4ll * tid;
        for (; base + trip_elems - 4ll * tid <= e0; base += trip_elems) trip_b(Bool<true>{}, base);
        // the guarded tail must be executed by whole warps together (flush checks are warp-wide)
        for (long long wb = base - 4ll * lane; wb < e0; wb += trip_elems) trip_b(Bool<false>{}, wb + 4ll * lane);
      });
    }
    flush_warp();
    if (fast) flush_warp_cand();
    ok = bar.sync();
    if (fast) {
      // ---- refinement on the candidate list: 12-bit and 7-bit levels, then the final picks ----
      const unsigned ncand = min(ld_acquire_gpu(&extra->need), a.cand_cap);
      const unsigned gtid = blockIdx.x * kBlock + tid, gstride = gridDim.x * kBlock;
      auto seg_of = [&](int idx) {
        int lo_s = 0, hi_s = a.nseg;
        while (lo_s + 1 < hi_s) {
          const int m = (lo_s + hi_s) >> 1;
          if (a.segs[m].offset <= idx) lo_s = m; else hi_s = m;
        }
        return lo_s;
      };
      for (int level = 1; level < 3; ++level) {
        if (ok) {
          for (unsigned e = gtid; e < ncand; e += gstride) {
            const unsigned key = __float_as_uint(a.cand_val[e]) & 0x7fffffffu;
            const int sg = seg_of(a.cand_idx[e]);
            if (level == 1) {
              if (!a.state[sg].fine) atomicAdd(&a.hist[(size_t)sg * kBins + ((key >> 7) & 0xfffu)], 1u);
            } else if ((key >> 7) == a.state[sg].prefix) {
              atomicAdd(&a.hist[(size_t)sg * kBins + (key & 0x7fu)], 1u);
            }
          }
        }
        ok = bar.sync();
        if (ok) {
          for (int sg = blockIdx.x; sg < a.nseg; sg += gridDim.x) {
            if (level == 1 && a.state[sg].fine) continue;
            pivot_segment(sm, a.hist + (size_t)sg * kBins, &a.state[sg], a.state[sg].need, level == 2 ? 7 : 12);
          }
        }
        ok = bar.sync();
      }
      if (ok) {
        for (unsigned e0 = blockIdx.x * kBlock; e0 < ncand; e0 += gstride) {   // warp-uniform trip count
          const unsigned e = e0 + tid;
          bool sel = false;
          float v = 0.f;
          int idx = 0;
          if (e < ncand) {
            v = a.cand_val[e];
            idx = a.cand_idx[e];
            const unsigned key = __float_as_uint(v) & 0x7fffffffu;
            const int sg = seg_of(idx);
            const unsigned thr_key = a.state[sg].prefix;
            sel = key > thr_key;
            if (key == thr_key) sel = atomicAdd(&a.state[sg].tie_taken, 1u) < a.state[sg].need;
          }
          const unsigned ballot = __ballot_sync(0xffffffffu, sel);
          unsigned wbase = 0;
          if ((tid & 31) == 0 && ballot) wbase = atomicAdd(&my_hdr[0], __popc(ballot));
          wbase = __shfl_sync(0xffffffffu, wbase, 0);
          if (sel) {
            const unsigned pos = wbase + __popc(ballot & ((1u << (tid & 31)) - 1u));
            if (pos < a.cap) {
              my_vals[pos] = v;
              my_idx[pos] = idx;
              if (a.acc) a.acc[idx] = 0.f;
              if (a.u) a.u[idx] = 0.f;
            } else {
              atomicAdd(&a.status[3], 1u);
            }
          }
        }
      }
      ok = bar.sync();
    }
    if constexpr (kTile) if (dense_decode) {
      // ---- order the list by output tile (counting sort of this rank's own picks, all in local memory) and
      //      publish a directory of tile offsets: the receivers then build whole tiles without any sorting ----
      const long long tiles = (a.total + kTileElems - 1) >> kTileShift;
      const unsigned nbins = (unsigned)tiles;
      const unsigned gtid = blockIdx.x * kBlock + tid, gstride = gridDim.x * kBlock;
      const unsigned n_mine = min(ld_cg_u32(my_hdr), a.cap);   // every pick is counted: a grid barrier lies behind us
      float* const s_vals = my_vals + 2 * (size_t)a.cap;       // second pair of arrays in the slot: the ordered list
      int* const s_idx = reinterpret_cast<int*>(s_vals + a.cap);
      unsigned* const dir = reinterpret_cast<unsigned*>(s_vals + 2 * (size_t)a.cap);
      __shared__ unsigned s_scan[kBlock / 32];
      __shared__ unsigned s_carry;
      const unsigned lane_id = tid & 31;
      const unsigned groups = (n_mine + 3) / 4;
      const unsigned trips = (groups + gstride - 1) / gstride;   // uniform trip count: warp collectives inside
      auto for_each_mine = [&](auto&& fn) {
        for (unsigned t = 0; t < trips; ++t) {
          const unsigned gidx = t * gstride + gtid;
          uint4 v = make_uint4(0u, 0u, 0u, 0u), ix = make_uint4(0u, 0u, 0u, 0u);
          if (gidx < groups) {
            v = ld_cg_u4(my_vals + (size_t)gidx * 4);
            ix = ld_cg_u4(my_idx + (size_t)gidx * 4);
          }
          const unsigned idx4[4] = {ix.x, ix.y, ix.z, ix.w};
          const unsigned val4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const bool use = gidx < groups && gidx * 4 + j < n_mine && idx4[j] < (unsigned)a.total;
            const unsigned bin = use ? idx4[j] >> kTileShift : 0xffffffffu;
            // lanes with the same tile elect a leader that touches the counter once
            const unsigned mask = __match_any_sync(0xffffffffu, bin);
            fn(use, bin, mask, idx4[j], val4[j]);
          }
        }
      };
      // S1: count the picks per tile (the counters were zeroed at the start of the kernel)
      if (ok) {
        for_each_mine([&](bool use, unsigned bin, unsigned mask, unsigned, unsigned) {
          if (use && lane_id == (unsigned)(__ffs(mask) - 1)) atomicAdd(&a.tile_start[bin], (unsigned)__popc(mask));
        });
      }
      ok = bar.sync();
      // S2: exclusive prefix sum over the tiles (CTA-chunked two-level scan) -> directory
      const unsigned chunk_bins = (nbins + gridDim.x - 1) / gridDim.x;
      const unsigned cb0 = blockIdx.x * chunk_bins, cb1 = min(cb0 + chunk_bins, nbins);
      auto block_sum = [&](unsigned v) {
        v = (unsigned)warp_sum((int)v);
        if ((tid & 31) == 0) s_scan[tid >> 5] = v;
        __syncthreads();
        unsigned tot = 0;
        for (int w = 0; w < kBlock / 32; ++w) tot += s_scan[w];
        __syncthreads();
        return tot;
      };
      if (ok) {
        unsigned part = 0;
        for (unsigned b = cb0 + tid; b < cb1; b += kBlock) part += __ldcg(a.tile_start + b);
        const unsigned tot = block_sum(part);
        if (tid == 0) a.scan_tmp[blockIdx.x] = tot;
      }
      ok = bar.sync();
      if (ok) {
        unsigned part = 0;
        for (unsigned c = tid; c < blockIdx.x; c += kBlock) part += __ldcg(a.scan_tmp + c);
        unsigned running = block_sum(part);   // pairs in all earlier chunks
        if (tid == 0) s_carry = running;
        __syncthreads();
        for (unsigned b0 = cb0; b0 < cb1; b0 += kBlock) {
          const unsigned b = b0 + tid;
          const unsigned c = b < cb1 ? __ldcg(a.tile_start + b) : 0u;
          // block-wide exclusive scan of c
          unsigned incl = c;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const unsigned nb = __shfl_up_sync(0xffffffffu, incl, o);
            if ((tid & 31) >= o) incl += nb;
          }
          if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
          __syncthreads();
          unsigned before = 0;
          for (int w = 0; w < (tid >> 5); ++w) before += s_scan[w];
          const unsigned excl = s_carry + before + incl - c;
          if (b < cb1) { a.tile_start[b] = excl; a.tile_cur[b] = excl; dir[b] = excl; }
          __syncthreads();
          if (tid == kBlock - 1) s_carry = excl + c;
          __syncthreads();
        }
        if (blockIdx.x == gridDim.x - 1 && tid == 0) { a.tile_start[nbins] = s_carry; dir[nbins] = s_carry; }  // sentinel = list length
      }
      ok = bar.sync();
      // S3: move every pick to its tile's block of the ordered list
      if (ok) {
        for_each_mine([&](bool use, unsigned bin, unsigned mask, unsigned idx, unsigned val) {
          unsigned base = 0;
          const unsigned leader = (unsigned)(__ffs(mask) - 1);
          if (use && lane_id == leader) base = atomicAdd(&a.tile_cur[bin], (unsigned)__popc(mask));
          base = __shfl_sync(0xffffffffu, base, leader);   // every lane takes part; only members of `mask` use it
          if (use) {
            const unsigned pos = base + __popc(mask & ((1u << lane_id) - 1u));
            if (GRACE_IN_RANGE(status, kKernelSparse, pos, a.cap)) {
              s_vals[pos] = __uint_as_float(val);
              s_idx[pos] = (int)idx;
            }
          }
        });
      }
      ok = bar.sync();
    }
    if (blockIdx.x == 0 && tid == 0) {
      // clamp the published count to the capacity
      const unsigned n = my_hdr[0];
      if (n > a.cap) { my_hdr[1] = n - a.cap; my_hdr[0] = a.cap; }
      __threadfence_system();
    }
  }

  if (a.phases & kPhasePublish) {
    // All CTAs' slot writes are ordered before this point by the barrier above
    // (or by the kernel boundary when phases are launched separately).
    if (blockIdx.x == 0) {
      __syncthreads();
      if (tid < world && !status.failed()) {
        __threadfence_system();
        uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ready_off) + rank;
        st_release_sys(flag, a.peers.seq);
      }
    }
  }

  if (a.phases & kPhaseExchange) {
    // ---- phase X: pull every rank's list and scatter-add it ----
    if (randomk) {
      __shared__ int s_rk_ok;
      if (tid == 0) s_rk_ok = 1;
      __syncthreads();
      if (tid < world) {
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + tid;
        if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) s_rk_ok = 0;
      }
      __syncthreads();
      const int total_k = a.kprefix[a.nseg];
      if (s_rk_ok) {
        for (int e = blockIdx.x * kBlock + tid; e < total_k; e += gridDim.x * kBlock) {
          float sum = 0.f;
          for (int p = 0; p < world; ++p)
            sum += ld_cg_f32(a.peers.heap[p] + a.peers.slot_off + kSlotHeaderBytes + (size_t)e * 4);
          a.out[my_idx[e]] = sum * a.scale;   // duplicates of a position write the same value
        }
      }
      bar.sync();
      if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
        uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
        st_release_sys(ack, a.peers.seq);
      }
      return;
    }
    if constexpr (kTile) if (dense_decode && a.out) {
      // ---- tile-ordered decode: every peer's list arrives sorted by 8192-element output tile with a
      //      directory of tile offsets, so each CTA builds whole output tiles in shared memory (source
      //      ranks in order 0..W-1) and writes them once, densely; nothing is scattered to global memory ----
      constexpr int kR = 8;                          // pairs per thread and chunk
      constexpr int kGroup = 2;                      // tiles per unit: stage.val and stage.idx hold one each
      constexpr int kUnitElems = kGroup * kTileElems;
      __shared__ unsigned s_n[kMaxWorld];
      __shared__ unsigned s_b[3][kMaxWorld][2];      // per unit (ring of 3) and peer: first and one-past-last entry
      __shared__ unsigned s_pref[3][kMaxWorld + 1];  // running sum of the peers' range lengths
      const long long tiles = (a.total + kTileElems - 1) >> kTileShift;
      const long long units = (tiles + kGroup - 1) / kGroup;
      const size_t sorted_off = kSlotHeaderBytes + (size_t)a.cap * 8, dir_off = sorted_off + (size_t)a.cap * 8;
      if (tid < world) {
        unsigned n = 0;
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + tid;
        if (wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid))
          n = ld_cg_u32(a.peers.heap[tid] + a.peers.slot_off);
        s_n[tid] = n < a.cap ? n : a.cap;
      }
      __syncthreads();
      __shared__ int s_go;
      if (tid == 0) s_go = !status.failed();         // one decision for the whole CTA: the loop below holds barriers
      __syncthreads();
      if (s_go) {
        float* tile = sm.stage.val;                  // val[8192] and idx[8192] are adjacent: 16384 floats
        auto fetch_bound = [&](long long u) {        // thread 2p+k: entry k (0: first, 1: end) of peer p
          const int p = tid >> 1;
          long long t = u * kGroup + (tid & 1) * kGroup;
          if (t > tiles) t = tiles;
          const unsigned d = ld_cg_u32(a.peers.heap[p] + a.peers.slot_off + dir_off + (size_t)t * 4);
          return d < s_n[p] ? d : s_n[p];            // a directory can never point past the list
        };
        auto prefix_of = [&](int ring) {             // warp 0: running sum of range lengths
          if (tid < 32) {
            unsigned len = 0;
            if (tid < world) {
              const unsigned d0 = s_b[ring][tid][0], d1 = s_b[ring][tid][1];
              len = d1 > d0 ? d1 - d0 : 0u;
            }
            unsigned incl = len;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const unsigned nb = __shfl_up_sync(0xffffffffu, incl, o);
              if (tid >= o) incl += nb;
            }
            if (tid < world) s_pref[ring][tid + 1] = incl;
            if (tid == 0) s_pref[ring][0] = 0;
          }
        };
        // pairs j0 + r * kBlock + tid of a unit's concatenated ranges (rank-major), fetched from the peers
        auto load_chunk = [&](uint2 (&pr)[kR], int (&src)[kR], int ring, unsigned j0) {
          const unsigned total_len = s_pref[ring][world];
#pragma unroll
          for (int r = 0; r < kR; ++r) {
            const unsigned j = j0 + r * kBlock + tid;
            src[r] = -1;
            pr[r] = make_uint2(0u, 0u);
            if (j < total_len) {
              int p = 0;                             // last p with pref[p] <= j (world <= 16: four halving steps)
#pragma unroll
              for (int step = 8; step > 0; step >>= 1)
                if (p + step < world && s_pref[ring][p + step] <= j) p += step;
              const size_t e = (size_t)s_b[ring][p][0] + (j - s_pref[ring][p]);
              const char* pv = a.peers.heap[p] + a.peers.slot_off + sorted_off;
              pr[r].x = ld_cg_u32(pv + e * 4);
              pr[r].y = ld_cg_u32(pv + ((size_t)a.cap + e) * 4);
              src[r] = p;
            }
          }
        };
        long long u = blockIdx.x;
        if (tid < 2 * world) {
          if (u < units) s_b[0][tid >> 1][tid & 1] = fetch_bound(u);
          if (u + gridDim.x < units) s_b[1][tid >> 1][tid & 1] = fetch_bound(u + gridDim.x);
        }
        __syncthreads();
        if (u < units) prefix_of(0);
        if (u + gridDim.x < units) prefix_of(1);
        __syncthreads();
        uint2 pr[kR], prn[kR];
        int src[kR], srcn[kR];
        if (u < units) load_chunk(pr, src, 0, 0u);
        int cur = 0;
        for (; u < units; u += gridDim.x) {
          const int nxt = cur == 2 ? 0 : cur + 1, nn = nxt == 2 ? 0 : nxt + 1;
          const bool more = u + gridDim.x < units, more2 = u + 2 * (long long)gridDim.x < units;
          // the directory entries two units ahead and the first chunk of the next unit travel while this one is built
          unsigned nb = 0;
          if (more2 && tid < 2 * world) nb = fetch_bound(u + 2 * (long long)gridDim.x);
          if (more) load_chunk(prn, srcn, nxt, 0u);
          for (int i = tid * 4; i < kUnitElems; i += kBlock * 4)
            *reinterpret_cast<float4*>(tile + i) = make_float4(0.f, 0.f, 0.f, 0.f);
          __syncthreads();
          const unsigned total_len = s_pref[cur][world];
          for (unsigned j0 = 0; j0 < total_len; j0 += kBlock * kR) {
            if (j0 != 0) load_chunk(pr, src, cur, j0);
            // ranks present in this chunk (uniform over the CTA)
            const unsigned jlast = min(j0 + kBlock * kR, total_len) - 1;
            int p_first = 0, p_last = 0;
#pragma unroll
            for (int step = 8; step > 0; step >>= 1) {
              if (p_first + step < world && s_pref[cur][p_first + step] <= j0) p_first += step;
              if (p_last + step < world && s_pref[cur][p_last + step] <= jlast) p_last += step;
            }
            for (int p = p_first; p <= p_last; ++p) {
#pragma unroll
              for (int r = 0; r < kR; ++r)
                if (src[r] == p) {
                  if ((long long)(pr[r].y >> (kTileShift + 1)) != u) {   // not an index of this unit: corrupt list
                    status.fail(kBadArgument, p, (unsigned)a.peers.seq);
                  } else {   // product rounded first, as in the scatter-add decode
                    float* slot = tile + (pr[r].y & (kUnitElems - 1));
                    *slot = __fadd_rn(*slot, __fmul_rn(__uint_as_float(pr[r].x), a.scale));
                  }
                }
              __syncthreads();
            }
          }
          const long long base = u * kUnitElems;
          for (int i = tid * 4; i < kUnitElems; i += kBlock * 4) {
            const long long gi = base + i;
            if (gi + 4 <= a.total) {
              *reinterpret_cast<float4*>(a.out + gi) = *reinterpret_cast<const float4*>(tile + i);
            } else {
              for (int j = 0; j < 4; ++j) if (gi + j < a.total) a.out[gi + j] = tile[i + j];
            }
          }
          if (more2 && tid < 2 * world) s_b[nn][tid >> 1][tid & 1] = nb;
#pragma unroll
          for (int r = 0; r < kR; ++r) { pr[r] = prn[r]; src[r] = srcn[r]; }
          __syncthreads();
          if (more2) prefix_of(nn);
          __syncthreads();
          cur = nxt;
        }
      }
      bar.sync();
      if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
        uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
        st_release_sys(ack, a.peers.seq);
      }
      return;
    }
    // Lists are applied in rank order 0..W-1 on every rank, with a grid barrier between
    // lists when more than two ranks contribute: floating-point addition is not
    // associative, and all replicas must end up with bit-identical gradients.
    for (int p = 0; p < world; ++p) {
      __shared__ unsigned peer_count;
      if (tid == 0) {
        unsigned n = 0;
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + p;
        if (wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, p))
          n = ld_cg_u32(a.peers.heap[p] + a.peers.slot_off);
        peer_count = n < a.cap ? n : a.cap;
      }
      __syncthreads();
      const unsigned n = peer_count;
      const char* pv = a.peers.heap[p] + a.peers.slot_off + kSlotHeaderBytes;
      const char* pi = pv + (size_t)a.cap * 4;
      const unsigned groups = (n + 3) / 4;
      for (unsigned gidx = blockIdx.x * kBlock + tid; gidx < groups; gidx += gridDim.x * kBlock) {
        const uint4 v = ld_cg_u4(pv + (size_t)gidx * 16);
        const uint4 ix = ld_cg_u4(pi + (size_t)gidx * 16);
        const unsigned e = gidx * 4;
        const unsigned lim = (unsigned)a.total;
        if ((ix.x >= lim) | (e + 1 < n && ix.y >= lim) | (e + 2 < n && ix.z >= lim) | (e + 3 < n && ix.w >= lim)) {
          status.fail(kBadArgument, p, (unsigned)a.peers.seq);  // corrupt index: skip, never dereference
          continue;
        }
        atomicAdd(a.out + ix.x, __uint_as_float(v.x) * a.scale);
        if (e + 1 < n) atomicAdd(a.out + ix.y, __uint_as_float(v.y) * a.scale);
        if (e + 2 < n) atomicAdd(a.out + ix.z, __uint_as_float(v.z) * a.scale);
        if (e + 3 < n) atomicAdd(a.out + ix.w, __uint_as_float(v.w) * a.scale);
      }
      __syncthreads();
      if (world > 2 && p + 1 < world) bar.sync();
    }
    // acknowledge: the peers may now reuse their slot of this parity
    bar.sync();
    if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
      uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
      st_release_sys(ack, a.peers.seq);
    }
  }
}

}  // namespace

size_t sparse_slot_bytes(unsigned cap, long long tiled_total) {
  size_t bytes = kSlotHeaderBytes + (size_t)cap * 8;
  if (tiled_total > 0) {   // tile-ordered copy of the list + directory (one entry per tile and a sentinel)
    const size_t tiles = (size_t)((tiled_total + kTileElems - 1) >> kTileShift);
    bytes += (size_t)cap * 8 + (tiles + 1 + 3) / 4 * 16;
  }
  return bytes;
}
size_t sparse_smem_bytes() { return sizeof(Smem); }

int sparse_max_grid(int device, int sm_limit) {
  static bool attr_set[64] = {};
  if (device >= 0 && device < 64 && !attr_set[device]) {
    cudaFuncSetAttribute(sparse_exchange_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
    cudaFuncSetAttribute(sparse_exchange_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
    attr_set[device] = true;
  }
  int per_sm = 0, per_sm_tile = 0, sms = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sparse_exchange_kernel<false>, kBlock, sizeof(Smem));
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_tile, sparse_exchange_kernel<true>, kBlock, sizeof(Smem));
  if (per_sm_tile < per_sm) per_sm = per_sm_tile;   // one grid size serves both variants
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  if (per_sm > 2) per_sm = 2;
  return per_sm * sms;
}

cudaError_t launch_sparse_exchange(const SparseArgs& a, int grid, cudaStream_t stream) {
  if ((a.phases & kPhaseClip) && (!a.clip_off || !a.clip_sq)) return cudaErrorInvalidValue;
  static const bool small_enabled = [] {
    const char* e = getenv("GRACE_SMALL_KERNEL");
    return !(e && e[0] == '0');
  }();
  if (small_enabled && sparse_small_applies(a)) return launch_sparse_small(a, stream);
  cudaError_t err = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (err != cudaSuccess) return err;
  if (a.phases & kPhaseCompress) {
    err = cudaMemsetAsync(a.state, 0, sizeof(SparseState) * (size_t)(a.nseg + 1), stream);
    if (err != cudaSuccess) return err;
  }
  SparseArgs copy = a;
  void* params[] = {&copy};
  const void* fn = a.tile_start ? (const void*)sparse_exchange_kernel<true> : (const void*)sparse_exchange_kernel<false>;
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kBlock), params, sizeof(Smem), stream);
}

}  // namespace grace
