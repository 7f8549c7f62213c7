// Fused quantised gradient exchange on sm_100a: QSGD, TernGrad, natural
// compression, the 8-bit dynamic-tree code, signSGD / signum (majority vote),
// EF-signSGD, 1-bit SGD and the fp16 cast.
//
// One persistent cooperative kernel per exchange:
//   S   (codecs that need per-tensor statistics) acc = beta*residual + gamma*g,
//       store acc, reduce sum / sum of squares / max|x| / signed partial sums
//       per segment;
//   E   encode 128 elements per warp step: stochastic rounding with
//       Philox4x32-10 drawn in registers, bit-pack with warp ballots, write the
//       codes into this rank's send slot and residual = acc - decode(code);
//   publish, then
//   X   every warp owns output groups of 128 elements: it loads the same
//       group of codes from all W send slots (ld.global.cg over NVLink, rank
//       order 0..W-1 so that every rank computes bit-identical sums),
//       dequantises, accumulates in fp32 or counts votes, and stores the
//       aggregate.
// For QSGD (128-element buckets) and natural compression the default at 2..8 ranks and 32 Mi elements or more is
// the pipelined form of this pull (quant_pipeline_kernel below): tiles of the buffer are drawn from one queue in
// which the encode tiles of chunk c + 1 come before the decode tiles of chunk c, every chunk is published as soon
// as its last tile is encoded, and the pull of chunk c over NVLink runs next to the encode of chunk c + 1.
// Two more transports exist besides this pull: the two-phase mode (compressed
// reduce-scatter, re-encode, compressed all-gather; `alltoall`), and the push
// mode (kPush instantiation): every store of pass E is a multimem.st through the
// NVSwitch multicast mapping into region `rank` of all GPUs' receive areas, and
// pass X reads local memory only.
//
// Replaces, in the reference: grace_dl/dist/compressor/{qsgd,terngrad,natural,
// signsgd,signum,efsignsgd,onebit,fp16}.py, qsgd_cuda/qsgd_cuda.cu (K4-K6 and
// the unbound fused attempts K7-K13), cnat_cuda/cnat_cuda.cu (K1-K3),
// grace_dl/tensorflow/compressor/u8bit.py, the W dense decompressions in
// communicator/allgather.py:40-45 and memory/{residual,efsignsgd}.py.
#include <cuda_fp16.h>

#include "common.cuh"
#include "exchange.h"
#include "philox.cuh"
#include "segments.cuh"
#include "gradio.cuh"

namespace grace {

__constant__ float c_u8_edges[128];

namespace {

constexpr int kBlock = 512;
constexpr int kWarps = kBlock / 32;
constexpr int kIterElems = kBlock * 4;
constexpr unsigned kHeaderBytes = 128;
constexpr int kU = 4;  // groups per warp trip whose loads are issued up front
// Staged decode (1-, 2- and 8-bit codes, 2..kStagePeers ranks): every warp owns a staging area in shared memory
// that takes 512 bytes of codes from each rank (and four QSGD norms), so the loads from ALL ranks are in flight
// together and no register has to hold them while the sums are formed.
constexpr int kStagePeers = 8;
constexpr int kStageWarpBytes = kStagePeers * (512 + 16);
constexpr int kStageBytes = kWarps * kStageWarpBytes;

template <int C> struct CodecTraits;
template <> struct CodecTraits<kCodecQSGD>     { static constexpr bool stats = false; static constexpr int bits = 8; };
template <> struct CodecTraits<kCodecTernGrad> { static constexpr bool stats = true;  static constexpr int bits = 2; };
template <> struct CodecTraits<kCodecNatural>  { static constexpr bool stats = false; static constexpr int bits = 8; };
template <> struct CodecTraits<kCodecU8bit>    { static constexpr bool stats = true;  static constexpr int bits = 8; };
template <> struct CodecTraits<kCodecSign>     { static constexpr bool stats = false; static constexpr int bits = 1; };
template <> struct CodecTraits<kCodecEFSign>   { static constexpr bool stats = true;  static constexpr int bits = 1; };
template <> struct CodecTraits<kCodecOneBit>   { static constexpr bool stats = true;  static constexpr int bits = 1; };
template <> struct CodecTraits<kCodecFP16>     { static constexpr bool stats = false; static constexpr int bits = 16; };
template <> struct CodecTraits<kCodecFP32>     { static constexpr bool stats = false; static constexpr int bits = 32; };
// QSGD with any bucket size (a multiple of 4) and up to 32767 levels: int16 codes, one norm per bucket of each tensor.
// A pass of its own computes the bucket norms before the encode pass; decode goes through the generic path.
template <> struct CodecTraits<kCodecQSGDX>    { static constexpr bool stats = false; static constexpr int bits = 16; };

__host__ __device__ inline size_t scalars_bytes(int nseg) { return ((size_t)nseg * 16 + 127) / 128 * 128; }
__host__ __device__ inline size_t codes_bytes(int bits, long long total) { return (size_t)total * bits / 8; }

__host__ __device__ inline size_t region1_bytes(int codec, int bits, long long total, int nseg, long long nbuckets = 0) {
  size_t b = kHeaderBytes + scalars_bytes(nseg) + codes_bytes(bits, total);
  if (codec == kCodecQSGD) b += (size_t)(total / 128) * 4;
  if (codec == kCodecQSGDX) b += (size_t)((nbuckets + 3) / 4 * 4) * 4;
  return (b + 255) / 256 * 256;
}

struct SegScalars { float s0, s1, s2, s3; };

// Turn the reduced statistics of a segment into the scalars that travel.
template <int C>
__device__ __forceinline__ SegScalars make_scalars(const QuantSegStats& st, int numel) {
  SegScalars r{0.f, 0.f, 0.f, 0.f};
  const float maxabs = __uint_as_float(st.maxabs_bits);
  if (C == kCodecTernGrad) {
    const double mean = st.sum / numel;
    double var = st.sumsq / numel - mean * mean;
    if (var < 0) var = 0;
    const float c = 2.5f * (float)sqrt(var);
    r.s0 = fminf(maxabs, c);  // max |clamp(x, -c, c)|
    r.s1 = c;
  } else if (C == kCodecU8bit) {
    r.s0 = maxabs;
  } else if (C == kCodecEFSign) {
    r.s0 = (float)(st.sumsq / numel);  // sumsq slot carries sum |x| for this codec
  } else if (C == kCodecOneBit) {
    const unsigned long long nneg = st.cnt_neg;
    const unsigned long long npos = (unsigned long long)numel - nneg;
    r.s0 = nneg ? (float)(st.sum_neg / (double)nneg) : 0.f;
    r.s1 = npos ? (float)(st.sum_pos / (double)npos) : 0.f;
  }
  return r;
}

__device__ __forceinline__ int u8_bin(float y, const float* __restrict__ edges) {
  // largest i in [0,126] with edges[i] <= y (0 when y is below the first edge)
  int lo = 0, hi = 127;  // invariant: answer in [lo, hi)
#pragma unroll
  for (int it = 0; it < 7; ++it) {
    const int mid = (lo + hi) >> 1;
    if (edges[mid] <= y) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float natural_decode(unsigned code) {
  const unsigned c7 = code & 0x7fu;
  const unsigned bits = c7 ? ((c7 + 17u) << 23) : 0u;
  return __uint_as_float(bits | ((code & 0x80u) << 24));
}

// kPush selects the push transport of the all-gather mode: every store of the encode pass goes through the
// NVSwitch multicast mapping (multimem.st) into region `rank` of ALL GPUs' receive areas, and the decode pass
// reads local memory.  It is a separate instantiation, so the pull variant keeps its code and registers.
template <int C, bool kPush>
__global__ void __launch_bounds__(kBlock, 2) quant_exchange_kernel(const QuantArgs a) {
  using T = CodecTraits<C>;
  __shared__ double red_d[kWarps][4];
  __shared__ unsigned long long red_c[kWarps];
  __shared__ float red_m[kWarps];
  __shared__ float s_edges[128];
  __shared__ SegScalars s_peer[kMaxWorld];
  extern __shared__ __align__(16) unsigned char s_dyn[];   // staging areas of the staged decode (kStageBytes, or nothing)

  const Status status{a.status};
  GridBarrier bar{a.barrier, 0u, a.peers.timeout_ns, status};
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = a.peers.rank, world = a.peers.world;
  char* const my_heap = a.peers.heap[rank];
  char* const my_slot = my_heap + a.peers.slot_off;
  // where rank p's payload is read from: its own slot over NVLink (pull), or the local receive area (push)
  auto slot_of = [&](int p) -> const char* {
    return kPush ? a.recv_local + (size_t)p * a.recv_stride : a.peers.heap[p] + a.peers.slot_off;
  };
  // stores of the encode pass: into the local slot (pull), or replicated by the switch into every GPU (push)
  char* const put_base = kPush ? a.recv_mc + (size_t)rank * a.recv_stride : my_slot;
  auto put_u32 = [&](size_t off, unsigned w) {
    if (!GRACE_IN_RANGE(status, kKernelQuant, off + 3, a.peers.slot_bytes)) return;
    if (kPush) asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(put_base + off), "r"(w) : "memory");
    else *reinterpret_cast<unsigned*>(put_base + off) = w;
  };
  auto put_f32 = [&](size_t off, float f) {
    if (!GRACE_IN_RANGE(status, kKernelQuant, off + 3, a.peers.slot_bytes)) return;
    if (kPush) asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(put_base + off), "f"(f) : "memory");
    else *reinterpret_cast<float*>(put_base + off) = f;
  };
  auto put_u2 = [&](size_t off, uint2 w) {
    if (!GRACE_IN_RANGE(status, kKernelQuant, off + 7, a.peers.slot_bytes)) return;
    if (kPush) {
      const unsigned long long q = ((unsigned long long)w.y << 32) | w.x;
      asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(put_base + off), "l"(q) : "memory");
    } else {
      *reinterpret_cast<uint2*>(put_base + off) = w;
    }
  };
  auto put_f4 = [&](size_t off, float4 v) {
    if (!GRACE_IN_RANGE(status, kKernelQuant, off + 15, a.peers.slot_bytes)) return;
    if (kPush) asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(put_base + off), "f"(v.x),
                            "f"(v.y), "f"(v.z), "f"(v.w)
                            : "memory");
    else *reinterpret_cast<float4*>(put_base + off) = v;
  };
  const size_t off_codes = kHeaderBytes + scalars_bytes(a.nseg);
  const size_t off_norms = off_codes + codes_bytes(T::bits, a.total);

  long long chunk = (a.total + gridDim.x - 1) / gridDim.x;
  chunk = (chunk + kIterElems - 1) / kIterElems * kIterElems;
  const long long lo = (long long)blockIdx.x * chunk;
  const long long hi = lo + chunk < a.total ? lo + chunk : a.total;
  if (C == kCodecU8bit) {
    if (tid < 128) s_edges[tid] = c_u8_edges[tid];
    __syncthreads();
  }

  if (a.phases & kPhaseCompress) {
    // The slot of this parity was last used by sequence seq-2: every CTA waits (on local memory) until all peers
    // have acknowledged reading it, and only then may any of its threads store into the slot or push to the peers.
    if (tid < world && tid != rank && a.peers.seq > 2) {
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ack_off) + tid;
      wait_flag_ge(ack, a.peers.seq - 2, a.peers.timeout_ns, status, kTimeoutPeerAck, tid);
    }
    __syncthreads();
    bool ok = !status.failed();
    if (T::stats) {
      // ---- pass S: compensate, store, per-segment statistics ----
      if (ok && lo < hi) {
        for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
          double t_sum = 0, t_sq = 0, t_neg = 0, t_pos = 0;
          unsigned long long t_cnt = 0;
          float t_max = 0.f;
          for (long long i = b0 + 4ll * tid; i < e0; i += kIterElems) {
            const int valid = (e0 - i) >= 4 ? 4 : (int)(e0 - i);
            float gv[4], rv[4] = {0.f, 0.f, 0.f, 0.f}, av[4];
            load4g(a.g, a.g_dtype, i, valid, gv);
            if (a.acc && a.beta != 0.f) load4(a.acc, i, valid, rv);
#pragma unroll
            for (int j = 0; j < 4; ++j) av[j] = a.beta * rv[j] + a.gamma * gv[j];
            if (a.acc) store4(a.acc, i, valid, av);
            float l_sum = 0.f, l_sq = 0.f, l_neg = 0.f, l_pos = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j >= valid) continue;
              const float x = av[j];
              t_max = fmaxf(t_max, fabsf(x));
              if (C == kCodecTernGrad) { l_sum += x; l_sq += x * x; }
              if (C == kCodecEFSign) l_sq += fabsf(x);
              if (C == kCodecOneBit) { if (x < 0.f) { l_neg += x; ++t_cnt; } else l_pos += x; }
            }
            t_sum += l_sum; t_sq += l_sq; t_neg += l_neg; t_pos += l_pos;
          }
          // CTA reduction, one global atomic per quantity
          t_sum = warp_sum(t_sum); t_sq = warp_sum(t_sq); t_neg = warp_sum(t_neg); t_pos = warp_sum(t_pos);
          t_max = warp_max(t_max);
          int cnt_i = warp_sum((int)t_cnt);
          if (lane == 0) {
            red_d[warp][0] = t_sum; red_d[warp][1] = t_sq; red_d[warp][2] = t_neg; red_d[warp][3] = t_pos;
            red_c[warp] = (unsigned long long)cnt_i; red_m[warp] = t_max;
          }
          __syncthreads();
          if (tid == 0) {
            double q0 = 0, q1 = 0, q2 = 0, q3 = 0; unsigned long long c = 0; float m = 0.f;
            for (int w = 0; w < kWarps; ++w) {
              q0 += red_d[w][0]; q1 += red_d[w][1]; q2 += red_d[w][2]; q3 += red_d[w][3];
              c += red_c[w]; m = fmaxf(m, red_m[w]);
            }
            QuantSegStats* st = a.stats + s;
            if (C == kCodecTernGrad) atomicAdd(&st->sum, q0);
            if (C == kCodecTernGrad || C == kCodecEFSign) atomicAdd(&st->sumsq, q1);
            if (C == kCodecOneBit) { atomicAdd(&st->sum_neg, q2); atomicAdd(&st->sum_pos, q3); atomicAdd(&st->cnt_neg, c); }
            if (C == kCodecTernGrad || C == kCodecU8bit) atomicMax(&st->maxabs_bits, __float_as_uint(m));
          }
          __syncthreads();
        });
      }
      ok = bar.sync();
    }

    if (C == kCodecQSGDX && ok) {
      // ---- pass N (general QSGD): one warp per bucket of `qsgd_bucket` consecutive elements of a tensor (the last
      //      bucket of a tensor may be shorter): L2 norm of the compensated values, in a fixed order ----
      const long long nb = a.qsgd_nbuckets;
      const long long gw = (long long)blockIdx.x * kWarps + warp, nw = (long long)gridDim.x * kWarps;
      for (long long b = gw; b < nb; b += nw) {
        int lo_s = 0, hi_s = a.nseg;            // segment whose first bucket (Segment::k) is the last one <= b
        while (lo_s + 1 < hi_s) {
          const int mid = (lo_s + hi_s) >> 1;
          if ((long long)a.segs[mid].k <= b) lo_s = mid; else hi_s = mid;
        }
        const Segment sg = a.segs[lo_s];
        const long long e_begin = sg.offset + (b - sg.k) * a.qsgd_bucket;
        long long e_end = e_begin + a.qsgd_bucket;
        if (e_end > sg.offset + sg.numel) e_end = sg.offset + sg.numel;
        float sq = 0.f;
        for (long long i = e_begin + 4ll * lane; i < e_end; i += 128) {
          const int valid = (e_end - i) >= 4 ? 4 : (int)(e_end - i);
          float gv[4], rv[4] = {0.f, 0.f, 0.f, 0.f};
          load4g(a.g, a.g_dtype, i, valid, gv);
          if (a.acc && a.beta != 0.f) load4(a.acc, i, valid, rv);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x = a.beta * rv[j] + a.gamma * gv[j];
            sq += x * x;
          }
        }
        sq = warp_sum(sq);
        if (lane == 0) *reinterpret_cast<float*>(my_slot + off_norms + (size_t)b * 4) = sqrtf(sq);
      }
      ok = bar.sync();
    }

    // ---- pass E: encode into the send slot, write the residual ----
    if (ok && lo < hi) {
      const void* __restrict__ src = (T::stats && a.acc) ? (const void*)a.acc : a.g;
      const int src_dtype = (T::stats && a.acc) ? (int)kGradF32 : a.g_dtype;
      for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
        SegScalars sc{0.f, 0.f, 0.f, 0.f};
        if (T::stats) {
          sc = make_scalars<C>(a.stats[s], a.segs[s].numel);
          if (b0 == a.segs[s].offset && tid == 0)
            put_f4(kHeaderBytes + (size_t)s * 16, make_float4(sc.s0, sc.s1, sc.s2, sc.s3));
        }
        // b0 is a multiple of 128: every warp step covers one whole code group
        for (long long gb0 = b0 + 128ll * warp; gb0 < e0; gb0 += 128ll * kWarps * kU) {
          // prefetch: all loads of kU groups are issued before the first encode
          float pav[kU][4];
          int pvalid[kU];
#pragma unroll
          for (int q = 0; q < kU; ++q) {
            const long long pi = gb0 + 128ll * kWarps * q + 4 * lane;
            pvalid[q] = pi < e0 ? ((e0 - pi) >= 4 ? 4 : (int)(e0 - pi)) : 0;
            float gv[4] = {0.f, 0.f, 0.f, 0.f}, rv[4] = {0.f, 0.f, 0.f, 0.f};
            if (pvalid[q]) {
              if (T::stats) {
                load4g(src, src_dtype, pi, pvalid[q], gv);
              } else {
                load4g(a.g, a.g_dtype, pi, pvalid[q], gv);
                if (a.acc && a.beta != 0.f) load4(a.acc, pi, pvalid[q], rv);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) pav[q][j] = T::stats ? gv[j] : a.beta * rv[j] + a.gamma * gv[j];
          }
#pragma unroll
          for (int q = 0; q < kU; ++q) {
          const long long gb = gb0 + 128ll * kWarps * q;
          if (gb >= e0) break;  // warp-uniform
          const long long i = gb + 4 * lane;
          const int valid = pvalid[q];
          float av[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) av[j] = pav[q][j];
          float xv[4];  // what is encoded (momentum for signum, else acc)
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[j] = av[j];
          if (C == kCodecSign && a.mom) {
            float mv[4] = {0.f, 0.f, 0.f, 0.f};
            if (valid && !a.first_step) load4(a.mom, i, valid, mv);
#pragma unroll
            for (int j = 0; j < 4; ++j) xv[j] = a.first_step ? av[j] : (1.f - a.mom_beta) * av[j] + a.mom_beta * mv[j];
            if (valid) store4(a.mom, i, valid, xv);
          }
          float dv[4] = {0.f, 0.f, 0.f, 0.f};  // decode(code) for the residual
          const size_t group = (size_t)(gb >> 7);
          Philox4 rnd{0u, 0u, 0u, 0u};
          if (C == kCodecQSGD || C == kCodecQSGDX || C == kCodecTernGrad || (C == kCodecNatural && !a.deterministic))
            rnd = philox_group((uint64_t)(i >> 2), a.step, 0u, a.seed);
          const unsigned rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};

          if (C == kCodecQSGD) {
            float sq = xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3];
            sq = warp_sum(sq);
            const float norm = sqrtf(sq);
            const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
            const float dq = norm / (float)a.quantum;
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lf = qn * fabsf(xv[j]);
              const float fl = floorf(lf);
              float level = fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f);
              level = fminf(level, 127.f);
              const int code = xv[j] < 0.f ? -(int)level : (int)level;
              word |= ((unsigned)code & 0xffu) << (8 * j);
              dv[j] = dq * (float)code;
            }
            put_u32(off_codes + (size_t)i, word);
            if (lane == 0) {
              // one scalar per 128 elements: as single 4-byte multicast stores these cost more than all the codes,
              // so in push mode they go to the local slot and are replicated in one vectorised sweep afterwards
              if (kPush) *reinterpret_cast<float*>(my_slot + off_norms + group * 4) = norm;
              else put_f32(off_norms + group * 4, norm);
            }
          } else if (C == kCodecQSGDX) {
            // the lane's four elements lie in one bucket (bucket sizes are multiples of 4)
            const long long bucket = a.segs[s].k + (i - a.segs[s].offset) / a.qsgd_bucket;
            const float norm = valid ? __ldcg(reinterpret_cast<const float*>(my_slot + off_norms) + bucket) : 0.f;
            const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
            const float dq = norm / (float)a.quantum;
            int codes[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lf = qn * fabsf(xv[j]);
              const float fl = floorf(lf);
              float level = fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f);
              level = fminf(level, 32767.f);
              codes[j] = xv[j] < 0.f ? -(int)level : (int)level;
              dv[j] = dq * (float)codes[j];
            }
            uint2 w;
            w.x = ((unsigned)codes[0] & 0xffffu) | ((unsigned)codes[1] << 16);
            w.y = ((unsigned)codes[2] & 0xffffu) | ((unsigned)codes[3] << 16);
            put_u2(off_codes + (size_t)i * 2, w);
          } else if (C == kCodecNatural) {
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const unsigned bits = __float_as_uint(xv[j]);
              const unsigned biased = (bits >> 23) & 0xffu;
              const unsigned mant = bits & 0x7fffffu;
              bool up;
              if (a.deterministic) up = mant > 0x400000u;
              else up = u01(rw[j]) < (float)mant * 1.1920928955078125e-07f;
              int b = (int)biased + (up ? 1 : 0);
              int c7 = b - 17;
              c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
              if (biased == 0) c7 = 0;
              const unsigned code = (unsigned)c7 | ((bits >> 24) & 0x80u);
              word |= code << (8 * j);
              dv[j] = natural_decode(code);
            }
            put_u32(off_codes + (size_t)i, word);
          } else if (C == kCodecU8bit) {
            const float s0 = sc.s0;
            const float safe = s0 > 0.f ? s0 : 1.f;
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float y = fabsf(xv[j]) / safe;
              const int bin = u8_bin(y, s_edges);
              const int sg = xv[j] > 0.f ? 1 : (xv[j] < 0.f ? -1 : 0);
              const int code = bin * sg;
              word |= ((unsigned)code & 0xffu) << (8 * j);
              dv[j] = code ? s_edges[bin] * s0 * (float)sg : 0.f;  // bin 0 decodes to exactly 0
            }
            put_u32(off_codes + (size_t)i, word);
          } else if (C == kCodecTernGrad) {
            const float s0 = sc.s0, c = sc.s1;
            unsigned nz[4], ng[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float mag = fminf(fabsf(xv[j]), c);
              const bool keep = (j < valid) && (u01(rw[j]) * s0 < mag);
              const bool neg = xv[j] < 0.f;
              nz[j] = __ballot_sync(0xffffffffu, keep);
              ng[j] = __ballot_sync(0xffffffffu, keep && neg);
              dv[j] = keep ? (neg ? -s0 : s0) : 0.f;
            }
            if (lane < 8) {
              const unsigned w = lane < 4 ? nz[lane & 3] : ng[lane & 3];
              put_u32(off_codes + group * 32 + lane * 4, w);
            }
          } else if (C == kCodecSign || C == kCodecEFSign || C == kCodecOneBit) {
            unsigned bw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // bit = 1 means "non-negative" (sign codecs) / "negative" (1-bit SGD)
              const bool bit = C == kCodecOneBit ? (xv[j] < 0.f) : (xv[j] >= 0.f);
              bw[j] = __ballot_sync(0xffffffffu, bit && j < valid);
              if (C == kCodecSign) dv[j] = bit ? 1.f : -1.f;
              if (C == kCodecEFSign) dv[j] = bit ? sc.s0 : -sc.s0;
              if (C == kCodecOneBit) dv[j] = bit ? sc.s0 : sc.s1;
            }
            if (lane < 4) put_u32(off_codes + group * 16 + lane * 4, bw[lane]);
          } else if (C == kCodecFP16) {
            __half2 h01 = __floats2half2_rn(xv[0], xv[1]);
            __half2 h23 = __floats2half2_rn(xv[2], xv[3]);
            uint2 w;
            w.x = *reinterpret_cast<unsigned*>(&h01);
            w.y = *reinterpret_cast<unsigned*>(&h23);
            put_u2(off_codes + (size_t)i * 2, w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            dv[0] = f01.x; dv[1] = f01.y; dv[2] = f23.x; dv[3] = f23.y;
          } else if (C == kCodecFP32) {
            put_f4(off_codes + (size_t)i * 4, make_float4(xv[0], xv[1], xv[2], xv[3]));
#pragma unroll
            for (int j = 0; j < 4; ++j) dv[j] = xv[j];
          }
          if (a.acc && valid) {
            float res[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) res[j] = av[j] - dv[j];
            store4(a.acc, i, valid, res);
          }
          }
        }
      });
    }
    if (kPush) __threadfence_system();   // the multicast stores precede the flag raised after this barrier
    ok = bar.sync();
    if (kPush && C == kCodecQSGD) {
      // replicate the norm array (total / 128 floats, complete after the barrier above), 16 bytes per store
      const size_t n16 = ((size_t)(a.total / 128) * 4 + 15) / 16;
      const uint4* nsrc = reinterpret_cast<const uint4*>(my_slot + off_norms);
      const size_t gt = (size_t)blockIdx.x * kBlock + tid, gs = (size_t)gridDim.x * kBlock;
      if (ok)
        for (size_t k = gt; k < n16; k += gs) {
          const uint4 v = ld_cg_u4(nsrc + k);
          put_f4(off_norms + k * 16, make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z),
                                                 __uint_as_float(v.w)));
        }
      __threadfence_system();
      ok = bar.sync();
    }
    if (T::stats && ok) {
      // leave the statistics scratch zeroed for the next launch
      for (int s = blockIdx.x * kBlock + tid; s < a.nseg; s += gridDim.x * kBlock) {
        QuantSegStats z{};
        a.stats[s] = z;
      }
    }
  }

  if (a.phases & kPhasePublish) {
    if (blockIdx.x == 0) {
      __syncthreads();
      if (tid < world && !status.failed()) {
        __threadfence_system();
        uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ready_off) + rank;
        st_release_sys(flag, a.peers.seq);
      }
    }
  }

  constexpr bool kTwoPhaseCodec = C == kCodecQSGD || C == kCodecNatural || C == kCodecFP16 || C == kCodecFP32;
  if (kTwoPhaseCodec && !kPush && a.alltoall) {
    // ---- two-phase mode: compressed reduce-scatter, re-encode, compressed all-gather ----
    // Rank j owns the contiguous chunk j of 128-element groups.  Region 2 of every
    // slot holds that rank's re-encoded chunk: codes, then (QSGD) one norm per group.
    const long long groups_total = a.total >> 7;
    const long long chunk_groups = (groups_total + world - 1) / world;
    const size_t off2_codes = region1_bytes(C, T::bits, a.total, a.nseg);
    const size_t off2_norms = off2_codes + codes_bytes(T::bits, chunk_groups * 128);
    __shared__ int s_ready2;
    if (a.phases & kPhaseReduce) {
      if (tid == 0) s_ready2 = 1;
      __syncthreads();
      if (tid < world) {
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + tid;
        if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) s_ready2 = 0;
      }
      __syncthreads();
      const long long g_begin = chunk_groups * rank;
      const long long g_end = g_begin + chunk_groups < groups_total ? g_begin + chunk_groups : groups_total;
      if (s_ready2 && T::bits == 8 && world <= kStagePeers) {
        // 8-bit codes: a warp trip covers 512 elements (four groups); lane l fetches its 16 code bytes from EVERY
        // rank (one 512-byte request per rank and warp, all in flight together) and parks them in the warp's staging
        // area; the sum is formed rank by rank, re-encoded with the chunk's own random stream and written as one
        // 16-byte store per lane.
        uint4* const st_codes = reinterpret_cast<uint4*>(s_dyn + warp * kStageWarpBytes);
        float* const st_norms = reinterpret_cast<float*>(s_dyn + warp * kStageWarpBytes + kStagePeers * 512);
        const long long e_begin = g_begin << 7, e_end = g_end << 7;
        for (long long w0 = e_begin + 512ll * ((long long)blockIdx.x * kWarps + warp); w0 < e_end;
             w0 += 512ll * gridDim.x * kWarps) {
          const long long i = w0 + 16ll * lane;     // this lane's 16 elements (inside one group)
          const bool have = i < e_end;
          {
            uint4 v[kStagePeers];
            float nv[kStagePeers];
#pragma unroll
            for (int p = 0; p < kStagePeers; ++p) {
              v[p] = make_uint4(0u, 0u, 0u, 0u);
              nv[p] = 0.f;
              if (p < world) {
                const char* slot = a.peers.heap[p] + a.peers.slot_off;
                if (have) v[p] = ld_cg_u4(slot + off_codes + (size_t)i);
                if (C == kCodecQSGD && lane < 4 && w0 + 128ll * lane < e_end)
                  nv[p] = ld_cg_f32(slot + off_norms + (size_t)((w0 >> 7) + lane) * 4);
              }
            }
            __syncwarp();
#pragma unroll
            for (int p = 0; p < kStagePeers; ++p) {
              if (p < world) {
                st_codes[p * 32 + lane] = v[p];
                if (C == kCodecQSGD && lane < 4) st_norms[p * 4 + lane] = nv[p];
              }
            }
            __syncwarp();
          }
          float xs[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) xs[j] = 0.f;
          for (int p = 0; p < world; ++p) {
            const uint4 cw = st_codes[p * 32 + lane];
            const unsigned words[4] = {cw.x, cw.y, cw.z, cw.w};
            const float d = C == kCodecQSGD ? st_norms[p * 4 + (lane >> 3)] / (float)a.quantum : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const unsigned byte = (words[j >> 2] >> (8 * (j & 3))) & 0xffu;
              if (C == kCodecQSGD) xs[j] += d * (float)(int)(signed char)byte;
              else xs[j] += natural_decode(byte);
            }
          }
          // re-encode the reduced values (a second lossy step, with its own random stream: counter = element / 4)
          unsigned out_words[4] = {0u, 0u, 0u, 0u};
          float sq = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) sq += xs[j] * xs[j];
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);     // the eight lanes of a group
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          const float norm = sqrtf(sq);
          const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            Philox4 rnd{0u, 0u, 0u, 0u};
            if (C == kCodecQSGD || !a.deterministic) rnd = philox_group((uint64_t)((i >> 2) + q4), a.step, 1u, a.seed);
            const unsigned rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x = xs[4 * q4 + j];
              unsigned code;
              if (C == kCodecQSGD) {
                const float lf = qn * fabsf(x);
                const float fl = floorf(lf);
                const float level = fminf(fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f), 127.f);
                code = (unsigned)(x < 0.f ? -(int)level : (int)level) & 0xffu;
              } else {
                const unsigned bits = __float_as_uint(x);
                const unsigned biased = (bits >> 23) & 0xffu;
                const unsigned mant = bits & 0x7fffffu;
                const bool up = a.deterministic ? mant > 0x400000u : u01(rw[j]) < (float)mant * 1.1920928955078125e-07f;
                int c7 = (int)biased + (up ? 1 : 0) - 17;
                c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
                if (biased == 0) c7 = 0;
                code = (unsigned)c7 | ((bits >> 24) & 0x80u);
              }
              out_words[q4] |= code << (8 * j);
            }
          }
          if (have) {
            const size_t li = (size_t)(i - e_begin);      // element index inside my chunk
            *reinterpret_cast<uint4*>(my_slot + off2_codes + li) = make_uint4(out_words[0], out_words[1], out_words[2], out_words[3]);
            if (C == kCodecQSGD && (lane & 7) == 0) *reinterpret_cast<float*>(my_slot + off2_norms + (li >> 7) * 4) = norm;
          }
        }
      } else
      if (s_ready2) {
        const long long wstride = (long long)gridDim.x * kWarps;
        for (long long grp0 = g_begin + (long long)blockIdx.x * kWarps + warp; grp0 < g_end; grp0 += wstride * kU) {
          // kU groups per warp trip; per peer, the kU loads are issued before they are consumed
          float xs[kU][4];
#pragma unroll
          for (int q = 0; q < kU; ++q)
#pragma unroll
            for (int j = 0; j < 4; ++j) xs[q][j] = 0.f;
          for (int p = 0; p < world; ++p) {
            const char* slot = a.peers.heap[p] + a.peers.slot_off;
            uint4 w4[kU];
            float dqs[kU];
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              const long long grp = grp0 + wstride * q;
              const long long i = (grp << 7) + 4 * lane;
              w4[q] = make_uint4(0u, 0u, 0u, 0u);
              dqs[q] = 0.f;
              if (grp >= g_end) continue;
              if (T::bits == 8) {
                w4[q].x = ld_cg_u32(slot + off_codes + (size_t)i);
                if (C == kCodecQSGD) dqs[q] = ld_cg_f32(slot + off_norms + (size_t)grp * 4);
              } else if (T::bits == 32) {
                w4[q] = ld_cg_u4(slot + off_codes + (size_t)i * 4);
              } else {
                const char* q16 = slot + off_codes + (size_t)i * 2;
                asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(w4[q].x), "=r"(w4[q].y) : "l"(q16));
              }
            }
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              if (T::bits == 8) {
                const float d = dqs[q] / (float)a.quantum;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned byte = (w4[q].x >> (8 * j)) & 0xffu;
                  if (C == kCodecQSGD) xs[q][j] += d * (float)(int)(signed char)byte;
                  else xs[q][j] += natural_decode(byte);
                }
              } else if (T::bits == 32) {
                xs[q][0] += __uint_as_float(w4[q].x); xs[q][1] += __uint_as_float(w4[q].y);
                xs[q][2] += __uint_as_float(w4[q].z); xs[q][3] += __uint_as_float(w4[q].w);
              } else {
                const float2 f01 = __half22float2(*reinterpret_cast<__half2*>(&w4[q].x));
                const float2 f23 = __half22float2(*reinterpret_cast<__half2*>(&w4[q].y));
                xs[q][0] += f01.x; xs[q][1] += f01.y; xs[q][2] += f23.x; xs[q][3] += f23.y;
              }
            }
          }
#pragma unroll
          for (int q = 0; q < kU; ++q) {
          const long long grp = grp0 + wstride * q;
          if (grp >= g_end) break;  // warp-uniform
          const long long i = (grp << 7) + 4 * lane;
          float xv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) xv[j] = xs[q][j];
          // re-encode the reduced group (a second lossy step, with its own random stream)
          const size_t li = (size_t)((grp - g_begin) << 7) + 4 * lane;   // element index inside my chunk
          if (C == kCodecQSGD) {
            const Philox4 rnd = philox_group((uint64_t)(i >> 2), a.step, 1u, a.seed);
            const unsigned rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
            float sq = warp_sum(xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3]);
            const float norm = sqrtf(sq);
            const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lf = qn * fabsf(xv[j]);
              const float fl = floorf(lf);
              const float level = fminf(fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f), 127.f);
              const int code = xv[j] < 0.f ? -(int)level : (int)level;
              word |= ((unsigned)code & 0xffu) << (8 * j);
            }
            *reinterpret_cast<unsigned*>(my_slot + off2_codes + li) = word;
            if (lane == 0) *reinterpret_cast<float*>(my_slot + off2_norms + (size_t)(grp - g_begin) * 4) = norm;
          } else if (C == kCodecNatural) {
            const Philox4 rnd = philox_group((uint64_t)(i >> 2), a.step, 1u, a.seed);
            const unsigned rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
            unsigned word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const unsigned bits = __float_as_uint(xv[j]);
              const unsigned biased = (bits >> 23) & 0xffu;
              const unsigned mant = bits & 0x7fffffu;
              const bool up = a.deterministic ? mant > 0x400000u : u01(rw[j]) < (float)mant * 1.1920928955078125e-07f;
              int c7 = (int)biased + (up ? 1 : 0) - 17;
              c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
              if (biased == 0) c7 = 0;
              word |= ((unsigned)c7 | ((bits >> 24) & 0x80u)) << (8 * j);
            }
            *reinterpret_cast<unsigned*>(my_slot + off2_codes + li) = word;
          } else if (C == kCodecFP32) {
            *reinterpret_cast<float4*>(my_slot + off2_codes + li * 4) = make_float4(xv[0], xv[1], xv[2], xv[3]);
          } else {
            __half2 h01 = __floats2half2_rn(xv[0], xv[1]);
            __half2 h23 = __floats2half2_rn(xv[2], xv[3]);
            uint2 w;
            w.x = *reinterpret_cast<unsigned*>(&h01);
            w.y = *reinterpret_cast<unsigned*>(&h23);
            *reinterpret_cast<uint2*>(my_slot + off2_codes + li * 2) = w;
          }
          }
        }
      }
      bar.sync();
      if (blockIdx.x == 0 && tid < world && !status.failed()) {
        __threadfence_system();
        uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.ready2_off) + rank;
        st_release_sys(flag, a.peers.seq);
      }
    }
    if (a.phases & kPhaseExchange) {
      if (tid == 0) s_ready2 = 1;
      __syncthreads();
      if (tid < world) {
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.ready2_off) + tid;
        if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) s_ready2 = 0;
      }
      __syncthreads();
      if (s_ready2 && lo < hi && T::bits == 8) {
        // 8-bit codes: every lane fetches 16 codes (and its group's norm) from the rank that owns the group; two
        // such 512-byte requests per warp are in flight before the first is decoded
        constexpr int kX = 2;
        for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
          for (long long w0 = b0 + 512ll * warp; w0 < e0; w0 += 512ll * kWarps * kX) {
            uint4 cw[kX];
            float dq[kX];
#pragma unroll
            for (int q = 0; q < kX; ++q) {
              const long long i = w0 + 512ll * kWarps * q + 16 * lane;
              cw[q] = make_uint4(0u, 0u, 0u, 0u);
              dq[q] = 0.f;
              if (i < e0) {
                const long long grp = i >> 7;
                const int owner = (int)(grp / chunk_groups);
                const long long lg = grp - (long long)owner * chunk_groups;
                const char* slot = a.peers.heap[owner] + a.peers.slot_off;
                cw[q] = ld_cg_u4(slot + off2_codes + (size_t)(lg << 7) + (size_t)(i & 127));
                if (C == kCodecQSGD) dq[q] = ld_cg_f32(slot + off2_norms + (size_t)lg * 4);
              }
            }
#pragma unroll
            for (int q = 0; q < kX; ++q) {
              const long long i = w0 + 512ll * kWarps * q + 16 * lane;
              const unsigned words[4] = {cw[q].x, cw[q].y, cw[q].z, cw[q].w};
              const float d = dq[q] / (float)a.quantum;
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                const long long iv = i + 4 * v4;
                if (iv >= e0) continue;
                const int valid = (e0 - iv) >= 4 ? 4 : (int)(e0 - iv);
                float ov[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned byte = (words[v4] >> (8 * j)) & 0xffu;
                  ov[j] = (C == kCodecQSGD ? d * (float)(int)(signed char)byte : natural_decode(byte)) * a.scale;
                }
                store4g(a.out, a.g_dtype, iv, valid, ov);
              }
            }
          }
        });
      } else
      if (s_ready2 && lo < hi) {
        for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
          for (long long gb0 = b0 + 128ll * warp; gb0 < e0; gb0 += 128ll * kWarps * kU) {
            uint4 w4[kU];
            float dqs[kU];
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              const long long gb = gb0 + 128ll * kWarps * q;
              w4[q] = make_uint4(0u, 0u, 0u, 0u);
              dqs[q] = 0.f;
              if (gb >= e0) continue;
              const long long grp = gb >> 7;
              const int owner = (int)(grp / chunk_groups);
              const long long lg = grp - (long long)owner * chunk_groups;
              const size_t li = (size_t)(lg << 7) + 4 * lane;
              const char* slot = a.peers.heap[owner] + a.peers.slot_off;
              if (T::bits == 8) {
                w4[q].x = ld_cg_u32(slot + off2_codes + li);
                if (C == kCodecQSGD) dqs[q] = ld_cg_f32(slot + off2_norms + (size_t)lg * 4);
              } else if (T::bits == 32) {
                w4[q] = ld_cg_u4(slot + off2_codes + li * 4);
              } else {
                const char* q16 = slot + off2_codes + li * 2;
                asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(w4[q].x), "=r"(w4[q].y) : "l"(q16));
              }
            }
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              const long long gb = gb0 + 128ll * kWarps * q;
              if (gb >= e0) break;  // warp-uniform
              const long long i = gb + 4 * lane;
              int valid = 0;
              if (i < e0) valid = (e0 - i) >= 4 ? 4 : (int)(e0 - i);
              float ov[4];
              if (T::bits == 8) {
                const float d = dqs[q] / (float)a.quantum;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned byte = (w4[q].x >> (8 * j)) & 0xffu;
                  ov[j] = (C == kCodecQSGD ? d * (float)(int)(signed char)byte : natural_decode(byte)) * a.scale;
                }
              } else if (T::bits == 32) {
                ov[0] = __uint_as_float(w4[q].x) * a.scale; ov[1] = __uint_as_float(w4[q].y) * a.scale;
                ov[2] = __uint_as_float(w4[q].z) * a.scale; ov[3] = __uint_as_float(w4[q].w) * a.scale;
              } else {
                const float2 f01 = __half22float2(*reinterpret_cast<__half2*>(&w4[q].x));
                const float2 f23 = __half22float2(*reinterpret_cast<__half2*>(&w4[q].y));
                ov[0] = f01.x * a.scale; ov[1] = f01.y * a.scale; ov[2] = f23.x * a.scale; ov[3] = f23.y * a.scale;
              }
              if (valid) store4g(a.out, a.g_dtype, i, valid, ov);
            }
          }
        });
      }
      bar.sync();
      if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
        uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
        st_release_sys(ack, a.peers.seq);
      }
    }
    return;
  }

  if (a.phases & kPhaseExchange) {
    // every CTA polls its own (local) copy of the peers' flags
    __shared__ int s_ready;
    if (tid == 0) s_ready = 1;
    __syncthreads();
    if (tid < world) {
      const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ready_off) + tid;
      if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid)) s_ready = 0;
    }
    __syncthreads();
    if (s_ready && lo < hi) {
      for_each_segment_range(a.segs, a.nseg, lo, hi, [&](int s, long long b0, long long e0) {
        if (T::stats) {
          __syncthreads();
          if (tid < world) {
            const uint4 v = ld_cg_u4(slot_of(tid) + kHeaderBytes + (size_t)s * 16);
            s_peer[tid] = SegScalars{__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
          }
          __syncthreads();
        }
        if ((T::bits == 1 || T::bits == 2 || T::bits == 8) && world > 1 && world <= kStagePeers) {
          // Staged decode.  Per trip a warp covers one block of 512 code bytes per rank: 512 elements of an
          // 8-bit code, 16 groups of a 2-bit code, 32 groups of a 1-bit code.  Lane l fetches bytes
          // [16 l, 16 l + 16) of the block from EVERY rank (one 512-byte request per rank and warp, all of them
          // in flight together), parks them in the warp's staging area and the registers are free again; the
          // sums are then formed rank by rank (0..W-1: identical bits on every GPU) from shared memory.
          constexpr long long kBlockElems = 512ll * 8 / T::bits;
          uint4* const st_codes = reinterpret_cast<uint4*>(s_dyn + warp * kStageWarpBytes);            // [rank][32]
          float* const st_norms = reinterpret_cast<float*>(s_dyn + warp * kStageWarpBytes + kStagePeers * 512);  // [rank][4]
          for (long long w0 = b0 + kBlockElems * warp; w0 < e0; w0 += kBlockElems * kWarps) {
            // ---- fetch: all ranks, then park ----
            {
              // first element covered by this lane's 16 bytes
              const long long le = w0 + (T::bits == 8 ? 16ll * lane : (T::bits == 2 ? 128ll * (lane >> 1) : 128ll * lane));
              const size_t byte_off = T::bits == 8 ? (size_t)le : (size_t)(w0 >> 7) * (T::bits * 16) + 16u * lane;
              const bool have = le < e0;
              uint4 v[kStagePeers];
              float nv[kStagePeers];
#pragma unroll
              for (int p = 0; p < kStagePeers; ++p) {
                v[p] = make_uint4(0u, 0u, 0u, 0u);
                nv[p] = 0.f;
                if (p < world) {
                  const char* slot = slot_of(p);
                  if (have && GRACE_IN_RANGE(status, kKernelQuant, off_codes + byte_off + 15, a.peers.slot_bytes))
                    v[p] = ld_cg_u4(slot + off_codes + byte_off);
                  if (C == kCodecQSGD && lane < 4 && w0 + 128ll * lane < e0)
                    nv[p] = ld_cg_f32(slot + off_norms + (size_t)((w0 >> 7) + lane) * 4);
                }
              }
              __syncwarp();   // the previous trip's readers are done with the staging area
#pragma unroll
              for (int p = 0; p < kStagePeers; ++p) {
                if (p < world) {
                  st_codes[p * 32 + lane] = v[p];
                  if (C == kCodecQSGD && lane < 4) st_norms[p * 4 + lane] = nv[p];
                }
              }
              __syncwarp();
            }
            if (T::bits == 8) {
              float acc16[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) acc16[j] = 0.f;
              for (int p = 0; p < world; ++p) {
                const uint4 cw = st_codes[p * 32 + lane];
                const unsigned words[4] = {cw.x, cw.y, cw.z, cw.w};
                float d = 0.f;
                if (C == kCodecQSGD) d = st_norms[p * 4 + (lane >> 3)] / (float)a.quantum;
                if (C == kCodecU8bit) d = s_peer[p].s0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const unsigned byte = (words[j >> 2] >> (8 * (j & 3))) & 0xffu;
                  if (C == kCodecQSGD) acc16[j] += d * (float)(int)(signed char)byte;
                  if (C == kCodecNatural) acc16[j] += natural_decode(byte);
                  if (C == kCodecU8bit) {
                    const int code = (int)(signed char)byte;
                    const int ab = code < 0 ? -code : code;
                    const float sg = code > 0 ? 1.f : (code < 0 ? -1.f : 0.f);
                    acc16[j] += s_edges[ab] * d * sg;
                  }
                }
              }
              const long long i = w0 + 16ll * lane;
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                const long long iv = i + 4 * v4;
                if (iv >= e0) continue;
                const int valid = (e0 - iv) >= 4 ? 4 : (int)(e0 - iv);
                const float ov[4] = {acc16[4 * v4] * a.scale, acc16[4 * v4 + 1] * a.scale,
                                     acc16[4 * v4 + 2] * a.scale, acc16[4 * v4 + 3] * a.scale};
                store4g(a.out, a.g_dtype, iv, valid, ov);
              }
            } else {
              // bit-packed codes: word j of a group holds, in bit l, the code bit of element 4 l + j
              constexpr int kGroups = T::bits == 2 ? 16 : 32;   // groups per block
              constexpr int kVec = T::bits == 2 ? 2 : 1;        // 16-byte vectors per group and rank
#pragma unroll 1
              for (int r0 = 0; r0 < kGroups; r0 += 8) {
                if (w0 + 128ll * r0 >= e0) break;   // warp-uniform
                float acc[8][4];
                int votes[8][4];
#pragma unroll
                for (int gi = 0; gi < 8; ++gi)
#pragma unroll
                  for (int j = 0; j < 4; ++j) { acc[gi][j] = 0.f; votes[gi][j] = 0; }
                for (int p = 0; p < world; ++p) {
                  const SegScalars sp = s_peer[p];
#pragma unroll
                  for (int gi = 0; gi < 8; ++gi) {
                    const uint4 w = st_codes[p * 32 + (r0 + gi) * kVec];   // same address in every lane: broadcast
                    const unsigned wj[4] = {w.x, w.y, w.z, w.w};
                    unsigned nj[4] = {0u, 0u, 0u, 0u};
                    if (T::bits == 2) {
                      const uint4 n = st_codes[p * 32 + (r0 + gi) * kVec + 1];
                      nj[0] = n.x; nj[1] = n.y; nj[2] = n.z; nj[3] = n.w;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const bool bit = (wj[j] >> lane) & 1u;
                      if (T::bits == 2) {
                        if (bit) acc[gi][j] += ((nj[j] >> lane) & 1u) ? -sp.s0 : sp.s0;
                      } else {
                        if (C == kCodecSign) votes[gi][j] += bit ? 1 : -1;
                        if (C == kCodecEFSign) acc[gi][j] += bit ? sp.s0 : -sp.s0;
                        if (C == kCodecOneBit) acc[gi][j] += bit ? sp.s0 : sp.s1;
                      }
                    }
                  }
                }
#pragma unroll
                for (int gi = 0; gi < 8; ++gi) {
                  const long long gb = w0 + 128ll * (r0 + gi);
                  if (gb >= e0) break;  // warp-uniform
                  const long long i = gb + 4 * lane;
                  int valid = 0;
                  if (i < e0) valid = (e0 - i) >= 4 ? 4 : (int)(e0 - i);
                  float ov[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (C == kCodecSign) ov[j] = votes[gi][j] >= 0 ? 1.f : -1.f;
                    else if (C == kCodecEFSign) ov[j] = acc[gi][j] / a.lr;
                    else ov[j] = acc[gi][j] * a.scale;
                  }
                  if (valid) store4g(a.out, a.g_dtype, i, valid, ov);
                }
              }
            }
          }
        } else
        for (long long gb0 = b0 + 128ll * warp; gb0 < e0; gb0 += 128ll * kWarps * kU) {
          // kU groups per warp trip; for every peer the kU loads are issued before they are consumed
          float sum[kU][4];
          int votes[kU][4];
#pragma unroll
          for (int q = 0; q < kU; ++q)
#pragma unroll
            for (int j = 0; j < 4; ++j) { sum[q][j] = 0.f; votes[q][j] = 0; }
          for (int p = 0; p < world; ++p) {
            const char* slot = slot_of(p);
            unsigned w0[kU], w1[kU];
            float dq[kU];
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              const long long gb = gb0 + 128ll * kWarps * q;
              const long long i = gb + 4 * lane;
              const size_t group = (size_t)(gb >> 7);
              w0[q] = 0; w1[q] = 0; dq[q] = 0.f;
              if (gb >= e0) continue;
              if (T::bits == 8) {
                w0[q] = ld_cg_u32(slot + off_codes + (size_t)i);
                if (C == kCodecQSGD) dq[q] = ld_cg_f32(slot + off_norms + group * 4);
              } else if (T::bits == 2) {
                if (lane < 8) w0[q] = ld_cg_u32(slot + off_codes + group * 32 + lane * 4);
              } else if (T::bits == 1) {
                if (lane < 4) w0[q] = ld_cg_u32(slot + off_codes + group * 16 + lane * 4);
              } else if (T::bits == 16) {
                const char* ptr16 = slot + off_codes + (size_t)i * 2;
                asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(w0[q]), "=r"(w1[q]) : "l"(ptr16));
                if (C == kCodecQSGDX && i < e0)
                  dq[q] = ld_cg_f32(slot + off_norms + (size_t)(a.segs[s].k + (i - a.segs[s].offset) / a.qsgd_bucket) * 4);
              }
            }
#pragma unroll
            for (int q = 0; q < kU; ++q) {
              const long long gb = gb0 + 128ll * kWarps * q;
              if (gb >= e0) continue;  // warp-uniform
              if (T::bits == 8) {
                const float d = dq[q] / (float)a.quantum;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned byte = (w0[q] >> (8 * j)) & 0xffu;
                  if (C == kCodecQSGD) sum[q][j] += d * (float)(int)(signed char)byte;
                  if (C == kCodecNatural) sum[q][j] += natural_decode(byte);
                  if (C == kCodecU8bit) {
                    const int code = (int)(signed char)byte;
                    const int ab = code < 0 ? -code : code;
                    const float sg = code > 0 ? 1.f : (code < 0 ? -1.f : 0.f);
                    sum[q][j] += s_edges[ab] * s_peer[p].s0 * sg;
                  }
                }
              } else if (T::bits == 2) {
                // 8 words per group: 4 "non-zero" ballots then 4 "negative" ballots
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned nz = __shfl_sync(0xffffffffu, w0[q], j);
                  const unsigned ng = __shfl_sync(0xffffffffu, w0[q], 4 + j);
                  const float s0 = s_peer[p].s0;
                  if ((nz >> lane) & 1u) sum[q][j] += ((ng >> lane) & 1u) ? -s0 : s0;
                }
              } else if (T::bits == 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const unsigned bits = __shfl_sync(0xffffffffu, w0[q], j);
                  const bool bit = (bits >> lane) & 1u;
                  if (C == kCodecSign) votes[q][j] += bit ? 1 : -1;
                  if (C == kCodecEFSign) sum[q][j] += bit ? s_peer[p].s0 : -s_peer[p].s0;
                  if (C == kCodecOneBit) sum[q][j] += bit ? s_peer[p].s0 : s_peer[p].s1;
                }
              } else if (T::bits == 32) {
                const long long i = gb + 4 * lane;
                const uint4 w = ld_cg_u4(slot + off_codes + (size_t)i * 4);
                sum[q][0] += __uint_as_float(w.x); sum[q][1] += __uint_as_float(w.y);
                sum[q][2] += __uint_as_float(w.z); sum[q][3] += __uint_as_float(w.w);
              } else if (C == kCodecQSGDX) {
                const float d = dq[q] / (float)a.quantum;
                sum[q][0] += d * (float)(short)(w0[q] & 0xffffu); sum[q][1] += d * (float)(short)(w0[q] >> 16);
                sum[q][2] += d * (float)(short)(w1[q] & 0xffffu); sum[q][3] += d * (float)(short)(w1[q] >> 16);
              } else {  // fp16
                const float2 f01 = __half22float2(*reinterpret_cast<__half2*>(&w0[q]));
                const float2 f23 = __half22float2(*reinterpret_cast<__half2*>(&w1[q]));
                sum[q][0] += f01.x; sum[q][1] += f01.y; sum[q][2] += f23.x; sum[q][3] += f23.y;
              }
            }
          }
#pragma unroll
          for (int q = 0; q < kU; ++q) {
            const long long gb = gb0 + 128ll * kWarps * q;
            if (gb >= e0) continue;
            const long long i = gb + 4 * lane;
            int valid = 0;
            if (i < e0) valid = (e0 - i) >= 4 ? 4 : (int)(e0 - i);
            float ov[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (C == kCodecSign) ov[j] = votes[q][j] >= 0 ? 1.f : -1.f;
              else if (C == kCodecEFSign) ov[j] = sum[q][j] / a.lr;
              else ov[j] = sum[q][j] * a.scale;
            }
            if (valid) store4g(a.out, a.g_dtype, i, valid, ov);
          }
        }
      });
    }
    bar.sync();
    if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
      uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
      st_release_sys(ack, a.peers.seq);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Pipelined all-gather mode: encode and pull overlap tile by tile inside one launch.
//
// The flat buffer is cut into tiles of `pipe_item_elems` elements and chunks of `pipe_chunk_items` tiles.  All
// CTAs draw work from one queue whose order is  E(0) | E(1) D(0) | E(2) D(1) | ... | E(C-1) D(C-2) | D(C-1)
// (E(c) = the encode tiles of chunk c, D(c) = its decode tiles).  The CTA that encodes the last tile of chunk c
// publishes the chunk to every peer (one flag per rank and chunk, value = sequence number); a CTA that draws a
// decode tile of chunk c waits (bounded) until all ranks have published chunks 0..c and then pulls that tile's
// codes from every rank with the staged decode.  While some CTAs pull chunk c over NVLink, the others encode chunk
// c + 1 out of HBM: the two halves of the exchange, one link bound and one memory bound, run side by side.
// Encode tiles never wait, and the encode tiles of chunks <= c + 1 are all handed out before the first decode tile
// of chunk c, so no wait can depend on work that is still in the queue.  Results are bit-identical to the
// phase-by-phase kernel above (same random streams by element index, same rank order of the sums).
template <int C>
__global__ void __launch_bounds__(kBlock, 2) quant_pipeline_kernel(const QuantArgs a) {
  static_assert(C == kCodecQSGD || C == kCodecNatural, "pipelined mode: 8-bit codecs without a statistics pass");
  extern __shared__ __align__(16) unsigned char s_dyn[];
  struct Work { int kind, chunk, chunk_tiles; long long lo; };
  __shared__ Work s_work[2];
  __shared__ int s_flag;

  const Status status{a.status};
  // CTAs that draw no tile reach the final grid barrier at once and wait there for those that are still waiting for
  // a peer's chunk: the barrier's limit is twice the limit of a flag wait, so that a missing peer is reported as
  // such (by the flag wait that expires first) and not as a barrier that gave up.
  GridBarrier bar{a.barrier, 0u, 2 * a.peers.timeout_ns, status};
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = a.peers.rank, world = a.peers.world;
  char* const my_heap = a.peers.heap[rank];
  char* const my_slot = my_heap + a.peers.slot_off;
  const size_t off_codes = kHeaderBytes + scalars_bytes(a.nseg);
  const size_t off_norms = off_codes + codes_bytes(8, a.total);

  // the slot of this parity was last used by sequence seq-2: wait until every peer has acknowledged reading it
  if (tid < world && tid != rank && a.peers.seq > 2) {
    const uint64_t* ack = reinterpret_cast<const uint64_t*>(my_heap + a.peers.ack_off) + tid;
    wait_flag_ge(ack, a.peers.seq - 2, a.peers.timeout_ns, status, kTimeoutPeerAck, tid);
  }
  __syncthreads();

  auto encode_range = [&](long long r_lo, long long r_hi) {
    for_each_segment_range(a.segs, a.nseg, r_lo, r_hi, [&](int, long long b0, long long e0) {
      // a tile is at most 2^20 elements: 32-bit offsets from b0 keep the loop's live state small
      const int len = (int)(e0 - b0);
      for (int o0 = 128 * warp; o0 < len; o0 += 128 * kWarps * kU) {
        float pav[kU][4];
#pragma unroll
        for (int q = 0; q < kU; ++q) {
          const int po = o0 + 128 * kWarps * q + 4 * lane;
          const int pv = po < len ? ((len - po) >= 4 ? 4 : len - po) : 0;
          float gv[4] = {0.f, 0.f, 0.f, 0.f}, rv[4] = {0.f, 0.f, 0.f, 0.f};
          if (pv) {
            load4g(a.g, a.g_dtype, b0 + po, pv, gv);
            if (a.acc && a.beta != 0.f) load4(a.acc, b0 + po, pv, rv);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) pav[q][j] = a.beta * rv[j] + a.gamma * gv[j];
        }
#pragma unroll
        for (int q = 0; q < kU; ++q) {
          const int go = o0 + 128 * kWarps * q;
          if (go >= len) break;  // warp-uniform
          const long long gb = b0 + go;
          const long long i = gb + 4 * lane;
          const int valid = (go + 4 * lane) < len ? ((len - go - 4 * lane) >= 4 ? 4 : len - go - 4 * lane) : 0;
          float xv[4], dv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) { xv[j] = pav[q][j]; dv[j] = 0.f; }
          Philox4 rnd{0u, 0u, 0u, 0u};
          if (C == kCodecQSGD || !a.deterministic) rnd = philox_group((uint64_t)(i >> 2), a.step, 0u, a.seed);
          const unsigned rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
          unsigned word = 0;
          if (C == kCodecQSGD) {
            float sq = xv[0] * xv[0] + xv[1] * xv[1] + xv[2] * xv[2] + xv[3] * xv[3];
            sq = warp_sum(sq);
            const float norm = sqrtf(sq);
            const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
            const float dq = norm / (float)a.quantum;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float lf = qn * fabsf(xv[j]);
              const float fl = floorf(lf);
              float level = fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f);
              level = fminf(level, 127.f);
              const int code = xv[j] < 0.f ? -(int)level : (int)level;
              word |= ((unsigned)code & 0xffu) << (8 * j);
              dv[j] = dq * (float)code;
            }
            if (lane == 0) *reinterpret_cast<float*>(my_slot + off_norms + (size_t)(gb >> 7) * 4) = norm;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const unsigned bits = __float_as_uint(xv[j]);
              const unsigned biased = (bits >> 23) & 0xffu;
              const unsigned mant = bits & 0x7fffffu;
              bool up;
              if (a.deterministic) up = mant > 0x400000u;
              else up = u01(rw[j]) < (float)mant * 1.1920928955078125e-07f;
              int c7 = (int)biased + (up ? 1 : 0) - 17;
              c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
              if (biased == 0) c7 = 0;
              const unsigned code = (unsigned)c7 | ((bits >> 24) & 0x80u);
              word |= code << (8 * j);
              dv[j] = natural_decode(code);
            }
          }
          if (GRACE_IN_RANGE(status, kKernelQuant, off_codes + (size_t)i + 3, a.peers.slot_bytes))
            *reinterpret_cast<unsigned*>(my_slot + off_codes + (size_t)i) = word;
          if (a.acc && valid) {
            float res[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) res[j] = xv[j] - dv[j];
            store4(a.acc, i, valid, res);
          }
        }
      }
    });
  };

  auto decode_range = [&](long long r_lo, long long r_hi) {
    uint4* const st_codes = reinterpret_cast<uint4*>(s_dyn + warp * kStageWarpBytes);                      // [rank][32]
    float* const st_norms = reinterpret_cast<float*>(s_dyn + warp * kStageWarpBytes + kStagePeers * 512);  // [rank][4]
    for_each_segment_range(a.segs, a.nseg, r_lo, r_hi, [&](int, long long b0, long long e0) {
      for (long long w0 = b0 + 512ll * warp; w0 < e0; w0 += 512ll * kWarps) {
        {
          const long long le = w0 + 16ll * lane;
          const bool have = le < e0;
          uint4 v[kStagePeers];
          // the four norms of the block from each of up to eight ranks: one load per lane (rank = lane / 4)
          float nv = 0.f;
          if (C == kCodecQSGD && (lane >> 2) < world && w0 + 128ll * (lane & 3) < e0)
            nv = ld_cg_f32(a.peers.heap[lane >> 2] + a.peers.slot_off + off_norms + (size_t)((w0 >> 7) + (lane & 3)) * 4);
#pragma unroll
          for (int p = 0; p < kStagePeers; ++p) {
            v[p] = make_uint4(0u, 0u, 0u, 0u);
            if (p < world) {
              const char* slot = a.peers.heap[p] + a.peers.slot_off;
              if (have && GRACE_IN_RANGE(status, kKernelQuant, off_codes + (size_t)le + 15, a.peers.slot_bytes))
                v[p] = ld_cg_u4(slot + off_codes + (size_t)le);
            }
          }
          __syncwarp();   // the previous trip's readers are done with the staging area
          if (C == kCodecQSGD) st_norms[lane] = nv;   // [rank][4]
#pragma unroll
          for (int p = 0; p < kStagePeers; ++p)
            if (p < world) st_codes[p * 32 + lane] = v[p];
          __syncwarp();
        }
        float acc16[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc16[j] = 0.f;
        for (int p = 0; p < world; ++p) {
          const uint4 cw = st_codes[p * 32 + lane];
          const unsigned words[4] = {cw.x, cw.y, cw.z, cw.w};
          float d = 0.f;
          if (C == kCodecQSGD) d = st_norms[p * 4 + (lane >> 3)] / (float)a.quantum;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const unsigned byte = (words[j >> 2] >> (8 * (j & 3))) & 0xffu;
            if (C == kCodecQSGD) acc16[j] += d * (float)(int)(signed char)byte;
            else acc16[j] += natural_decode(byte);
          }
        }
        const long long i = w0 + 16ll * lane;
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const long long iv = i + 4 * v4;
          if (iv >= e0) continue;
          const int valid = (e0 - iv) >= 4 ? 4 : (int)(e0 - iv);
          const float ov[4] = {acc16[4 * v4] * a.scale, acc16[4 * v4 + 1] * a.scale, acc16[4 * v4 + 2] * a.scale,
                               acc16[4 * v4 + 3] * a.scale};
          store4g(a.out, a.g_dtype, iv, valid, ov);
        }
      }
    });
  };

  // ---- the queue: thread 0 draws a position and turns it into (encode or decode, chunk, element range) ----
  auto draw = [&](int slot) {
    const unsigned n_items = (unsigned)((a.total + a.pipe_item_elems - 1) / a.pipe_item_elems);   // tiles of one pass
    const unsigned T = (unsigned)a.pipe_chunk_items, NC = (unsigned)a.pipe_chunks;
    const unsigned n_last = n_items - (NC - 1) * T;                                                // tiles of the last chunk
    const unsigned q = atomicAdd(&a.pipe[0], 1u);
    int kind = 0;   // 0: the queue is empty, 1: encode, 2: decode
    unsigned c = 0, t = 0;
    if (q < 2u * n_items) {
      if (q < (NC > 1 ? T : n_last)) {
        kind = 1; c = 0; t = q;
      } else if (NC == 1) {
        kind = 2; c = 0; t = q - n_last;
      } else {
        const unsigned q1 = q - T;
        if (q1 < (NC - 2) * 2u * T) {                  // full blocks: E(k) then D(k - 1), k = 1 .. NC - 2
          const unsigned k = 1 + q1 / (2u * T), r = q1 % (2u * T);
          kind = r < T ? 1 : 2; c = r < T ? k : k - 1; t = r < T ? r : r - T;
        } else {                                        // the last block: E(NC - 1), D(NC - 2), D(NC - 1)
          const unsigned r = q1 - (NC - 2) * 2u * T;
          if (r < n_last) { kind = 1; c = NC - 1; t = r; }
          else if (r < n_last + T) { kind = 2; c = NC - 2; t = r - n_last; }
          else { kind = 2; c = NC - 1; t = r - n_last - T; }
        }
      }
    }
    s_work[slot].kind = kind;
    s_work[slot].chunk = (int)c;
    s_work[slot].chunk_tiles = (int)(c + 1 < NC ? T : n_last);
    s_work[slot].lo = ((long long)c * T + t) * a.pipe_item_elems;
  };
  if (tid == 0) draw(0);
  __syncthreads();
  for (unsigned n = 0;; ++n) {
    const int kind = s_work[n & 1].kind;
    if (kind == 0) break;
    if (tid == 0) draw((n + 1) & 1);   // the next draw travels while this tile is worked on
    const long long r_lo = s_work[n & 1].lo;
    const long long r_hi = r_lo + a.pipe_item_elems < a.total ? r_lo + a.pipe_item_elems : a.total;
    if (kind == 1) {
      if (!status.failed()) encode_range(r_lo, r_hi);
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        const unsigned done = atomicAdd(&a.pipe[1 + s_work[n & 1].chunk], 1u) + 1u;
        s_flag = done == (unsigned)s_work[n & 1].chunk_tiles;
        if (s_flag) __threadfence();
      }
      __syncthreads();
      if (s_flag && tid < world && !status.failed()) {   // this CTA encoded the chunk's last tile: publish it
        __threadfence_system();
        uint64_t* flag = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.chunk_ready_off) +
                         (size_t)rank * kPipeMaxChunks + s_work[n & 1].chunk;
        st_release_sys(flag, a.peers.seq);
      }
    } else {
      if (tid == 0) s_flag = 1;
      __syncthreads();
      if (tid < world * (s_work[n & 1].chunk + 1)) {      // chunks 0..c of every rank (own rank included)
        const uint64_t* flag = reinterpret_cast<const uint64_t*>(my_heap + a.chunk_ready_off) +
                               (size_t)(tid % world) * kPipeMaxChunks + tid / world;
        if (!wait_flag_ge(flag, a.peers.seq, a.peers.timeout_ns, status, kTimeoutPeerReady, tid % world)) s_flag = 0;
      }
      __syncthreads();
      if (s_flag) decode_range(r_lo, r_hi);
    }
    __syncthreads();
  }
  bar.sync();
  if (blockIdx.x == 0 && tid < world && tid != rank && !status.failed()) {
    uint64_t* ack = reinterpret_cast<uint64_t*>(a.peers.heap[tid] + a.peers.ack_off) + rank;
    st_release_sys(ack, a.peers.seq);
  }
}

// Dynamic shared memory of a launch: the staging areas, when the staged decode can run.
template <int C>
constexpr bool staged_codec() { return CodecTraits<C>::bits == 1 || CodecTraits<C>::bits == 2 || CodecTraits<C>::bits == 8; }

template <int C>
cudaError_t launch_codec(const QuantArgs& a, int grid, cudaStream_t stream) {
  QuantArgs copy = a;
  void* params[] = {&copy};
  const void* fn = a.recv_mc ? (const void*)quant_exchange_kernel<C, true> : (const void*)quant_exchange_kernel<C, false>;
  size_t smem = 0;
  if (staged_codec<C>() && a.peers.world > 1 && a.peers.world <= kStagePeers && (a.phases & (kPhaseExchange | kPhaseReduce))) {
    smem = kStageBytes;
    static bool attr_set[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int v = a.recv_mc ? 1 : 0;
    if (dev >= 0 && dev < 64 && !attr_set[dev][v]) {
      cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
      if (err != cudaSuccess) return err;
      attr_set[dev][v] = true;
    }
  }
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kBlock), params, smem, stream);
}

template <int C>
int occupancy(int device, int sm_limit) {
  int per_sm = 0, sms = 0;
  int per_sm_push = 0;
  cudaFuncSetAttribute(quant_exchange_kernel<C, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
  cudaFuncSetAttribute(quant_exchange_kernel<C, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_exchange_kernel<C, false>, kBlock, kStageBytes);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_push, quant_exchange_kernel<C, true>, kBlock, kStageBytes);
  if (per_sm_push < per_sm) per_sm = per_sm_push;   // one grid size serves both variants
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  if (per_sm > 2) per_sm = 2;
  return per_sm * sms;
}

void build_u8_edges(float* e) {
  // 8-bit dynamic-tree bin edges: seven hand-placed small values, then eight
  // linear runs whose step grows from run to run, then the top edge.
  const float head[7] = {1.5000001e-06f, 2.7500000e-06f, 7.2499997e-06f, 1.8750001e-05f,
                         3.6250000e-05f, 5.8749996e-05f, 8.6249995e-05f};
  int n = 0;
  for (int i = 0; i < 7; ++i) e[n++] = head[i];
  const double start[8] = {1.4375e-04, 5.1875e-04, 1.21875e-03, 4.84375e-03, 1.109375e-02, 4.671875e-02, 1.0546875e-01, 4.5859375e-01};
  const double step[8] = {8.75e-05, 1.375e-04, 4.375e-04, 6.875e-04, 2.1875e-03, 3.4375e-03, 1.09375e-02, 1.71875e-02};
  const int count[8] = {4, 4, 8, 8, 16, 16, 32, 32};
  for (int r = 0; r < 8; ++r)
    for (int i = 0; i < count[r]; ++i) e[n++] = (float)(start[r] + i * step[r]);
  e[n++] = 9.9570298e-01f;
}

}  // namespace

size_t quant_slot_bytes(int codec, long long total, int nseg, int alltoall_world, long long nbuckets) {
  int bits = 8;
  switch (codec) {
    case kCodecQSGDX: bits = 16; break;
    case kCodecTernGrad: bits = 2; break;
    case kCodecSign: case kCodecEFSign: case kCodecOneBit: bits = 1; break;
    case kCodecFP16: bits = 16; break;
    case kCodecFP32: bits = 32; break;
    default: bits = 8;
  }
  size_t bytes = region1_bytes(codec, bits, total, nseg, nbuckets);
  if (alltoall_world > 0) {
    const long long groups = total / 128;
    const long long chunk_groups = (groups + alltoall_world - 1) / alltoall_world;
    bytes += codes_bytes(bits, chunk_groups * 128) + (size_t)chunk_groups * 4;
  }
  return (bytes + 255) / 256 * 256;
}

int quant_max_grid(int device, int sm_limit) { return occupancy<kCodecQSGD>(device, sm_limit); }

template <int C>
static cudaError_t launch_pipeline(const QuantArgs& a, int grid, cudaStream_t stream) {
  const void* fn = (const void*)quant_pipeline_kernel<C>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes);
    if (err != cudaSuccess) return err;
    attr_set[dev] = true;
  }
  int per_sm = 0;
  cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kBlock, kStageBytes);
  if (err != cudaSuccess) return err;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  QuantArgs copy = a;
  void* params[] = {&copy};
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kBlock), params, kStageBytes, stream);
}

cudaError_t launch_quant_pipeline(const QuantArgs& a, int grid, cudaStream_t stream) {
  const long long items = a.pipe_item_elems > 0 ? (a.total + a.pipe_item_elems - 1) / a.pipe_item_elems : 0;
  if (!a.pipe || !a.chunk_ready_off || a.pipe_chunks < 1 || a.pipe_chunks > kPipeMaxChunks || a.pipe_item_elems < 8192 ||
      a.pipe_item_elems % 8192 || a.pipe_chunk_items < 1 || a.peers.world < 1 || a.peers.world > kStagePeers ||
      a.alltoall || a.recv_mc || a.phases != kPhaseAll || !a.out ||
      (long long)(a.pipe_chunks - 1) * a.pipe_chunk_items >= items || (long long)a.pipe_chunks * a.pipe_chunk_items < items)
    return cudaErrorInvalidValue;
  cudaError_t err = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (err != cudaSuccess) return err;
  err = cudaMemsetAsync(a.pipe, 0, sizeof(unsigned) * (1 + kPipeMaxChunks), stream);
  if (err != cudaSuccess) return err;
  if (a.codec == kCodecQSGD) return launch_pipeline<kCodecQSGD>(a, grid, stream);
  if (a.codec == kCodecNatural) return launch_pipeline<kCodecNatural>(a, grid, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_quant_exchange(const QuantArgs& a, int grid, cudaStream_t stream) {
  static bool edges_loaded[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !edges_loaded[dev]) {
    float e[128];
    build_u8_edges(e);
    cudaError_t err = cudaMemcpyToSymbol(c_u8_edges, e, sizeof(e));
    if (err != cudaSuccess) return err;
    edges_loaded[dev] = true;
  }
  cudaError_t err = cudaMemsetAsync(a.barrier, 0, sizeof(unsigned), stream);
  if (err != cudaSuccess) return err;
  switch (a.codec) {
    case kCodecQSGD: return launch_codec<kCodecQSGD>(a, grid, stream);
    case kCodecTernGrad: return launch_codec<kCodecTernGrad>(a, grid, stream);
    case kCodecNatural: return launch_codec<kCodecNatural>(a, grid, stream);
    case kCodecU8bit: return launch_codec<kCodecU8bit>(a, grid, stream);
    case kCodecSign: return launch_codec<kCodecSign>(a, grid, stream);
    case kCodecEFSign: return launch_codec<kCodecEFSign>(a, grid, stream);
    case kCodecOneBit: return launch_codec<kCodecOneBit>(a, grid, stream);
    case kCodecFP16: return launch_codec<kCodecFP16>(a, grid, stream);
    case kCodecFP32: return launch_codec<kCodecFP32>(a, grid, stream);
    case kCodecQSGDX:
      if (a.qsgd_bucket < 4 || a.qsgd_bucket % 4 || a.qsgd_nbuckets < 1 || a.alltoall || a.recv_mc) return cudaErrorInvalidValue;
      return launch_codec<kCodecQSGDX>(a, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace grace
