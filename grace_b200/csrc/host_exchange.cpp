// Host engine of the exchange protocol (see host_exchange.h): CPU ranks over
// POSIX shared memory, the same flags / slots / bounded waits as the kernels.
#include "host_exchange.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>
#include <vector>

#include <cuda_runtime.h>   // __host__ / __device__ markers of philox.cuh for the host compiler

#include "philox.cuh"

namespace grace {
namespace host {

namespace {

inline uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

inline uint64_t load_acquire(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void store_release(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

struct StatusBlock {
  unsigned* words;
  bool failed() const { return __atomic_load_n(words, __ATOMIC_ACQUIRE) != kOk; }
  unsigned code() const { return __atomic_load_n(words, __ATOMIC_ACQUIRE); }
  void fail(unsigned code, unsigned detail, unsigned seq) const {
    unsigned expected = kOk;
    if (__atomic_compare_exchange_n(words, &expected, code, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
      words[1] = detail;
      words[2] = seq;
    }
  }
};

// Bounded wait on a flag that a peer stores with release order.  Spins briefly, then yields the core: the ranks of
// a test usually outnumber the cores.
bool wait_flag_ge(const uint64_t* flag, uint64_t want, uint64_t timeout_ns, const StatusBlock& st, unsigned code,
                  unsigned detail) {
  if (load_acquire(flag) >= want) return true;
  const uint64_t t0 = now_ns();
  unsigned spins = 0;
  while (load_acquire(flag) < want) {
    if (++spins > 64) {
      if (now_ns() - t0 > timeout_ns) {
        st.fail(code, detail, (unsigned)want);
        return false;
      }
      timespec nap{0, spins > 4096 ? 200000 : 2000};
      nanosleep(&nap, nullptr);
    }
  }
  return true;
}

struct SlotView {
  char* base;
  uint64_t* count() const { return reinterpret_cast<uint64_t*>(base); }
  float* scalar(int i) const { return reinterpret_cast<float*>(base + 8) + i; }
  char* payload() const { return base + kSlotHeaderBytes; }
};

inline long long groups128(long long n) { return (n + 127) / 128; }

// Position e of a random-k exchange: word e of Philox stream 7 (the stream the GPU kernel uses), modulo the length.
inline long long randomk_position(const Args& a, long long e) {
  const Philox4 r = philox_group((uint64_t)(e >> 2), a.step, 7u, a.seed);
  const unsigned w = (e & 3) == 0 ? r.x : ((e & 3) == 1 ? r.y : ((e & 3) == 2 ? r.z : r.w));
  return (long long)(w % (unsigned)a.n);
}

inline uint32_t float_bits(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  return b;
}
inline float bits_float(uint32_t b) {
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

// Natural compression, the code of the CUDA extension (cnat_cuda.cu:8-66): 7 bits of biased exponent minus 17
// (0 = zero, saturating at 127) and the sign in bit 7.
inline float natural_decode(unsigned code) {
  const unsigned c7 = code & 0x7fu;
  return bits_float((c7 ? ((c7 + 17u) << 23) : 0u) | ((code & 0x80u) << 24));
}

// fp32 -> fp16 -> fp32 with round-to-nearest-even (what __float2half_rn does), without relying on a half type.
inline uint16_t float_to_half(float f) {
  const uint32_t b = float_bits(f), sign = (b >> 16) & 0x8000u;
  const uint32_t e = (b >> 23) & 0xffu, m = b & 0x7fffffu;
  if (e == 0xffu) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0u));
  const int he = (int)e - 127 + 15;
  if (he >= 31) return (uint16_t)(sign | 0x7c00u);
  if (he <= 0) {
    if (he < -10) return (uint16_t)sign;
    const uint32_t mant = m | 0x800000u;
    const int shift = 14 - he;
    uint32_t h = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
  }
  uint32_t h = ((uint32_t)he << 10) | (m >> 13);
  const uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;   // a carry into the exponent is the right answer
  return (uint16_t)(sign | h);
}
inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) {
    if (!m) return bits_float(sign);
    const float v = std::ldexp((float)m, -24);
    return sign ? -v : v;
  }
  if (e == 31) return bits_float(sign | 0x7f800000u | (m << 13));
  return bits_float(sign | ((e + 112u) << 23) | (m << 13));
}

// The 128 bin edges of the 8-bit dynamic-tree data type (grace_dl/tensorflow/compressor/u8bit.py:12-47): seven
// hand-placed small values, eight linear runs whose step grows from run to run, the top edge.
const float* u8_edges() {
  static float e[128];
  static const bool built = [] {
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
    return n == 128;
  }();
  (void)built;
  return e;
}
inline int u8_bin(float y, const float* edges) {   // largest i in [0, 126] with edges[i] <= y (0 below the first edge)
  int lo = 0, hi = 127;
  for (int it = 0; it < 7; ++it) {
    const int mid = (lo + hi) >> 1;
    if (edges[mid] <= y) lo = mid; else hi = mid;
  }
  return lo;
}
inline long long words32(long long n) { return (n + 31) / 32; }

// ---- compress: x = beta * acc + gamma * g, encode x into the slot, acc = x - decode(code) ----
unsigned compress(const Args& a, const SlotView& slot, uint64_t slot_bytes_avail, float clip_bound) {
  const long long n = a.n;
  if (slot_bytes(a.codec, n, a.codec == kQSGDX ? a.bucket : a.k) > slot_bytes_avail) return kSlotOverflow;
  std::vector<float> xbuf;
  const float* x = a.g;
  if (a.u && a.acc) {   // DGC momentum correction (memory/dgc.py:21-30): u = m u + g, v += u, v is what is encoded
    for (long long i = 0; i < n; ++i) {
      const float g = std::max(std::min(a.g[i], clip_bound), -clip_bound);   // the bound is +inf without clipping
      a.u[i] = a.momentum * a.u[i] + g;
      a.acc[i] += a.u[i];
    }
    x = a.acc;
  } else if (a.acc) {   // error feedback: the accumulator holds x while it is encoded
    for (long long i = 0; i < n; ++i) a.acc[i] = a.beta * a.acc[i] + a.gamma * a.g[i];
    x = a.acc;
  } else if (a.gamma != 1.f) {
    xbuf.resize(n);
    for (long long i = 0; i < n; ++i) xbuf[i] = a.gamma * a.g[i];
    x = xbuf.data();
  }
  char* pay = slot.payload();
  switch (a.codec) {
    case kTopK: {
      const long long k = std::min(a.k, n);
      if (k < 1) return kBadArgument;
      // Radix select as on the GPU: a 4096-bin histogram of the top 12 key bits finds the bin of the k-th largest
      // magnitude; everything above that bin travels, the bin itself is partitioned (ties: lowest index first).
      auto key_of = [x](long long i) {
        uint32_t b;
        std::memcpy(&b, x + i, 4);
        return b & 0x7fffffffu;
      };
      std::vector<uint32_t> hist(4096, 0);
      for (long long i = 0; i < n; ++i) ++hist[key_of(i) >> 19];
      long long above = 0;
      int bin = 4095;
      for (; bin > 0; --bin) {
        if (above + hist[bin] >= k) break;
        above += hist[bin];
      }
      std::vector<int> order, cand;
      order.reserve((size_t)k);
      cand.reserve(hist[bin]);
      for (long long i = 0; i < n; ++i) {
        const uint32_t top = key_of(i) >> 19;
        if (top > (uint32_t)bin) order.push_back((int)i);
        else if (top == (uint32_t)bin) cand.push_back((int)i);
      }
      const long long need = k - above;
      auto larger = [&](int p, int q) {
        const uint32_t kp = key_of(p), kq = key_of(q);
        return kp > kq || (kp == kq && p < q);
      };
      if (need < (long long)cand.size()) std::nth_element(cand.begin(), cand.begin() + need, cand.end(), larger);
      order.insert(order.end(), cand.begin(), cand.begin() + need);
      std::sort(order.begin(), order.end());   // ascending indices: the same list whatever the partition did
      float* val = reinterpret_cast<float*>(pay);
      int* idx = reinterpret_cast<int*>(pay + (size_t)a.k * 4);
      for (long long j = 0; j < k; ++j) {
        idx[j] = order[j];
        val[j] = x[order[j]];
        if (a.acc) a.acc[order[j]] = 0.f;
        if (a.u) a.u[order[j]] = 0.f;
      }
      *slot.count() = (uint64_t)k;
      break;
    }
    case kThreshold: {
      float* val = reinterpret_cast<float*>(pay);
      int* idx = reinterpret_cast<int*>(pay + (size_t)a.k * 4);
      long long m = 0;
      for (long long i = 0; i < n && m < a.k; ++i) {
        const float ax = std::fabs(x[i]);
        if (a.strict ? ax > a.threshold : ax >= a.threshold) {
          idx[m] = (int)i;
          val[m] = x[i];
          if (a.acc) a.acc[i] = 0.f;
          ++m;
        }
      }
      *slot.count() = (uint64_t)m;   // what did not fit stays in the accumulator
      break;
    }
    case kQSGD: {
      if (a.quantum < 1 || a.quantum > 127) return kBadArgument;
      float* norms = reinterpret_cast<float*>(pay);
      signed char* codes = reinterpret_cast<signed char*>(pay + (size_t)groups128(n) * 4);
      for (long long b = 0; b < groups128(n); ++b) {
        const long long lo = b * 128, hi = std::min(n, lo + 128);
        float sq = 0.f;
        for (long long i = lo; i < hi; ++i) sq += x[i] * x[i];
        const float norm = std::sqrt(sq);
        norms[b] = norm;
        const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f, dq = norm / (float)a.quantum;
        for (long long g4 = lo; g4 < hi; g4 += 4) {
          const Philox4 r = philox_group((uint64_t)(g4 >> 2), a.step, 0u, a.seed);
          const unsigned rw[4] = {r.x, r.y, r.z, r.w};
          for (int j = 0; j < 4 && g4 + j < hi; ++j) {
            const long long i = g4 + j;
            const float lf = qn * std::fabs(x[i]), fl = std::floor(lf);
            float level = fl + ((u01(rw[j]) < lf - fl) ? 1.f : 0.f);
            level = std::min(level, 127.f);
            const int code = x[i] < 0.f ? -(int)level : (int)level;
            codes[i] = (signed char)code;
            if (a.acc) a.acc[i] = x[i] - dq * (float)code;
          }
        }
      }
      break;
    }
    case kSign:
    case kEFSign: {
      unsigned* bits = reinterpret_cast<unsigned*>(pay);
      float mean = 0.f;
      if (a.codec == kEFSign) {
        double s = 0.0;
        for (long long i = 0; i < n; ++i) s += std::fabs(x[i]);
        mean = n ? (float)(s / (double)n) : 0.f;
        *slot.scalar(0) = mean;
      }
      std::vector<float> mbuf;
      const float* enc = x;
      if (a.codec == kSign && a.mom) {   // signum: the sign of the momentum
        for (long long i = 0; i < n; ++i)
          a.mom[i] = a.first_step ? x[i] : (1.f - a.mom_beta) * x[i] + a.mom_beta * a.mom[i];
        enc = a.mom;
      }
      for (long long w = 0; w < words32(n); ++w) {
        unsigned word = 0;
        const long long lim = std::min<long long>(32, n - w * 32);
        for (long long j = 0; j < lim; ++j) word |= (unsigned)(enc[w * 32 + j] >= 0.f) << j;   // no branch: signs are coin flips
        bits[w] = word;
      }
      if (a.acc) {
        const float mag = a.codec == kEFSign ? mean : 1.f;
        for (long long i = 0; i < n; ++i) a.acc[i] = x[i] - mag * (float)(2 * (int)(enc[i] >= 0.f) - 1);
      }
      break;
    }
    case kDense: {
      std::memcpy(pay, x, (size_t)n * 4);
      if (a.acc) std::memset(a.acc, 0, (size_t)n * 4);
      break;
    }
    case kTernGrad: {
      double sum = 0.0, sumsq = 0.0;
      float maxabs = 0.f;
      for (long long i = 0; i < n; ++i) {
        sum += x[i];
        sumsq += (double)x[i] * x[i];
        maxabs = std::max(maxabs, std::fabs(x[i]));
      }
      const double mean = n ? sum / (double)n : 0.0;
      const double var = n ? std::max(0.0, sumsq / (double)n - mean * mean) : 0.0;
      const float c = 2.5f * (float)std::sqrt(var), s0 = std::min(maxabs, c);   // max |clamp(x, -c, c)|
      *slot.scalar(0) = s0;
      signed char* codes = reinterpret_cast<signed char*>(pay);
      for (long long g4 = 0; g4 < n; g4 += 4) {
        const Philox4 r = philox_group((uint64_t)(g4 >> 2), a.step, 0u, a.seed);
        const unsigned rw[4] = {r.x, r.y, r.z, r.w};
        for (int j = 0; j < 4 && g4 + j < n; ++j) {
          const long long i = g4 + j;
          const bool keep = u01(rw[j]) * s0 < std::min(std::fabs(x[i]), c);
          const int code = keep ? (x[i] < 0.f ? -1 : 1) : 0;
          codes[i] = (signed char)code;
          if (a.acc) a.acc[i] = x[i] - s0 * (float)code;
        }
      }
      break;
    }
    case kNatural: {
      unsigned char* codes = reinterpret_cast<unsigned char*>(pay);
      for (long long g4 = 0; g4 < n; g4 += 4) {
        Philox4 r{0u, 0u, 0u, 0u};
        if (!a.deterministic) r = philox_group((uint64_t)(g4 >> 2), a.step, 0u, a.seed);
        const unsigned rw[4] = {r.x, r.y, r.z, r.w};
        for (int j = 0; j < 4 && g4 + j < n; ++j) {
          const long long i = g4 + j;
          const uint32_t bits = float_bits(x[i]), biased = (bits >> 23) & 0xffu, mant = bits & 0x7fffffu;
          const bool up = a.deterministic ? mant > 0x400000u : u01(rw[j]) < (float)mant * 1.1920928955078125e-07f;
          int c7 = (int)biased + (up ? 1 : 0) - 17;
          c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
          if (biased == 0) c7 = 0;
          const unsigned code = (unsigned)c7 | ((bits >> 24) & 0x80u);
          codes[i] = (unsigned char)code;
          if (a.acc) a.acc[i] = x[i] - natural_decode(code);
        }
      }
      break;
    }
    case kU8bit: {
      const float* edges = u8_edges();
      float s0 = 0.f;
      for (long long i = 0; i < n; ++i) s0 = std::max(s0, std::fabs(x[i]));
      *slot.scalar(0) = s0;
      const float safe = s0 > 0.f ? s0 : 1.f;
      signed char* codes = reinterpret_cast<signed char*>(pay);
      for (long long i = 0; i < n; ++i) {
        const int bin = u8_bin(std::fabs(x[i]) / safe, edges);
        const int sg = x[i] > 0.f ? 1 : (x[i] < 0.f ? -1 : 0);
        const int code = bin * sg;
        codes[i] = (signed char)code;
        if (a.acc) a.acc[i] = x[i] - (code ? edges[bin] * s0 * (float)sg : 0.f);   // bin 0 decodes to exactly 0
      }
      break;
    }
    case kOneBit: {
      double sneg = 0.0, spos = 0.0;
      long long nneg = 0;
      for (long long i = 0; i < n; ++i) {
        if (x[i] < 0.f) { sneg += x[i]; ++nneg; } else spos += x[i];
      }
      const float m0 = nneg ? (float)(sneg / (double)nneg) : 0.f;
      const float m1 = n - nneg ? (float)(spos / (double)(n - nneg)) : 0.f;
      *slot.scalar(0) = m0;
      *slot.scalar(1) = m1;
      unsigned* bits = reinterpret_cast<unsigned*>(pay);
      for (long long w = 0; w < words32(n); ++w) {
        unsigned word = 0;
        const long long lim = std::min<long long>(32, n - w * 32);
        for (long long j = 0; j < lim; ++j) word |= (unsigned)(x[w * 32 + j] < 0.f) << j;
        bits[w] = word;
      }
      if (a.acc)
        for (long long i = 0; i < n; ++i) a.acc[i] = x[i] - (x[i] < 0.f ? m0 : m1);
      break;
    }
    case kQSGDX: {
      if (a.quantum < 1 || a.quantum > 32767 || a.bucket < 1) return kBadArgument;
      const long long nb = (n + a.bucket - 1) / a.bucket;
      float* norms = reinterpret_cast<float*>(pay);
      int16_t* codes = reinterpret_cast<int16_t*>(pay + (size_t)((nb + 3) / 4 * 4) * 4);
      for (long long b = 0; b < nb; ++b) {
        const long long lo = b * a.bucket, hi = std::min(n, lo + a.bucket);
        float sq = 0.f;
        for (long long i = lo; i < hi; ++i) sq += x[i] * x[i];
        const float norm = std::sqrt(sq);
        norms[b] = norm;
        const float qn = norm > 0.f ? (float)a.quantum / norm : 0.f, dq = norm / (float)a.quantum;
        for (long long i = lo; i < hi; ++i) {   // element i draws word i % 4 of Philox group i / 4, whatever the bucket size
          const Philox4 r = philox_group((uint64_t)(i >> 2), a.step, 0u, a.seed);
          const unsigned w = (i & 3) == 0 ? r.x : ((i & 3) == 1 ? r.y : ((i & 3) == 2 ? r.z : r.w));
          const float lf = qn * std::fabs(x[i]), fl = std::floor(lf);
          float level = fl + ((u01(w) < lf - fl) ? 1.f : 0.f);
          level = std::min(level, 32767.f);
          const int code = x[i] < 0.f ? -(int)level : (int)level;
          codes[i] = (int16_t)code;
          if (a.acc) a.acc[i] = x[i] - dq * (float)code;
        }
      }
      break;
    }
    case kRandomK: {
      if (a.k < 1 || n < 1) return kBadArgument;
      float* val = reinterpret_cast<float*>(pay);
      for (long long e = 0; e < a.k; ++e) val[e] = x[randomk_position(a, e)];
      // the residual is zeroed only after every value was read: a position drawn twice sends the same value twice
      if (a.acc)
        for (long long e = 0; e < a.k; ++e) a.acc[randomk_position(a, e)] = 0.f;
      *slot.count() = (uint64_t)a.k;
      break;
    }
    case kFP16: {
      uint16_t* h = reinterpret_cast<uint16_t*>(pay);
      for (long long i = 0; i < n; ++i) {
        h[i] = float_to_half(x[i]);
        if (a.acc) a.acc[i] = x[i] - half_to_float(h[i]);
      }
      break;
    }
    default:
      return kBadArgument;
  }
  return kOk;
}

// ---- decode one rank's slot into the running sum (called in rank order: the sum has one fixed order) ----
unsigned accumulate(const Args& a, const SlotView& slot, float* sum, int* votes) {
  const long long n = a.n;
  const char* pay = slot.payload();
  switch (a.codec) {
    case kTopK:
    case kThreshold: {
      const uint64_t m = *slot.count();
      if (m > (uint64_t)a.k) return kBadArgument;
      const float* val = reinterpret_cast<const float*>(pay);
      const int* idx = reinterpret_cast<const int*>(pay + (size_t)a.k * 4);
      for (uint64_t j = 0; j < m; ++j) {
        if (idx[j] < 0 || idx[j] >= n) return kBadArgument;   // a corrupt index is reported, never followed
        sum[idx[j]] += val[j];
      }
      break;
    }
    case kQSGD: {
      const float* norms = reinterpret_cast<const float*>(pay);
      const signed char* codes = reinterpret_cast<const signed char*>(pay + (size_t)groups128(n) * 4);
      for (long long i = 0; i < n; ++i) sum[i] += norms[i >> 7] / (float)a.quantum * (float)codes[i];
      break;
    }
    case kSign:
    case kEFSign: {
      const unsigned* bits = reinterpret_cast<const unsigned*>(pay);
      const float mean = *slot.scalar(0);
      if (a.codec == kSign) {
        for (long long i = 0; i < n; ++i) votes[i] += 2 * (int)((bits[i >> 5] >> (i & 31)) & 1u) - 1;
      } else {
        for (long long i = 0; i < n; ++i) sum[i] += mean * (float)(2 * (int)((bits[i >> 5] >> (i & 31)) & 1u) - 1);
      }
      break;
    }
    case kDense: {
      const float* v = reinterpret_cast<const float*>(pay);
      for (long long i = 0; i < n; ++i) sum[i] += v[i];
      break;
    }
    case kTernGrad: {
      const signed char* codes = reinterpret_cast<const signed char*>(pay);
      const float s0 = *slot.scalar(0);
      for (long long i = 0; i < n; ++i) sum[i] += s0 * (float)codes[i];
      break;
    }
    case kNatural: {
      const unsigned char* codes = reinterpret_cast<const unsigned char*>(pay);
      for (long long i = 0; i < n; ++i) sum[i] += natural_decode(codes[i]);
      break;
    }
    case kU8bit: {
      const float* edges = u8_edges();
      const signed char* codes = reinterpret_cast<const signed char*>(pay);
      const float s0 = *slot.scalar(0);
      for (long long i = 0; i < n; ++i) {
        const int code = codes[i], bin = code < 0 ? -code : code;
        if (bin > 126) return kBadArgument;
        sum[i] += code ? edges[bin] * s0 * (code < 0 ? -1.f : 1.f) : 0.f;
      }
      break;
    }
    case kOneBit: {
      const unsigned* bits = reinterpret_cast<const unsigned*>(pay);
      const float m0 = *slot.scalar(0), m1 = *slot.scalar(1);
      for (long long i = 0; i < n; ++i) sum[i] += ((bits[i >> 5] >> (i & 31)) & 1u) ? m0 : m1;
      break;
    }
    case kFP16: {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(pay);
      for (long long i = 0; i < n; ++i) sum[i] += half_to_float(h[i]);
      break;
    }
    case kQSGDX: {
      const long long nb = (n + a.bucket - 1) / a.bucket;
      const float* norms = reinterpret_cast<const float*>(pay);
      const int16_t* codes = reinterpret_cast<const int16_t*>(pay + (size_t)((nb + 3) / 4 * 4) * 4);
      for (long long i = 0; i < n; ++i) sum[i] += norms[i / a.bucket] / (float)a.quantum * (float)codes[i];
      break;
    }
    case kRandomK: {   // entry e of every rank belongs to the same position: the first k sums are per entry
      if (*slot.count() != (uint64_t)a.k || a.k > n) return kBadArgument;
      const float* val = reinterpret_cast<const float*>(pay);
      for (long long e = 0; e < a.k; ++e) sum[e] += val[e];
      break;
    }
    default:
      return kBadArgument;
  }
  return kOk;
}

}  // namespace

size_t slot_bytes(int codec, long long n, long long k) {
  size_t b = kSlotHeaderBytes;
  switch (codec) {
    case kQSGDX: {   // k carries the bucket size
      const long long nb = k > 0 ? (n + k - 1) / k : 0;
      b += (size_t)((nb + 3) / 4 * 4) * 4 + (size_t)n * 2;
      break;
    }
    case kTopK:
    case kThreshold: b += (size_t)k * 8; break;
    case kRandomK: b += (size_t)k * 4; break;
    case kQSGD: b += (size_t)groups128(n) * 4 + (size_t)n; break;
    case kSign:
    case kEFSign:
    case kOneBit: b += (size_t)words32(n) * 4; break;
    case kTernGrad:
    case kNatural:
    case kU8bit: b += (size_t)n; break;
    case kFP16: b += (size_t)n * 2; break;
    default: b += (size_t)n * 4; break;
  }
  return (b + 63) / 64 * 64;
}

namespace {

struct Chunking {
  long long chunk;                       // elements per chunk (a multiple of 128)
  long long begin(int r, long long n) const { return std::min(n, chunk * r); }
  long long end(int r, long long n) const { return std::min(n, chunk * (r + 1)); }
};
inline Chunking chunking(long long n, int world) {
  const long long groups = groups128(n), per = (groups + world - 1) / world;
  return Chunking{per * 128};
}
inline size_t region2_bytes(int codec, long long chunk) {
  switch (codec) {
    case kQSGD: return (size_t)(chunk / 128) * 4 + (size_t)chunk;
    case kNatural: return (size_t)chunk;
    case kFP16: return (size_t)chunk * 2;
    default: return (size_t)chunk * 4;
  }
}
inline bool two_phase_codec(int codec) { return codec == kQSGD || codec == kNatural || codec == kFP16 || codec == kDense; }

// Encode the reduced chunk xs[0 .. len) (elements e0 .. e0 + len of the tensor) into region 2.
void encode_chunk(const Args& a, char* r2, const float* xs, long long e0, long long len, long long chunk) {
  switch (a.codec) {
    case kQSGD: {
      float* norms = reinterpret_cast<float*>(r2);
      signed char* codes = reinterpret_cast<signed char*>(r2 + (size_t)(chunk / 128) * 4);
      for (long long b = 0; b * 128 < len; ++b) {
        const long long lo = b * 128, hi = std::min(len, lo + 128);
        float sq = 0.f;
        for (long long i = lo; i < hi; ++i) sq += xs[i] * xs[i];
        const float norm = std::sqrt(sq), qn = norm > 0.f ? (float)a.quantum / norm : 0.f;
        norms[b] = norm;
        for (long long i = lo; i < hi; ++i) {
          const long long gi = e0 + i;   // the random stream is indexed by the element's place in the tensor
          const Philox4 r = philox_group((uint64_t)(gi >> 2), a.step, 1u, a.seed);
          const unsigned w = (gi & 3) == 0 ? r.x : ((gi & 3) == 1 ? r.y : ((gi & 3) == 2 ? r.z : r.w));
          const float lf = qn * std::fabs(xs[i]), fl = std::floor(lf);
          const float level = std::min(fl + ((u01(w) < lf - fl) ? 1.f : 0.f), 127.f);
          codes[i] = (signed char)(xs[i] < 0.f ? -(int)level : (int)level);
        }
      }
      break;
    }
    case kNatural: {
      unsigned char* codes = reinterpret_cast<unsigned char*>(r2);
      for (long long i = 0; i < len; ++i) {
        const long long gi = e0 + i;
        unsigned w = 0;
        if (!a.deterministic) {
          const Philox4 r = philox_group((uint64_t)(gi >> 2), a.step, 1u, a.seed);
          w = (gi & 3) == 0 ? r.x : ((gi & 3) == 1 ? r.y : ((gi & 3) == 2 ? r.z : r.w));
        }
        const uint32_t bits = float_bits(xs[i]), biased = (bits >> 23) & 0xffu, mant = bits & 0x7fffffu;
        const bool up = a.deterministic ? mant > 0x400000u : u01(w) < (float)mant * 1.1920928955078125e-07f;
        int c7 = (int)biased + (up ? 1 : 0) - 17;
        c7 = c7 < 0 ? 0 : (c7 > 127 ? 127 : c7);
        if (biased == 0) c7 = 0;
        codes[i] = (unsigned char)((unsigned)c7 | ((bits >> 24) & 0x80u));
      }
      break;
    }
    case kFP16: {
      uint16_t* h = reinterpret_cast<uint16_t*>(r2);
      for (long long i = 0; i < len; ++i) h[i] = float_to_half(xs[i]);
      break;
    }
    default:
      if (len > 0) std::memcpy(r2, xs, (size_t)len * 4);   // a rank past the end of a short tensor owns an empty chunk
  }
}

void decode_chunk(const Args& a, const char* r2, float* out, long long len, long long chunk) {
  switch (a.codec) {
    case kQSGD: {
      const float* norms = reinterpret_cast<const float*>(r2);
      const signed char* codes = reinterpret_cast<const signed char*>(r2 + (size_t)(chunk / 128) * 4);
      for (long long i = 0; i < len; ++i) out[i] = norms[i >> 7] / (float)a.quantum * (float)codes[i] * a.scale;
      break;
    }
    case kNatural: {
      const unsigned char* codes = reinterpret_cast<const unsigned char*>(r2);
      for (long long i = 0; i < len; ++i) out[i] = natural_decode(codes[i]) * a.scale;
      break;
    }
    case kFP16: {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(r2);
      for (long long i = 0; i < len; ++i) out[i] = half_to_float(h[i]) * a.scale;
      break;
    }
    default: {
      const float* v = reinterpret_cast<const float*>(r2);
      for (long long i = 0; i < len; ++i) out[i] = v[i] * a.scale;
    }
  }
}

// Sum of all ranks' decoded payloads over [e0, e1) (rank order), for the codecs of the two-phase mode.
void reduce_range(const Args& a, const SlotView& slot, float* sum, long long e0, long long e1) {
  const char* pay = slot.payload();
  switch (a.codec) {
    case kQSGD: {
      const float* norms = reinterpret_cast<const float*>(pay);
      const signed char* codes = reinterpret_cast<const signed char*>(pay + (size_t)groups128(a.n) * 4);
      for (long long i = e0; i < e1; ++i) sum[i - e0] += norms[i >> 7] / (float)a.quantum * (float)codes[i];
      break;
    }
    case kNatural: {
      const unsigned char* codes = reinterpret_cast<const unsigned char*>(pay);
      for (long long i = e0; i < e1; ++i) sum[i - e0] += natural_decode(codes[i]);
      break;
    }
    case kFP16: {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(pay);
      for (long long i = e0; i < e1; ++i) sum[i - e0] += half_to_float(h[i]);
      break;
    }
    default: {
      const float* v = reinterpret_cast<const float*>(pay);
      for (long long i = e0; i < e1; ++i) sum[i - e0] += v[i];
    }
  }
}

}  // namespace

size_t two_phase_slot_bytes(int codec, long long n, int world) {
  if (world < 1) world = 1;
  return slot_bytes(codec, n, 0) + (region2_bytes(codec, chunking(n, world).chunk) + 63) / 64 * 64;
}

unsigned exchange(const Channel& ch, const Args& a) {
  if (ch.world < 1 || ch.world > kMaxWorld || ch.rank < 0 || ch.rank >= ch.world || a.n < 0 || a.seq < 1 || !a.g ||
      !a.out)
    return kBadArgument;
  char* mine = ch.heap[ch.rank];
  const StatusBlock st{reinterpret_cast<unsigned*>(mine + ch.status_off)};
  if (st.failed()) return st.code();   // a failed channel stays failed until it is reset
  const unsigned parity = (unsigned)(a.seq & 1);
  const SlotView my_slot{mine + ch.slot_off[parity]};

  if (a.phases & kCompress) {
    // the slot of this parity was last used by sequence seq - 2: every peer must have read it
    if (a.seq > 2) {
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(mine + ch.ack_off);
      for (int p = 0; p < ch.world; ++p)
        if (p != ch.rank && !wait_flag_ge(ack + p, a.seq - 2, ch.timeout_ns, st, kTimeoutPeerAck, (unsigned)p))
          return st.code();
    }
    float clip_bound = INFINITY;
    if (a.clip_ready_off) {
      // every rank's sum of squares first: the bound must be known before the first element is encoded
      double sq = 0.0;
      for (long long i = 0; i < a.n; ++i) sq += (double)a.g[i] * (double)a.g[i];
      *reinterpret_cast<double*>(my_slot.base + 16) = sq;
      for (int p = 0; p < ch.world; ++p)
        store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + a.clip_ready_off) + ch.rank, a.seq);
      const uint64_t* clip_ready = reinterpret_cast<const uint64_t*>(mine + a.clip_ready_off);
      double total = 0.0;
      for (int p = 0; p < ch.world; ++p) {   // rank order: the same bound, bit for bit, on every rank
        if (!wait_flag_ge(clip_ready + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
        total += *reinterpret_cast<const double*>(ch.heap[p] + ch.slot_off[parity] + 16);
      }
      clip_bound = (float)std::sqrt(total / (double)ch.world);
    }
    const unsigned rc = compress(a, my_slot, ch.slot_bytes, clip_bound);
    if (rc != kOk) {
      st.fail(rc, 0, (unsigned)a.seq);
      return st.code();
    }
  }

  if (a.phases & kPublish) {
    for (int p = 0; p < ch.world; ++p)
      store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + ch.ready_off) + ch.rank, a.seq);
  }

  if ((a.phases & kExchange) && a.ready2_off) {
    // ---- two-phase mode: reduce my chunk, encode it again, publish; then decode everybody's chunk ----
    if (!two_phase_codec(a.codec) || two_phase_slot_bytes(a.codec, a.n, ch.world) > ch.slot_bytes) {
      st.fail(kBadArgument, 0, (unsigned)a.seq);
      return st.code();
    }
    const Chunking ck = chunking(a.n, ch.world);
    const size_t r2_off = slot_bytes(a.codec, a.n, 0);          // region 2 follows the one-phase payload
    const uint64_t* ready = reinterpret_cast<const uint64_t*>(mine + ch.ready_off);
    for (int p = 0; p < ch.world; ++p)
      if (!wait_flag_ge(ready + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
    const long long e0 = ck.begin(ch.rank, a.n), e1 = ck.end(ch.rank, a.n);
    std::vector<float> xs((size_t)std::max<long long>(e1 - e0, 0), 0.f);
    for (int p = 0; p < ch.world; ++p) reduce_range(a, SlotView{ch.heap[p] + ch.slot_off[parity]}, xs.data(), e0, e1);
    encode_chunk(a, mine + ch.slot_off[parity] + r2_off, xs.data(), e0, e1 - e0, ck.chunk);
    for (int p = 0; p < ch.world; ++p)
      store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + a.ready2_off) + ch.rank, a.seq);
    const uint64_t* ready2 = reinterpret_cast<const uint64_t*>(mine + a.ready2_off);
    for (int p = 0; p < ch.world; ++p) {
      if (!wait_flag_ge(ready2 + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
      const long long b0 = ck.begin(p, a.n), b1 = ck.end(p, a.n);
      decode_chunk(a, ch.heap[p] + ch.slot_off[parity] + r2_off, a.out + b0, b1 - b0, ck.chunk);
    }
    for (int p = 0; p < ch.world; ++p)
      if (p != ch.rank) store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + ch.ack_off) + ch.rank, a.seq);
    return kOk;
  }

  if (a.phases & kExchange) {
    std::vector<float> sum((size_t)a.n, 0.f);
    std::vector<int> votes(a.codec == kSign ? (size_t)a.n : 0, 0);
    const uint64_t* ready = reinterpret_cast<const uint64_t*>(mine + ch.ready_off);
    for (int p = 0; p < ch.world; ++p) {
      if (!wait_flag_ge(ready + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
      const SlotView peer{ch.heap[p] + ch.slot_off[parity]};
      const unsigned rc = accumulate(a, peer, sum.data(), votes.data());
      if (rc != kOk) {
        st.fail(rc, (unsigned)p, (unsigned)a.seq);
        return st.code();
      }
    }
    // every slot of this sequence has been read: the peers may reuse theirs
    for (int p = 0; p < ch.world; ++p)
      if (p != ch.rank) store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + ch.ack_off) + ch.rank, a.seq);
    if (a.codec == kSign) {
      for (long long i = 0; i < a.n; ++i) a.out[i] = votes[i] >= 0 ? 1.f : -1.f;
    } else if (a.codec == kEFSign) {
      for (long long i = 0; i < a.n; ++i) a.out[i] = sum[i] / a.lr;
    } else if (a.codec == kRandomK) {
      std::vector<float> per_entry(sum.begin(), sum.begin() + a.k);
      for (long long i = 0; i < a.n; ++i) a.out[i] = 0.f;
      for (long long e = 0; e < a.k; ++e) a.out[randomk_position(a, e)] = per_entry[(size_t)e] * a.scale;   // a store, as scatter_ does
    } else {
      for (long long i = 0; i < a.n; ++i) a.out[i] = sum[i] * a.scale;
    }
  }
  return kOk;
}

size_t lowrank_slot_bytes(int rows, int cols, int rank) {
  return (kSlotHeaderBytes + ((size_t)rows + (size_t)cols) * (size_t)rank * 4 + 63) / 64 * 64;
}

unsigned lowrank_exchange(const Channel& ch, const LowRankArgs& a) {
  if (ch.world < 1 || ch.world > kMaxWorld || ch.rank < 0 || ch.rank >= ch.world || a.seq < 1 || !a.g || !a.out || !a.q ||
      !a.p_work || a.rows < 1 || a.cols < 1 || a.rank < 1 || a.rank > 16 || a.rank > a.rows || a.rank > a.cols)
    return kBadArgument;
  char* mine = ch.heap[ch.rank];
  const StatusBlock st{reinterpret_cast<unsigned*>(mine + ch.status_off)};
  if (st.failed()) return st.code();
  if (lowrank_slot_bytes(a.rows, a.cols, a.rank) > ch.slot_bytes) {
    st.fail(kSlotOverflow, 0, (unsigned)a.seq);
    return st.code();
  }
  const int n = a.rows, m = a.cols, r = a.rank;
  const unsigned parity = (unsigned)(a.seq & 1);
  auto slot_p = [&](int p) { return reinterpret_cast<float*>(ch.heap[p] + ch.slot_off[parity] + kSlotHeaderBytes); };
  auto slot_q = [&](int p) { return slot_p(p) + (size_t)n * r; };
  const float inv_world = 1.f / (float)ch.world;
  // without error feedback M' is the gradient itself
  const float* mprime = a.acc ? a.acc : a.g;

  if (a.phases & kCompress) {
    if (a.seq > 2) {
      const uint64_t* ack = reinterpret_cast<const uint64_t*>(mine + ch.ack_off);
      for (int p = 0; p < ch.world; ++p)
        if (p != ch.rank && !wait_flag_ge(ack + p, a.seq - 2, ch.timeout_ns, st, kTimeoutPeerAck, (unsigned)p))
          return st.code();
    }
    if (a.acc)
      for (size_t i = 0; i < (size_t)n * m; ++i) a.acc[i] += a.g[i];   // M' = g + residual
    float* P = slot_p(ch.rank);
    for (int i = 0; i < n; ++i) {                                      // P = M' Q
      float accum[16] = {};
      const float* row = mprime + (size_t)i * m;
      for (int j = 0; j < m; ++j) {
        const float v = row[j];
        const float* qj = a.q + (size_t)j * r;
        for (int c = 0; c < r; ++c) accum[c] += v * qj[c];
      }
      for (int c = 0; c < r; ++c) P[(size_t)i * r + c] = accum[c];
    }
  }
  if (a.phases & kPublish) {
    for (int p = 0; p < ch.world; ++p)
      store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + ch.ready_off) + ch.rank, a.seq);
  }
  if (!(a.phases & kExchange)) return kOk;

  // ---- mean of P over the ranks (rank order), orthogonalisation ----
  const uint64_t* ready = reinterpret_cast<const uint64_t*>(mine + ch.ready_off);
  for (int p = 0; p < ch.world; ++p)
    if (!wait_flag_ge(ready + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
  float* P = a.p_work;
  for (size_t i = 0; i < (size_t)n * r; ++i) {
    float s = 0.f;
    for (int p = 0; p < ch.world; ++p) s += slot_p(p)[i];
    P[i] = s * inv_world;
  }
  double gram[16][16] = {}, R[16][16] = {}, inv[16][16] = {};
  for (int i = 0; i < n; ++i)
    for (int c = 0; c < r; ++c)
      for (int d = c; d < r; ++d) gram[c][d] += (double)P[(size_t)i * r + c] * (double)P[(size_t)i * r + d];
  for (int j = 0; j < r; ++j)                       // upper Cholesky factor: R^T R = Gram
    for (int i = 0; i <= j; ++i) {
      double s = gram[i][j];
      for (int k = 0; k < i; ++k) s -= R[k][i] * R[k][j];
      if (i == j) R[i][j] = s > 0.0 ? std::sqrt(s) : 0.0;
      else R[i][j] = R[i][i] > 0.0 ? s / R[i][i] : 0.0;
    }
  for (int j = 0; j < r; ++j) {                     // its inverse by back substitution
    if (R[j][j] > 0.0) inv[j][j] = 1.0 / R[j][j];
    for (int i = j - 1; i >= 0; --i) {
      double s = 0.0;
      for (int k = i + 1; k <= j; ++k) s += R[i][k] * inv[k][j];
      inv[i][j] = R[i][i] > 0.0 ? -s / R[i][i] : 0.0;
    }
  }
  for (int i = 0; i < n; ++i) {                     // P <- P R^-1
    float v[16];
    for (int c = 0; c < r; ++c) v[c] = P[(size_t)i * r + c];
    for (int c = 0; c < r; ++c) {
      double s = 0.0;
      for (int k = 0; k <= c; ++k) s += (double)v[k] * inv[k][c];
      P[(size_t)i * r + c] = (float)s;
    }
  }

  // ---- Q = M'^T P, published through the second flag pad ----
  float* Q = slot_q(ch.rank);
  std::memset(Q, 0, (size_t)m * r * 4);
  for (int i = 0; i < n; ++i) {
    const float* row = mprime + (size_t)i * m;
    const float* pi = P + (size_t)i * r;
    for (int j = 0; j < m; ++j) {
      const float v = row[j];
      float* qj = Q + (size_t)j * r;
      for (int c = 0; c < r; ++c) qj[c] += v * pi[c];
    }
  }
  for (int p = 0; p < ch.world; ++p)
    store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + a.ready2_off) + ch.rank, a.seq);
  const uint64_t* ready2 = reinterpret_cast<const uint64_t*>(mine + a.ready2_off);
  for (int p = 0; p < ch.world; ++p)
    if (!wait_flag_ge(ready2 + p, a.seq, ch.timeout_ns, st, kTimeoutPeerReady, (unsigned)p)) return st.code();
  for (size_t i = 0; i < (size_t)m * r; ++i) {
    float s = 0.f;
    for (int p = 0; p < ch.world; ++p) s += slot_q(p)[i];
    a.q[i] = s * inv_world;                          // also the start of the next step
  }
  for (int p = 0; p < ch.world; ++p)                 // both regions of every slot of this sequence have been read
    if (p != ch.rank) store_release(reinterpret_cast<uint64_t*>(ch.heap[p] + ch.ack_off) + ch.rank, a.seq);

  // ---- out = P Q^T, residual = M' - out ----
  for (int i = 0; i < n; ++i) {
    const float* pi = P + (size_t)i * r;
    for (int j = 0; j < m; ++j) {
      const float* qj = a.q + (size_t)j * r;
      float o = 0.f;
      for (int c = 0; c < r; ++c) o += pi[c] * qj[c];
      const size_t at = (size_t)i * m + j;
      if (a.acc) a.acc[at] = a.acc[at] - o;          // M' lives in acc
      a.out[at] = o;
    }
  }
  return kOk;
}

void* heap_create(const char* name, size_t bytes) {
  const int fd = shm_open(name, O_CREAT | O_RDWR | O_TRUNC, 0600);
  if (fd < 0) return nullptr;
  if (ftruncate(fd, (off_t)bytes) != 0) {
    close(fd);
    shm_unlink(name);
    return nullptr;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    shm_unlink(name);
    return nullptr;
  }
  return p;   // a fresh shared-memory object reads as zeros
}

void* heap_open(const char* name, size_t bytes) {
  const int fd = shm_open(name, O_RDWR, 0600);
  if (fd < 0) return nullptr;
  struct stat sb;
  if (fstat(fd, &sb) != 0 || (size_t)sb.st_size < bytes) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  return p == MAP_FAILED ? nullptr : p;
}

int heap_close(void* base, size_t bytes) { return munmap(base, bytes); }
int heap_unlink(const char* name) { return shm_unlink(name); }

}  // namespace host
}  // namespace grace
