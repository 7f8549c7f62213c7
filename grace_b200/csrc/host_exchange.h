// Host engine of the exchange protocol: the state machine of the fused GPU
// kernels (sequence-numbered ready / ack flags, two send slots keyed by
// sequence parity, bounded waits that end in a status block) run by CPU ranks
// over POSIX shared memory.  Every rank owns one shared-memory segment that all
// other ranks of the host map, so "heap[r] + offset" addresses any rank's flags
// and slots exactly as the kernels address the peers' device heaps.
//
// It serves CPU tensors behind the same communicator API, and it lets the
// protocol (slot reuse, late or missing peers, recovery) be exercised among
// real concurrent ranks - processes or threads - without a GPU.
// The reference has no counterpart: its CPU ranks only meet inside Gloo calls
// (grace_dl/dist/communicator/allgather.py:8-45).
#pragma once
#include <cstddef>
#include <cstdint>

namespace grace {
namespace host {

constexpr int kMaxWorld = 16;
constexpr size_t kSlotHeaderBytes = 64;   // [0] u64 entry count, [8] f32 scalar, [12] f32 scalar, [16] f64 sum of squares (clipping)

enum Codec : int {
  kTopK = 0,        // k largest magnitudes (ties: lowest index), values + int32 indices
  kThreshold = 1,   // |x| >= threshold (strict: >), at most `cap` entries, the rest stays in the residual
  kQSGD = 2,        // int8 levels + one fp32 norm per 128 elements, Philox stochastic rounding
  kSign = 3,        // 1 bit per element, majority vote (ties -> +1)
  kEFSign = 4,      // 1 bit per element + mean |x|, sum of mean * sign divided by lr
  kDense = 5,       // no compression: sum of the ranks' tensors
  kTernGrad = 6,    // {-1, 0, +1} codes (one byte each) + scale min(max|x|, 2.5 sigma), Philox keep probability |x| / scale
  kNatural = 7,     // 8-bit sign / exponent code, exponent rounded up with probability mantissa / 2^23 (or at 1/2)
  kU8bit = 8,       // 8-bit table code (128 non-uniform bin edges) + scale max|x|
  kOneBit = 9,      // 1 bit per element (x < 0) + the means of the negative and of the other elements
  kFP16 = 10,       // half-precision values, summed in fp32
  kQSGDX = 12,      // QSGD with any bucket size and up to 32767 levels: int16 codes + one fp32 norm per bucket
  kRandomK = 11,    // k positions drawn with replacement from Philox(seed, step), the same on every rank: only values travel
};

enum Phase : int { kCompress = 1, kPublish = 2, kExchange = 4, kAll = 7 };

// Same codes as the device status block (common.cuh).
enum Code : unsigned { kOk = 0, kTimeoutPeerReady = 2, kTimeoutPeerAck = 3, kSlotOverflow = 4, kBadArgument = 5 };

// Where a channel lives inside every rank's heap (identical offsets on all ranks).
struct Channel {
  int rank, world;
  char* heap[kMaxWorld];
  uint64_t ready_off;    // u64[kMaxWorld]: ready[p] = last sequence rank p published to me
  uint64_t ack_off;      // u64[kMaxWorld]: ack[p]   = last sequence rank p finished reading from me
  uint64_t status_off;   // unsigned[8]: code, detail, seq (first error wins)
  uint64_t slot_off[2];  // send slots, used alternately (sequence parity)
  uint64_t slot_bytes;
  uint64_t timeout_ns;
};

struct Args {
  int codec, phases;
  uint64_t seq;          // 1, 2, 3, ... identical on all ranks
  const float* g;        // gradient [n]
  float* acc;            // error-feedback accumulator [n] or null
  float* mom;            // signum momentum [n] or null
  float* u;              // DGC momentum correction [n] or null: u = momentum * u + g, acc += u, both zeroed at the picks
  float momentum;        // DGC
  int deterministic;     // kNatural: round the exponent at mantissa 1/2 instead of drawing
  float* out;            // aggregate [n] (may alias g)
  long long n;
  long long k;           // kTopK: entries; kThreshold: slot capacity
  float beta, gamma;     // acc = beta * acc + gamma * g
  float scale;           // multiplies the sum (1 / W for averaging codecs)
  float threshold;
  int strict;            // kThreshold: > instead of >=
  float lr;              // kEFSign
  float mom_beta;        // kSign with momentum
  int first_step;
  int quantum;           // kQSGD levels (< 128); kQSGDX levels (< 32768)
  int bucket;            // kQSGDX: elements per bucket
  // Two-phase mode (the reference's AllToAll communicator, communicator/all_to_all.py:29-124: compressed
  // reduce-scatter, re-encode, compressed all-gather; kQSGD, kNatural, kFP16, kDense): rank j sums chunk j of all
  // ranks' payloads, encodes the sum again (Philox stream 1) into the second region of its slot and publishes it
  // through the flag pad at ready2_off; every rank then decodes the W chunks.  0 = one-phase (all-gather) mode.
  uint64_t ready2_off;
  // DGC gradient clipping (memory/dgc.py:16-19 of the Horovod flavour): every rank publishes the sum of squares of
  // its gradient (in its slot header, through the flag pad at clip_ready_off) BEFORE anything is encoded; the
  // gradient is then clamped element-wise to +-sqrt(mean over ranks of the sums).  0 = no clipping.
  uint64_t clip_ready_off;
  uint64_t seed;
  unsigned step;
};

// PowerSGD (compressor/powersgd.py:21-65 and memory/powersgd.py:12-37 of the reference) for one matrix: P = M' Q with
// M' = g + residual, mean of P over the ranks, orthogonalisation (Cholesky factor of P^T P in fp64: what modified
// Gram-Schmidt computes in exact arithmetic; a dependent direction is dropped), Q = M'^T P, mean of Q over the ranks
// (kept as the next step's start), out = P Q^T, residual = M' - out.  Two rendezvous per exchange: the slot holds
// P [rows x rank] followed by Q [cols x rank]; the second one uses the flag pad at ready2_off.
struct LowRankArgs {
  int phases;            // kCompress | kPublish: up to the publication of P; kExchange: everything after it
  uint64_t seq;
  const float* g;        // [rows x cols], row-major
  float* acc;            // residual [rows x cols] or null (no error feedback); holds M' between the two phases
  float* out;            // [rows x cols] (may alias g)
  float* q;              // [cols x rank]: start of this step in, mean Q out
  float* p_work;         // [rows x rank] scratch that survives between the phases (the orthogonalised P)
  int rows, cols, rank;
  uint64_t ready2_off;
  // DGC gradient clipping (memory/dgc.py:16-19 of the Horovod flavour): every rank publishes the sum of squares of
  // its gradient (in its slot header, through the flag pad at clip_ready_off) BEFORE anything is encoded; the
  // gradient is then clamped element-wise to +-sqrt(mean over ranks of the sums).  0 = no clipping.
  uint64_t clip_ready_off;   // u64[kMaxWorld] in every heap
};
size_t lowrank_slot_bytes(int rows, int cols, int rank);
unsigned lowrank_exchange(const Channel& ch, const LowRankArgs& args);

size_t slot_bytes(int codec, long long n, long long k);
size_t two_phase_slot_bytes(int codec, long long n, int world);   // both regions

// Runs the phases named by args.phases; returns the status code (0 = ok).  On a timeout the code, the peer and
// the sequence number are also left in the status words of this rank's heap.
unsigned exchange(const Channel& ch, const Args& args);

// Shared-memory segments.  create() makes (or truncates) and maps the segment `name`, zero filled; open() maps an
// existing one of at least `bytes`; both return nullptr on failure with errno set.
void* heap_create(const char* name, size_t bytes);
void* heap_open(const char* name, size_t bytes);
int heap_close(void* base, size_t bytes);
int heap_unlink(const char* name);

}  // namespace host
}  // namespace grace
