// Host/device shared argument blocks and launcher declarations for the fused
// gradient-exchange kernels.  No torch headers here: the .cu files compile in
// seconds and are linked into the extension by bindings.cpp.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace grace {

constexpr int kMaxWorldH = 16;

// One named gradient inside a flat buffer.  `offset` (in elements) must be a
// multiple of 128 so that 16-byte vector accesses and 128-element code groups
// never straddle two tensors.
struct Segment {
  long long offset;
  int numel;
  int k;  // number of elements to keep (TopK / DGC); unused otherwise
};

// Where the other ranks are.  heap[r] is rank r's symmetric heap mapped into
// this process (heap[rank] is the local one).  All offsets are identical on
// every rank.  `ready`/`ack` are arrays of kMaxWorldH uint64 flags:
//   ready[p] on rank r = last sequence number whose send slot rank p published,
//   ack[p]   on rank r = last sequence number rank p finished reading from r.
// Send slots are double buffered by sequence parity; slot_off already selects
// the parity of `seq`.
struct PeerTable {
  int rank;
  int world;
  unsigned long long seq;
  unsigned long long timeout_ns;
  char* heap[kMaxWorldH];
  unsigned long long ready_off;
  unsigned long long ack_off;
  unsigned long long slot_off;
  unsigned long long slot_bytes;   // size of one send slot (bounds of the checked build)
};

enum Phase : int {
  kPhaseCompress = 1,  // compensate + encode into the local send slot
  kPhasePublish = 2,   // release the slot to the peers
  kPhaseExchange = 4,  // wait for peers, pull, decode, aggregate, acknowledge
  kPhaseAll = 7,
  kPhaseReduce = 8,    // two-phase ("alltoall") mode only: reduce my chunk, re-encode, publish again
  kPhaseClip = 16,     // sparse exchange with DGC gradient clipping: per-tensor sum of squares, published to the peers
};

// ---------------------------------------------------------------- sparse ----
enum SparseMode : int { kSparseTopK = 0, kSparseThreshold = 1, kSparseRandomK = 2 };

struct SparseState {       // per segment, device scratch
  unsigned prefix;         // selected key prefix after each radix level
  unsigned need;           // how many elements to take from the pivot bin
  unsigned tie_taken;      // claimed so far among keys equal to the pivot
  unsigned max_bits;       // ordered-int encoding of max(acc) (threshold mode)
  unsigned pivot_count;    // keys in the pivot bin of the last level done on the histograms
  unsigned fine;           // 1: the first pass already resolved 24 key bits for this segment (hinted histogram)
};

struct SparseArgs {
  const void* g;      // gradients, flat: fp32, bf16 or fp16 (g_dtype, a GradType of gradio.cuh)
  int g_dtype;
  float* acc;         // accumulator / residual state (nullable: no memory)
  float* u;           // DGC momentum state (nullable)
  float* out;         // dense aggregated output; may alias g (nullable)
  const Segment* segs;
  int nseg;
  long long total;    // padded flat length, multiple of 128
  int mode;
  int levels;         // 3 = exact k-th magnitude, 2 = top 24 key bits
  float beta, gamma, momentum, threshold;
  float scale;        // factor applied while aggregating (1/W when averaging)
  unsigned* hist;     // nseg * 4096, zero on entry, left zero on exit
  int fine_hint;      // 1: hist is followed by nseg * 4096 words of second-level histograms (zero between launches)
                      //    and nseg hint words (the previous launch's first-level pivot bin, 0xffffffff = none)
  SparseState* state; // nseg + 1 (the extra entry holds the candidate counters), zeroed by the launcher
  float* cand_val;    // candidate list of the fast select path (nullable)
  int* cand_idx;
  unsigned cand_cap;  // capacity of the candidate list in entries (0 disables the fast path)
  // Random-k: every rank draws the same positions from Philox(seed of the tensor, step), so only values travel.
  const int* kprefix;               // nseg + 1 prefix sums of k (entry e belongs to the segment with kprefix[s] <= e)
  const unsigned long long* seg_seed;  // nseg seeds (derived from the tensor names, identical on every rank)
  unsigned rk_step;                 // per-plan step counter (part of the Philox counter)
  // DGC gradient clipping (0 = off): element-wise clamp of g to +-sqrt(mean over ranks of sum g^2) per tensor.
  unsigned long long clip_off;      // heap offset of 2 (parities) x nseg doubles: this rank's sums, read by the peers
  unsigned long long clip_ready_off;  // flag pad of their publication
  double* clip_sq;                  // nseg local accumulators, zero on entry, left zero on exit
  int strict;                       // threshold mode: |x| > threshold (no cap by max(x))
  // Tile-ordered exchange (nullable: then lists travel unordered and are scatter-added with red.global):
  // the sender orders its list by 8192-element output tile into a second pair of arrays in the slot,
  // followed by a directory of tile offsets; receivers build whole tiles in shared memory.  The slot
  // must then be sized with sparse_slot_bytes(cap, total).  Local scratch of the ordering step:
  unsigned* tile_start;             // tiles + 1 counters / prefix sums
  unsigned* tile_cur;               // tiles running cursors
  unsigned* scan_tmp;               // one word per CTA
  unsigned* barrier;  // one word, zeroed by the launcher
  unsigned* status;   // 4 words
  unsigned cap;       // slot capacity in entries (multiple of 16)
  int phases;
  PeerTable peers;
};

size_t sparse_slot_bytes(unsigned cap, long long tiled_total = 0);
size_t sparse_smem_bytes();
int sparse_max_grid(int device, int sm_limit);
cudaError_t launch_sparse_exchange(const SparseArgs& a, int grid, cudaStream_t stream);
// Single-CTA variant for one tensor of at most 8192 elements (sparse_small.cu): same arguments, phases, flags and
// slot header; needs none of the scratch areas.  launch_sparse_exchange() uses it whenever it applies, unless the
// environment variable GRACE_SMALL_KERNEL is "0".
bool sparse_small_applies(const SparseArgs& a);
cudaError_t launch_sparse_small(const SparseArgs& a, cudaStream_t stream);

// ----------------------------------------------------------------- quant ----
enum Codec : int {
  kCodecQSGD = 0,      // int8 codes + fp32 norm per 128 elements
  kCodecTernGrad = 1,  // 2 bits per element + scale per segment
  kCodecNatural = 2,   // 8-bit sign/exponent code
  kCodecU8bit = 3,     // 8-bit table code + scale per segment
  kCodecSign = 4,      // 1 bit, majority vote (signSGD / signum)
  kCodecEFSign = 5,    // 1 bit + mean |x| per segment, scaled sum / lr
  kCodecOneBit = 6,    // 1 bit + two means per segment
  kCodecFP16 = 7,      // half cast, sum
  kCodecFP32 = 8,      // no compression: one-shot all-gather-sum (small dense tensors)
  kCodecQSGDX = 9,     // QSGD, any bucket size that is a multiple of 4, up to 32767 levels: int16 codes + fp32 norm per bucket
};

struct QuantSegStats {   // per segment, device scratch (double for stable sums)
  double sum, sumsq, sum_neg, sum_pos;
  unsigned long long cnt_neg;
  unsigned maxabs_bits;
  unsigned pad;
};

struct QuantArgs {
  const void* g;       // gradients: fp32, bf16 or fp16 (g_dtype, a GradType of gradio.cuh)
  float* acc;          // residual state (nullable), always fp32
  float* mom;          // signum momentum state (nullable), always fp32
  void* out;           // aggregated gradients, same element type as g; may alias g
  int g_dtype;
  const Segment* segs;
  int nseg;
  long long total;     // padded flat length, multiple of 128
  int codec;
  int quantum;         // QSGD levels
  int qsgd_bucket;     // kCodecQSGDX: elements per bucket (Segment::k = index of the tensor's first bucket)
  long long qsgd_nbuckets;  // kCodecQSGDX: buckets of all tensors together
  int deterministic;   // natural: round at 0.5 instead of drawing
  int first_step;      // signum: momentum not yet initialised
  float beta, gamma;   // acc = beta*residual + gamma*g
  float mom_beta;      // signum
  float lr;            // EF-signSGD aggregate divisor
  float scale;         // 1/W when averaging
  unsigned long long seed;
  unsigned step;
  QuantSegStats* stats;  // nseg, zero on entry, left zero on exit
  unsigned* barrier;
  unsigned* status;
  int phases;
  int alltoall;          // 1: compressed reduce-scatter + compressed all-gather (QSGD, natural, fp16, fp32)
  unsigned long long ready2_off;  // flag pad of the second publication (alltoall mode)
  // Push transport (all-gather mode only; null = peers pull from each other's slots with remote loads):
  // the encode pass stores its codes, norms and scalars with multimem.st into region `rank` of the receive
  // area of EVERY GPU (the NVSwitch replicates the stores), and the decode pass reads local memory only.
  char* recv_local;               // this GPU's receive area of the current parity: world regions of recv_stride bytes
  char* recv_mc;                  // multicast address of the same area
  unsigned long long recv_stride;
  // Pipelined all-gather mode (quant_pipeline_kernel; QSGD with 128-element buckets and natural compression, pull
  // transport, 2..8 ranks): the buffer is cut into chunks of tiles; CTAs take tiles from one queue in which the
  // encode tiles of chunk c + 1 come before the decode tiles of chunk c, and a chunk is published to the peers as
  // soon as its last tile is encoded, so that pulling chunk c over NVLink runs next to encoding chunk c + 1.
  unsigned* pipe;                 // [0] queue head, [1 + c] encoded tiles of chunk c; zeroed by the launcher
  unsigned long long chunk_ready_off;   // kMaxWorldH x kPipeMaxChunks uint64 flags in every heap (value = seq)
  int pipe_chunks;                // 0: not pipelined
  int pipe_chunk_items;           // tiles per chunk (the last chunk may have fewer)
  int pipe_item_elems;            // elements per tile, a multiple of 8192
  PeerTable peers;
};
constexpr int kPipeMaxChunks = 16;

// alltoall_world > 0 adds the second region (one re-encoded chunk per rank) used by the two-phase mode.
size_t quant_slot_bytes(int codec, long long total, int nseg, int alltoall_world = 0, long long nbuckets = 0);
int quant_max_grid(int device, int sm_limit);
cudaError_t launch_quant_exchange(const QuantArgs& a, int grid, cudaStream_t stream);
cudaError_t launch_quant_pipeline(const QuantArgs& a, int grid, cudaStream_t stream);   // pipelined all-gather mode

// ------------------------------------------------------------ dense NVLS ----
// Uncompressed all-reduce over the NVSwitch multicast mapping of a symmetric buffer
// (dense_allreduce.cu).  `symm` is this rank's copy of the buffer, `mc` the multicast
// address of the same buffer; `g` / `out` may equal `symm` (no staging copies then).
struct DenseArgs {
  const float* g;
  float* out;
  float* symm;
  float* mc;
  long long total;                // floats, multiple of 4
  float scale;                    // applied to the sum (1/W for the mean)
  unsigned* barrier;
  unsigned* status;
  unsigned long long ready2_off;  // flag pad of the second rendezvous
  PeerTable peers;
};
int dense_max_grid(int device, int sm_limit);
cudaError_t launch_dense_allreduce(const DenseArgs& a, int grid, cudaStream_t stream);

// -------------------------------------------------------------- low rank ----
// One matrix (n x m, row-major) of a PowerSGD launch.  All offsets in floats.
struct LowRankMatrix {
  long long g_off;   // start of the matrix in the flat gradient / accumulator buffers
  int n, m;
  int p_off;         // row-major [n][16] block inside the P regions
  int q_off;         // row-major [m][16] block inside the Q regions
  int pt_off;        // [16][n] block inside pt_orth
  int qt_off;        // [16][m] block inside qt
  int item1_begin;   // first stage-1 work item (prefix sum over matrices)
  int item2_begin;   // first stage-2 work item
  int splits1;       // K splits per 128-row block in stage 1 (work items of a block are consecutive)
  int splits2;       // same for stage 2
};

enum LowRankMap : int { kMapG1 = 0, kMapA1 = 1, kMapM2 = 2, kMapQt = 3, kMapPt = 4, kMapsPerMatrix = 5 };

struct CUtensorMap_st;

struct LowRankArgs {
  const float* g;          // flat gradients
  float* acc;              // flat accumulator / residual (used when has_memory)
  float* out;              // flat output (may alias g)
  const LowRankMatrix* mats;
  const CUtensorMap_st* maps;  // nmat * kMapsPerMatrix tensor maps in device memory (64-byte aligned)
  int nmat;
  int rank;                // actual rank r <= 16 (buffers are padded to 16 columns)
  int has_memory;
  int divisor;             // world size (P and Q are averaged)
  int items_s1, items_s2;
  int p_floats, q_floats;  // sizes of the P and Q regions (multiples of 4)
  float* p_mean;           // [p_floats]
  float* q_mean;           // [q_floats]
  float* pt_orth;          // sum_n 16*n
  float* qt;               // sum_m 16*m: Q^T, persistent across steps (warm start)
  double* gram_part;       // grid * nmat * 256: one partial Gram matrix per CTA and matrix (added in CTA order)
  float* partial;          // (items_s1 + items_s2) blocks of 128 x 16: split-K partial sums, one block per work item
  unsigned* barrier;
  unsigned* status;
  unsigned long long ready2_off;  // second flag pad (Q); peers.ready_off is the first (P)
  int phases;
  int part;                // 0 = whole exchange; 1, 2, 3 = that part only (one-GPU emulation)
  PeerTable peers;
};

size_t lowrank_smem_bytes();
int lowrank_max_grid(int device, int sm_limit);
int lowrank_occupancy(int dynamic_smem_bytes);
cudaError_t launch_powersgd(const LowRankArgs& a, int grid, cudaStream_t stream);
int lowrank_encode_maps(void* maps_out, const float* g, float* acc, const float* qt, const float* pt, int n, int m);

// ---------------------------------------------------------------- memory ----
// Stand-alone error-feedback kernels of the library path (memory.cu).  g_dtype is a GradType of gradio.cuh.
cudaError_t launch_residual_compensate(const void* g, int g_dtype, const float* r, float* out, long long n, float beta,
                                       float gamma, cudaStream_t stream);   // r nullable: out = gamma * g
cudaError_t launch_residual_update(const float* acc, const float* dec, float* r, long long n, cudaStream_t stream);
cudaError_t launch_zero_at(float* a, float* b, const void* idx, int idx64, long long k, long long n, cudaStream_t stream);
cudaError_t launch_dgc_compensate(const void* g, int g_dtype, float* u, float* v, long long n, float momentum, float bound,
                                  int first, cudaStream_t stream);
cudaError_t launch_dgc_mask(float* u, float* v, const unsigned char* mask, long long n, cudaStream_t stream);
int sum_squares_scratch_doubles();
cudaError_t launch_sum_squares(const void* g, int g_dtype, long long n, double* scratch, cudaStream_t stream);   // result in scratch[0]

// ------------------------------------------------------------------- sgd ----
struct SgdTensor {
  float* p;
  const float* g;
  float* buf;
  int numel;
};
cudaError_t launch_fused_sgd(float* p, float* g, float* buf, long long numel, float lr, float momentum, float dampening,
                             float weight_decay, int nesterov, int first_step, int zero_grad, float grad_scale,
                             cudaStream_t stream);
int sgd_table_chunk();
cudaError_t launch_multi_sgd(const SgdTensor* table, const int* blocks_xy, int nblocks, float lr, float momentum,
                             float dampening, float weight_decay, int nesterov, int first_step, int zero_grad,
                             float grad_scale, cudaStream_t stream);

}  // namespace grace
