// Python bindings (pybind11, no torch headers): kernels take raw device
// pointers that the Python side obtains from tensor.data_ptr(), so this file
// compiles in a few seconds and the extension has no ABI tie to libtorch.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cerrno>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "exchange.h"
#include "host_exchange.h"
#include "runtime.h"

namespace py = pybind11;
using namespace grace;

namespace {

template <class T> T* ptr(uintptr_t p) { return reinterpret_cast<T*>(p); }

void check(cudaError_t err, const char* what) {
  if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

PeerTable make_peers(int rank, int world, unsigned long long seq, unsigned long long timeout_ns,
                     const std::vector<uintptr_t>& heaps, unsigned long long ready_off, unsigned long long ack_off,
                     unsigned long long slot_off, unsigned long long slot_bytes = ~0ull) {
  if (world < 1 || world > kMaxWorldH || (int)heaps.size() != world || rank < 0 || rank >= world)
    throw std::invalid_argument("bad rank/world/heap table");
  PeerTable t{};
  t.rank = rank; t.world = world; t.seq = seq; t.timeout_ns = timeout_ns;
  for (int i = 0; i < world; ++i) t.heap[i] = reinterpret_cast<char*>(heaps[i]);
  t.ready_off = ready_off; t.ack_off = ack_off; t.slot_off = slot_off; t.slot_bytes = slot_bytes;
  return t;
}

}  // namespace

#ifndef GRACE_MODULE_NAME
#define GRACE_MODULE_NAME _C
#endif

PYBIND11_MODULE(GRACE_MODULE_NAME, m) {
#ifdef GRACE_CHECKED
  m.attr("CHECKED") = true;
#else
  m.attr("CHECKED") = false;
#endif
  m.doc() = "grace_b200 native kernels and runtime (sm_100a)";

  // ---- symmetric heap ----
  m.def("heap_alloc", [](size_t bytes) {
    void* p = nullptr;
    check(symm_alloc(&p, bytes), "heap_alloc");
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("heap_free", [](uintptr_t p) { check(symm_free(ptr<void>(p)), "heap_free"); });
  m.def("heap_export", [](uintptr_t p) {
    char handle[kIpcHandleBytes];
    check(symm_export(ptr<void>(p), handle), "heap_export");
    return py::bytes(handle, kIpcHandleBytes);
  });
  m.def("heap_import", [](const std::string& handle) {
    if (handle.size() != kIpcHandleBytes) throw std::invalid_argument("bad ipc handle size");
    void* p = nullptr;
    check(symm_import(handle.data(), &p), "heap_import");
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("heap_release", [](uintptr_t p) { check(symm_release(ptr<void>(p)), "heap_release"); });
  m.def("enable_peer_access", [](int peer_device) { check(symm_enable_peer(peer_device), "enable_peer_access"); });
  m.def("memset_async", [](uintptr_t p, int value, size_t bytes, uintptr_t stream) {
    check(cudaMemsetAsync(ptr<void>(p), value, bytes, reinterpret_cast<cudaStream_t>(stream)), "memset_async");
  });

  // ---- events (plain CUDA events: recording one costs a microsecond; the framework's event objects cost ten) ----
  m.def("event_create", []() {
    cudaEvent_t e = nullptr;
    check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event_create");
    return reinterpret_cast<uintptr_t>(e);
  });
  m.def("event_record", [](uintptr_t e, uintptr_t stream) {
    check(cudaEventRecord(reinterpret_cast<cudaEvent_t>(e), reinterpret_cast<cudaStream_t>(stream)), "event_record");
  });
  m.def("event_query", [](uintptr_t e) {
    const cudaError_t r = cudaEventQuery(reinterpret_cast<cudaEvent_t>(e));
    if (r == cudaErrorNotReady) {
      cudaGetLastError();   // "not ready" is an answer, not an error: it must not linger as the thread's last error
      return false;
    }
    check(r, "event_query");
    return true;
  });
  m.def("event_synchronize", [](uintptr_t e) {
    py::gil_scoped_release release;
    check(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(e)), "event_synchronize");
  });
  m.def("event_destroy", [](uintptr_t e) { cudaEventDestroy(reinterpret_cast<cudaEvent_t>(e)); });

  // ---- sizes / occupancy ----
  m.def("sparse_slot_bytes", &sparse_slot_bytes, pybind11::arg("cap"), pybind11::arg("tiled_total") = 0);
  m.def("sparse_max_grid", &sparse_max_grid);
  m.def("quant_slot_bytes", &quant_slot_bytes, py::arg("codec"), py::arg("total"), py::arg("nseg"), py::arg("alltoall_world") = 0,
        py::arg("nbuckets") = 0);
  m.def("quant_max_grid", &quant_max_grid);
  m.def("sgd_table_chunk", &sgd_table_chunk);
  m.attr("SEGMENT_BYTES") = sizeof(Segment);
  m.attr("SPARSE_STATE_BYTES") = sizeof(SparseState);
  m.attr("QUANT_STATS_BYTES") = sizeof(QuantSegStats);
  m.attr("SGD_TENSOR_BYTES") = sizeof(SgdTensor);
  m.attr("MAX_WORLD") = (int)kMaxWorldH;
  m.attr("PIPE_MAX_CHUNKS") = (int)kPipeMaxChunks;

  // ---- fused sparse exchange ----
  m.def("sparse_exchange",
        [](uintptr_t g, uintptr_t acc, uintptr_t u, uintptr_t out, uintptr_t segs, int nseg, long long total, int mode,
           int levels, float beta, float gamma, float momentum, float threshold, float scale, uintptr_t hist,
           uintptr_t state, uintptr_t barrier, uintptr_t status, unsigned cap, int phases, int rank, int world,
           unsigned long long seq, unsigned long long timeout_ns, const std::vector<uintptr_t>& heaps,
           unsigned long long ready_off, unsigned long long ack_off, unsigned long long slot_off, int grid,
           uintptr_t stream, uintptr_t cand_val, uintptr_t cand_idx, unsigned cand_cap, uintptr_t kprefix,
           uintptr_t seg_seed, unsigned rk_step, unsigned long long clip_off, unsigned long long clip_ready_off,
           uintptr_t clip_sq, int strict, int g_dtype, uintptr_t tile_start, uintptr_t tile_cur, uintptr_t scan_tmp,
           unsigned long long slot_bytes, int fine_hint) {
          SparseArgs a{};
          a.fine_hint = fine_hint;
          a.tile_start = ptr<unsigned>(tile_start); a.tile_cur = ptr<unsigned>(tile_cur); a.scan_tmp = ptr<unsigned>(scan_tmp);
          a.clip_off = clip_off; a.clip_ready_off = clip_ready_off; a.clip_sq = ptr<double>(clip_sq); a.strict = strict;
          if (g_dtype < 0 || g_dtype > 2) throw std::invalid_argument("g_dtype: 0 fp32, 1 bf16, 2 fp16");
          a.g_dtype = g_dtype;
          if ((clip_off != 0) != (clip_sq != 0)) throw std::invalid_argument("clipping needs both the heap area and the accumulators");
          a.kprefix = ptr<const int>(kprefix); a.seg_seed = ptr<const unsigned long long>(seg_seed); a.rk_step = rk_step;
          if (mode == kSparseRandomK && (!kprefix || !seg_seed)) throw std::invalid_argument("random-k needs kprefix and seeds");
          a.cand_val = ptr<float>(cand_val); a.cand_idx = ptr<int>(cand_idx); a.cand_cap = cand_val ? cand_cap : 0;
          a.g = ptr<const void>(g); a.acc = ptr<float>(acc); a.u = ptr<float>(u); a.out = ptr<float>(out);
          a.segs = ptr<const Segment>(segs); a.nseg = nseg; a.total = total; a.mode = mode; a.levels = levels;
          a.beta = beta; a.gamma = gamma; a.momentum = momentum; a.threshold = threshold; a.scale = scale;
          a.hist = ptr<unsigned>(hist); a.state = ptr<SparseState>(state); a.barrier = ptr<unsigned>(barrier);
          a.status = ptr<unsigned>(status); a.cap = cap; a.phases = phases;
          a.peers = make_peers(rank, world, seq, timeout_ns, heaps, ready_off, ack_off, slot_off, slot_bytes);
          if (total % 128 != 0 || cap % 16 != 0) throw std::invalid_argument("total %128 / cap %16");
          check(launch_sparse_exchange(a, grid, reinterpret_cast<cudaStream_t>(stream)), "sparse_exchange");
        });

  // ---- fused quantised exchange ----
  m.def("quant_exchange",
        [](uintptr_t g, uintptr_t acc, uintptr_t mom, uintptr_t out, uintptr_t segs, int nseg, long long total,
           int codec, int quantum, int deterministic, int first_step, float beta, float gamma, float mom_beta, float lr,
           float scale, unsigned long long seed, unsigned step, uintptr_t stats, uintptr_t barrier, uintptr_t status,
           int phases, int rank, int world, unsigned long long seq, unsigned long long timeout_ns,
           const std::vector<uintptr_t>& heaps, unsigned long long ready_off, unsigned long long ack_off,
           unsigned long long slot_off, int grid, uintptr_t stream, int alltoall, unsigned long long ready2_off,
           uintptr_t recv_local, uintptr_t recv_mc, unsigned long long recv_stride, int g_dtype, int qsgd_bucket,
           long long qsgd_nbuckets, unsigned long long slot_bytes, uintptr_t pipe, unsigned long long chunk_ready_off,
           int pipe_chunks, int pipe_chunk_items, int pipe_item_elems) {
          QuantArgs a{};
          a.pipe = ptr<unsigned>(pipe); a.chunk_ready_off = chunk_ready_off; a.pipe_chunks = pipe_chunks;
          a.pipe_chunk_items = pipe_chunk_items; a.pipe_item_elems = pipe_item_elems;
          a.qsgd_bucket = qsgd_bucket; a.qsgd_nbuckets = qsgd_nbuckets;
          if (g_dtype < 0 || g_dtype > 2) throw std::invalid_argument("g_dtype: 0 fp32, 1 bf16, 2 fp16");
          a.g_dtype = g_dtype;
          a.recv_local = ptr<char>(recv_local); a.recv_mc = ptr<char>(recv_mc); a.recv_stride = recv_stride;
          if ((recv_local != 0) != (recv_mc != 0) || (recv_mc && (alltoall || recv_stride % 16 || recv_local % 16 || recv_mc % 16)))
            throw std::invalid_argument("quant_exchange: bad push-transport arguments");
          a.alltoall = alltoall; a.ready2_off = ready2_off;
          a.g = ptr<const void>(g); a.acc = ptr<float>(acc); a.mom = ptr<float>(mom); a.out = ptr<void>(out);
          a.segs = ptr<const Segment>(segs); a.nseg = nseg; a.total = total; a.codec = codec; a.quantum = quantum;
          a.deterministic = deterministic; a.first_step = first_step; a.beta = beta; a.gamma = gamma;
          a.mom_beta = mom_beta; a.lr = lr; a.scale = scale; a.seed = seed; a.step = step;
          a.stats = ptr<QuantSegStats>(stats); a.barrier = ptr<unsigned>(barrier); a.status = ptr<unsigned>(status);
          a.phases = phases;
          a.peers = make_peers(rank, world, seq, timeout_ns, heaps, ready_off, ack_off, slot_off, slot_bytes);
          if (total % 128 != 0) throw std::invalid_argument("total must be a multiple of 128");
          if (pipe_chunks > 0)
            check(launch_quant_pipeline(a, grid, reinterpret_cast<cudaStream_t>(stream)), "quant_exchange (pipelined)");
          else
            check(launch_quant_exchange(a, grid, reinterpret_cast<cudaStream_t>(stream)), "quant_exchange");
        });

  // ---- dense all-reduce over the NVSwitch multicast mapping ----
  m.def("dense_max_grid", &dense_max_grid);
  m.def("dense_allreduce",
        [](uintptr_t g, uintptr_t out, uintptr_t symm, uintptr_t mc, long long total, float scale, uintptr_t barrier,
           uintptr_t status, unsigned long long ready2_off, int rank, int world, unsigned long long seq,
           unsigned long long timeout_ns, const std::vector<uintptr_t>& heaps, unsigned long long ready_off,
           unsigned long long ack_off, int grid, uintptr_t stream) {
          DenseArgs a{};
          a.g = ptr<const float>(g); a.out = ptr<float>(out); a.symm = ptr<float>(symm); a.mc = ptr<float>(mc);
          a.total = total; a.scale = scale; a.barrier = ptr<unsigned>(barrier); a.status = ptr<unsigned>(status);
          a.ready2_off = ready2_off;
          a.peers = make_peers(rank, world, seq, timeout_ns, heaps, ready_off, ack_off, 0);
          if ((g | out | symm | mc) % 16 != 0) throw std::invalid_argument("dense_allreduce: pointers must be 16-byte aligned");
          check(launch_dense_allreduce(a, grid, reinterpret_cast<cudaStream_t>(stream)), "dense_allreduce");
        });

  // ---- fused PowerSGD (tcgen05) ----
  m.def("lowrank_smem_bytes", &lowrank_smem_bytes);
  m.def("lowrank_max_grid", &lowrank_max_grid);
  m.def("lowrank_occupancy", &lowrank_occupancy);
  m.attr("LOWRANK_MATRIX_BYTES") = sizeof(LowRankMatrix);
  m.attr("TENSOR_MAP_BYTES") = 128;
  m.attr("MAPS_PER_MATRIX") = (int)kMapsPerMatrix;
  m.def("lowrank_encode_maps", [](uintptr_t host_out, uintptr_t g, uintptr_t acc, uintptr_t qt, uintptr_t pt, int n, int mm) {
    const int rc = lowrank_encode_maps(ptr<void>(host_out), ptr<const float>(g), ptr<float>(acc), ptr<const float>(qt),
                                       ptr<const float>(pt), n, mm);
    if (rc != 0) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(rc));
  });
  m.def("powersgd_exchange",
        [](uintptr_t g, uintptr_t acc, uintptr_t out, uintptr_t mats, uintptr_t maps, int nmat, int rank_r,
           int has_memory, int divisor, int items_s1, int items_s2, int p_floats, int q_floats, uintptr_t p_mean,
           uintptr_t q_mean, uintptr_t pt_orth, uintptr_t qt, uintptr_t gram, uintptr_t partial,
           uintptr_t barrier, uintptr_t status,
           unsigned long long ready2_off, int part, int rank, int world, unsigned long long seq,
           unsigned long long timeout_ns, const std::vector<uintptr_t>& heaps, unsigned long long ready_off,
           unsigned long long ack_off, unsigned long long slot_off, int grid, uintptr_t stream) {
          LowRankArgs a{};
          a.g = ptr<const float>(g); a.acc = ptr<float>(acc); a.out = ptr<float>(out);
          a.mats = ptr<const LowRankMatrix>(mats); a.maps = ptr<const CUtensorMap_st>(maps); a.nmat = nmat;
          a.rank = rank_r; a.has_memory = has_memory; a.divisor = divisor; a.items_s1 = items_s1; a.items_s2 = items_s2;
          a.p_floats = p_floats; a.q_floats = q_floats; a.p_mean = ptr<float>(p_mean); a.q_mean = ptr<float>(q_mean);
          a.pt_orth = ptr<float>(pt_orth); a.qt = ptr<float>(qt); a.gram_part = ptr<double>(gram);
          a.partial = ptr<float>(partial);
          if (!partial) throw std::invalid_argument("powersgd_exchange: split-K scratch missing");
          a.barrier = ptr<unsigned>(barrier); a.status = ptr<unsigned>(status); a.ready2_off = ready2_off;
          a.phases = kPhaseAll; a.part = part;
          a.peers = make_peers(rank, world, seq, timeout_ns, heaps, ready_off, ack_off, slot_off);
          if (rank_r < 1 || rank_r > 16 || nmat < 1) throw std::invalid_argument("rank must be in [1,16], nmat >= 1");
          if (part < 0 || part > 3) throw std::invalid_argument("part: 0 (all) or 1..3");
          check(launch_powersgd(a, grid, reinterpret_cast<cudaStream_t>(stream)), "powersgd_exchange");
        });

  // ---- stand-alone error-feedback kernels (library path) ----
  m.def("residual_compensate", [](uintptr_t g, int g_dtype, uintptr_t r, uintptr_t out, long long n, float beta, float gamma,
                                  uintptr_t stream) {
    check(launch_residual_compensate(ptr<const void>(g), g_dtype, ptr<const float>(r), ptr<float>(out), n, beta, gamma,
                                     reinterpret_cast<cudaStream_t>(stream)), "residual_compensate");
  });
  m.def("residual_update", [](uintptr_t acc, uintptr_t dec, uintptr_t r, long long n, uintptr_t stream) {
    check(launch_residual_update(ptr<const float>(acc), ptr<const float>(dec), ptr<float>(r), n,
                                 reinterpret_cast<cudaStream_t>(stream)), "residual_update");
  });
  m.def("zero_at", [](uintptr_t a, uintptr_t b, uintptr_t idx, int idx64, long long k, long long n, uintptr_t stream) {
    check(launch_zero_at(ptr<float>(a), ptr<float>(b), ptr<const void>(idx), idx64, k, n,
                         reinterpret_cast<cudaStream_t>(stream)), "zero_at");
  });
  m.def("dgc_compensate", [](uintptr_t g, int g_dtype, uintptr_t u, uintptr_t v, long long n, float momentum, float bound,
                             int first, uintptr_t stream) {
    check(launch_dgc_compensate(ptr<const void>(g), g_dtype, ptr<float>(u), ptr<float>(v), n, momentum, bound, first,
                                reinterpret_cast<cudaStream_t>(stream)), "dgc_compensate");
  });
  m.def("dgc_mask", [](uintptr_t u, uintptr_t v, uintptr_t mask, long long n, uintptr_t stream) {
    check(launch_dgc_mask(ptr<float>(u), ptr<float>(v), ptr<const unsigned char>(mask), n,
                          reinterpret_cast<cudaStream_t>(stream)), "dgc_mask");
  });
  m.def("sum_squares_scratch_doubles", &sum_squares_scratch_doubles);
  m.def("sum_squares", [](uintptr_t g, int g_dtype, long long n, uintptr_t scratch, uintptr_t stream) {
    check(launch_sum_squares(ptr<const void>(g), g_dtype, n, ptr<double>(scratch), reinterpret_cast<cudaStream_t>(stream)),
          "sum_squares");
  });

  // ---- fused SGD ----
  m.def("fused_sgd", [](uintptr_t p, uintptr_t g, uintptr_t buf, long long numel, float lr, float momentum,
                        float dampening, float weight_decay, int nesterov, int first_step, int zero_grad,
                        float grad_scale, uintptr_t stream) {
    check(launch_fused_sgd(ptr<float>(p), ptr<float>(g), ptr<float>(buf), numel, lr, momentum, dampening, weight_decay,
                           nesterov, first_step, zero_grad, grad_scale, reinterpret_cast<cudaStream_t>(stream)),
          "fused_sgd");
  });
  m.def("multi_sgd", [](uintptr_t table, uintptr_t blocks, int nblocks, float lr, float momentum, float dampening,
                        float weight_decay, int nesterov, int first_step, int zero_grad, float grad_scale,
                        uintptr_t stream) {
    check(launch_multi_sgd(ptr<const SgdTensor>(table), ptr<const int>(blocks), nblocks, lr, momentum, dampening,
                           weight_decay, nesterov, first_step, zero_grad, grad_scale,
                           reinterpret_cast<cudaStream_t>(stream)),
          "multi_sgd");
  });

  // ---- host engine of the exchange protocol (CPU ranks over POSIX shared memory) ----
  m.attr("HOST_MAX_WORLD") = host::kMaxWorld;
  m.def("host_heap_create", [](const std::string& name, size_t bytes) {
    void* p = host::heap_create(name.c_str(), bytes);
    if (!p) throw std::runtime_error("host_heap_create(" + name + "): " + std::strerror(errno));
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("host_heap_open", [](const std::string& name, size_t bytes) {
    void* p = host::heap_open(name.c_str(), bytes);
    if (!p) throw std::runtime_error("host_heap_open(" + name + "): " + std::strerror(errno));
    return reinterpret_cast<uintptr_t>(p);
  });
  m.def("host_heap_close", [](uintptr_t base, size_t bytes) { return host::heap_close(ptr<void>(base), bytes); });
  m.def("host_heap_unlink", [](const std::string& name) { return host::heap_unlink(name.c_str()); });
  m.def("host_slot_bytes", &host::slot_bytes);
  m.def("host_two_phase_slot_bytes", &host::two_phase_slot_bytes);
  m.def("host_lowrank_slot_bytes", &host::lowrank_slot_bytes);
  m.def("host_lowrank_exchange",
        [](int rank, int world, const std::vector<uintptr_t>& heaps, unsigned long long ready_off,
           unsigned long long ack_off, unsigned long long status_off, unsigned long long slot0_off,
           unsigned long long slot1_off, unsigned long long slot_bytes, unsigned long long timeout_ns,
           unsigned long long ready2_off, int phases, unsigned long long seq, uintptr_t g, uintptr_t acc, uintptr_t out,
           uintptr_t q, uintptr_t p_work, int rows, int cols, int lr_rank) {
          if (world < 1 || world > host::kMaxWorld || (int)heaps.size() != world || rank < 0 || rank >= world)
            throw std::invalid_argument("bad rank/world/heap table");
          host::Channel ch{};
          ch.rank = rank; ch.world = world;
          for (int i = 0; i < world; ++i) ch.heap[i] = reinterpret_cast<char*>(heaps[i]);
          ch.ready_off = ready_off; ch.ack_off = ack_off; ch.status_off = status_off;
          ch.slot_off[0] = slot0_off; ch.slot_off[1] = slot1_off; ch.slot_bytes = slot_bytes; ch.timeout_ns = timeout_ns;
          host::LowRankArgs a{};
          a.phases = phases; a.seq = seq; a.g = ptr<const float>(g); a.acc = ptr<float>(acc); a.out = ptr<float>(out);
          a.q = ptr<float>(q); a.p_work = ptr<float>(p_work); a.rows = rows; a.cols = cols; a.rank = lr_rank;
          a.ready2_off = ready2_off;
          unsigned rc;
          {
            py::gil_scoped_release release;
            rc = host::lowrank_exchange(ch, a);
          }
          return rc;
        });
  m.def("host_exchange",
        [](int rank, int world, const std::vector<uintptr_t>& heaps, unsigned long long ready_off,
           unsigned long long ack_off, unsigned long long status_off, unsigned long long slot0_off,
           unsigned long long slot1_off, unsigned long long slot_bytes, unsigned long long timeout_ns, int codec,
           int phases, unsigned long long seq, uintptr_t g, uintptr_t acc, uintptr_t mom, uintptr_t out, long long n,
           long long k, float beta, float gamma, float scale, float threshold, int strict, float lr, float mom_beta,
           int first_step, int quantum, unsigned long long seed, unsigned step, uintptr_t u, float momentum,
           int deterministic, int bucket, unsigned long long ready2_off, unsigned long long clip_ready_off) {
          if (world < 1 || world > host::kMaxWorld || (int)heaps.size() != world || rank < 0 || rank >= world)
            throw std::invalid_argument("bad rank/world/heap table");
          host::Channel ch{};
          ch.rank = rank; ch.world = world;
          for (int i = 0; i < world; ++i) ch.heap[i] = reinterpret_cast<char*>(heaps[i]);
          ch.ready_off = ready_off; ch.ack_off = ack_off; ch.status_off = status_off;
          ch.slot_off[0] = slot0_off; ch.slot_off[1] = slot1_off; ch.slot_bytes = slot_bytes; ch.timeout_ns = timeout_ns;
          host::Args a{};
          a.codec = codec; a.phases = phases; a.seq = seq;
          a.g = ptr<const float>(g); a.acc = ptr<float>(acc); a.mom = ptr<float>(mom); a.out = ptr<float>(out);
          a.n = n; a.k = k; a.beta = beta; a.gamma = gamma; a.scale = scale; a.threshold = threshold; a.strict = strict;
          a.lr = lr; a.mom_beta = mom_beta; a.first_step = first_step; a.quantum = quantum; a.seed = seed; a.step = step;
          a.u = ptr<float>(u); a.momentum = momentum; a.deterministic = deterministic; a.bucket = bucket; a.ready2_off = ready2_off; a.clip_ready_off = clip_ready_off;
          unsigned rc;
          {
            py::gil_scoped_release release;   // ranks of a test may be threads of one process
            rc = host::exchange(ch, a);
          }
          return rc;
        });
}
