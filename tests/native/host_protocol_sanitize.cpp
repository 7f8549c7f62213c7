// Driver for sanitizer builds of the host engine of the exchange protocol (csrc/host_exchange.cpp).
//
// W ranks run as threads of this process over ONE copy of every rank's heap, so ThreadSanitizer sees every
// access of every rank at the same address: the flags are atomic (release / acquire), the slots and the
// error-feedback arrays are plain memory, and a protocol error - a slot rewritten while a peer still reads it, a
// payload read before its flag - shows up as a reported race.  AddressSanitizer / UBSan builds of the same driver
// catch indexing errors in the slot layouts.  Ranks are de-synchronised on purpose (different sleeps per rank and
// step) and the step count makes every slot parity get reused many times.
//
// Build (see tests/test_host_sanitizers_cpu.py):
//   g++ -std=c++17 -O1 -g -fsanitize=thread -I grace_b200/csrc -I <cuda>/include \
//       tests/native/host_protocol_sanitize.cpp grace_b200/csrc/host_exchange.cpp -o drv -lpthread -lrt
// Exit code 0 = every rank got identical, finite results in every step and (in a second scenario) the peer that
// never publishes was reported as a time-out on the waiting rank.
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "host_exchange.h"

using namespace grace::host;

namespace {

struct World {
  int world;
  size_t heap_bytes;
  std::vector<void*> base;
};

// The ranks' heaps are ordinary zeroed allocations here: all threads use the same addresses anyway, and the
// sanitizers track heap memory reliably (a race planted in a MAP_SHARED mapping went unreported).  The
// shared-memory calls themselves are exercised once in main().
void* heap_new(size_t bytes) { return std::calloc(1, bytes); }
void heap_delete(void* p) { std::free(p); }

Channel channel_for(const World& w, int rank, size_t slot_bytes_, uint64_t timeout_ns) {
  Channel ch{};
  ch.rank = rank;
  ch.world = w.world;
  for (int r = 0; r < w.world; ++r) ch.heap[r] = static_cast<char*>(w.base[r]);
  ch.ready_off = 0;
  ch.ack_off = kMaxWorld * 8;                 // the third pad (second rendezvous of the two-phase mode) follows
  ch.status_off = 3 * kMaxWorld * 8;
  ch.slot_off[0] = 3 * kMaxWorld * 8 + 64;
  ch.slot_off[1] = ch.slot_off[0] + slot_bytes_;
  ch.slot_bytes = slot_bytes_;
  ch.timeout_ns = timeout_ns;
  return ch;
}

float pseudo(int rank, int step, long long i) {   // deterministic test gradients, different on every rank
  uint32_t h = (uint32_t)(i * 2654435761u) ^ (uint32_t)(rank * 40503u + step * 9973u + 12345u);
  h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
  return ((float)(h & 0xffffu) / 65536.f - 0.5f) * 2e-3f;
}

int run_codec(int codec, int world, long long n, int steps, bool two_phase = false) {
  const long long k = codec == kTopK ? std::max<long long>(1, n / 50)
                      : (codec == kThreshold ? std::max<long long>(1, n / 4) : (codec == kRandomK ? std::max<long long>(1, n / 20) : 0));
  const size_t sb = two_phase ? two_phase_slot_bytes(codec, n, world) : slot_bytes(codec, n, codec == kQSGDX ? 100 : k);
  World w{world, 3 * kMaxWorld * 8 + 64 + 2 * sb + 256, {}};
  for (int r = 0; r < world; ++r) {
    void* p = heap_new(w.heap_bytes);
    if (!p) return 2;
    w.base.push_back(p);
  }
  std::vector<std::vector<float>> outs(world, std::vector<float>((size_t)n));
  std::vector<int> rc(world, 0);
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r) {
    threads.emplace_back([&, r] {
      const Channel ch = channel_for(w, r, sb, 20ull * 1000000000ull);
      std::vector<float> g((size_t)n), acc((size_t)n, 0.f), mom((size_t)n, 0.f), u((size_t)n, 0.f);
      const bool ef = codec != kSign && codec != kDense;
      for (int s = 0; s < steps; ++s) {
        for (long long i = 0; i < n; ++i) g[(size_t)i] = pseudo(r, s, i);
        if ((r + s) % 3 == 0) std::this_thread::sleep_for(std::chrono::microseconds(300 * (r + 1)));
        Args a{};
        a.codec = codec; a.phases = kAll; a.seq = (uint64_t)s + 1;
        a.g = g.data(); a.acc = ef ? acc.data() : nullptr; a.mom = codec == kSign ? mom.data() : nullptr;
        a.u = codec == kTopK ? u.data() : nullptr; a.out = outs[r].data(); a.n = n; a.k = k;
        a.beta = s == 0 ? 0.f : 1.f; a.gamma = 1.f; a.scale = 1.f / (float)world; a.threshold = 5e-4f; a.strict = 0;
        a.lr = 0.1f; a.mom_beta = 0.9f; a.first_step = s == 0; a.quantum = 64; a.seed = 77; a.step = (unsigned)s;
        a.momentum = 0.f; a.deterministic = 0; a.bucket = 100; a.ready2_off = two_phase ? 2 * kMaxWorld * 8 : 0;
        a.clip_ready_off = codec == kTopK ? 2 * kMaxWorld * 8 : 0;   // DGC memory with gradient clipping
        a.momentum = 0.9f;
        // split phases on odd steps: publish first, pull later (what send_step / receive_step do)
        unsigned code;
        if (s & 1) {
          a.phases = kCompress | kPublish;
          code = exchange(ch, a);
          if (code == kOk) { a.phases = kExchange; code = exchange(ch, a); }
        } else {
          code = exchange(ch, a);
        }
        if (code != kOk) { rc[r] = 10 + (int)code; return; }
        for (long long i = 0; i < n; ++i) if (!std::isfinite(outs[r][(size_t)i])) { rc[r] = 3; return; }
      }
    });
  }
  for (auto& t : threads) t.join();
  int bad = 0;
  for (int r = 0; r < world; ++r) bad |= rc[r];
  for (int r = 1; r < world && !bad; ++r)
    if (std::memcmp(outs[0].data(), outs[r].data(), (size_t)n * 4) != 0) bad = 4;   // replicas must agree bit for bit
  for (int r = 0; r < world; ++r) heap_delete(w.base[r]);
  return bad;
}

// A peer that never publishes: the waiting rank must come back with a time-out naming that peer.
int run_timeout() {
  const long long n = 1000;
  const size_t sb = slot_bytes(kDense, n, 0);
  World w{2, 3 * kMaxWorld * 8 + 64 + 2 * sb + 256, {}};
  for (int r = 0; r < 2; ++r) {
    w.base.push_back(heap_new(w.heap_bytes));
    if (!w.base.back()) return 2;
  }
  const Channel ch = channel_for(w, 0, sb, 100ull * 1000000ull);   // 100 ms
  std::vector<float> g((size_t)n, 1.f), out((size_t)n);
  Args a{};
  a.codec = kDense; a.phases = kAll; a.seq = 1; a.g = g.data(); a.out = out.data(); a.n = n; a.gamma = 1.f; a.scale = 0.5f;
  const unsigned code = exchange(ch, a);
  const unsigned* st = reinterpret_cast<const unsigned*>(static_cast<char*>(w.base[0]) + ch.status_off);
  const int bad = (code == kTimeoutPeerReady && st[0] == kTimeoutPeerReady && st[1] == 1 && st[2] == 1) ? 0 : 5;
  for (int r = 0; r < 2; ++r) heap_delete(w.base[r]);
  return bad;
}

// PowerSGD: two rendezvous per exchange (P, then Q through the second flag pad), warm-started Q, error feedback.
int run_lowrank(int world, int steps) {
  const int rows = 24, cols = 20, rank = 3;
  const size_t sb = lowrank_slot_bytes(rows, cols, rank);
  World w{world, 3 * kMaxWorld * 8 + 64 + 2 * sb + 256, {}};
  for (int r = 0; r < world; ++r) {
    w.base.push_back(heap_new(w.heap_bytes));
    if (!w.base.back()) return 2;
  }
  std::vector<std::vector<float>> outs(world, std::vector<float>((size_t)rows * cols));
  std::vector<int> rc(world, 0);
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r) {
    threads.emplace_back([&, r] {
      Channel ch{};
      ch.rank = r; ch.world = world;
      for (int p = 0; p < world; ++p) ch.heap[p] = static_cast<char*>(w.base[p]);
      ch.ready_off = 0; ch.ack_off = kMaxWorld * 8; ch.status_off = 3 * kMaxWorld * 8;
      ch.slot_off[0] = 3 * kMaxWorld * 8 + 64; ch.slot_off[1] = ch.slot_off[0] + sb; ch.slot_bytes = sb;
      ch.timeout_ns = 20ull * 1000000000ull;
      std::vector<float> g((size_t)rows * cols), acc((size_t)rows * cols, 0.f), q((size_t)cols * rank), pw((size_t)rows * rank);
      for (size_t i = 0; i < q.size(); ++i) q[i] = pseudo(99, 0, (long long)i) * 500.f;   // the same start on every rank
      for (int s = 0; s < steps; ++s) {
        for (size_t i = 0; i < g.size(); ++i) g[i] = pseudo(r, s, (long long)i);
        if ((r + s) % 2 == 0) std::this_thread::sleep_for(std::chrono::microseconds(200 * (r + 1)));
        LowRankArgs a{};
        a.seq = (uint64_t)s + 1; a.g = g.data(); a.acc = acc.data(); a.out = outs[r].data(); a.q = q.data();
        a.p_work = pw.data(); a.rows = rows; a.cols = cols; a.rank = rank; a.ready2_off = 2 * kMaxWorld * 8;
        unsigned code;
        if (s & 1) {
          a.phases = kCompress | kPublish;
          code = lowrank_exchange(ch, a);
          if (code == kOk) { a.phases = kExchange; code = lowrank_exchange(ch, a); }
        } else {
          a.phases = kAll;
          code = lowrank_exchange(ch, a);
        }
        if (code != kOk) { rc[r] = 10 + (int)code; return; }
        for (float v : outs[r]) if (!std::isfinite(v)) { rc[r] = 3; return; }
      }
    });
  }
  for (auto& t : threads) t.join();
  int bad = 0;
  for (int r = 0; r < world; ++r) bad |= rc[r];
  for (int r = 1; r < world && !bad; ++r)
    if (std::memcmp(outs[0].data(), outs[r].data(), outs[0].size() * 4) != 0) bad = 4;
  for (int r = 0; r < world; ++r) heap_delete(w.base[r]);
  return bad;
}

// Negative control (argument "broken"): rank 1 raises its ready flag BEFORE it writes its slot, which is exactly
// the error the protocol exists to prevent.  A ThreadSanitizer build must report the race between rank 1's slot
// writes and rank 0's reads; this shows that the clean runs above are clean because of the protocol, not because
// the detector cannot see these accesses.
int run_broken_publish() {
  const long long n = 2000;
  const size_t sb = slot_bytes(kDense, n, 0);
  World w{2, 3 * kMaxWorld * 8 + 64 + 2 * sb + 256, {}};
  for (int r = 0; r < 2; ++r) {
    w.base.push_back(heap_new(w.heap_bytes));
    if (!w.base.back()) return 2;
  }
  std::vector<float> g0((size_t)n, 1.f), g1((size_t)n, 2.f), out((size_t)n);
  std::thread t1([&] {
    const Channel ch = channel_for(w, 1, sb, 1000000000ull);
    for (int p = 0; p < 2; ++p)   // the premature flag
      __atomic_store_n(reinterpret_cast<uint64_t*>(static_cast<char*>(w.base[p]) + ch.ready_off) + 1, 1, __ATOMIC_RELEASE);
    Args a{};
    a.codec = kDense; a.phases = kCompress; a.seq = 1; a.g = g1.data(); a.out = g1.data(); a.n = n; a.gamma = 1.f; a.scale = 0.5f;
    exchange(ch, a);
  });
  std::thread t0([&] {
    const Channel ch = channel_for(w, 0, sb, 1000000000ull);
    Args a{};
    a.codec = kDense; a.phases = kAll; a.seq = 1; a.g = g0.data(); a.out = out.data(); a.n = n; a.gamma = 1.f; a.scale = 0.5f;
    exchange(ch, a);
  });
  t0.join();
  t1.join();
  for (int r = 0; r < 2; ++r) heap_delete(w.base[r]);
  return 0;
}

// The shared-memory calls: create, open the same object a second time, see one's own writes through the other
// mapping, close, unlink.
int run_shm() {
  const std::string name = "/grace_san_" + std::to_string((long long)getpid());
  char* a = static_cast<char*>(heap_create(name.c_str(), 8192));
  if (!a) return 2;
  char* b = static_cast<char*>(heap_open(name.c_str(), 8192));
  if (!b) return 3;
  a[100] = 42;
  const int bad = (b[100] == 42 && b[101] == 0 && heap_open(name.c_str(), 1 << 20) == nullptr) ? 0 : 6;
  heap_close(a, 8192);
  heap_close(b, 8192);
  heap_unlink(name.c_str());
  return bad;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc > 1 && std::string(argv[1]) == "broken") return run_broken_publish();
  const int world = argc > 1 ? std::atoi(argv[1]) : 4;
  const int steps = argc > 2 ? std::atoi(argv[2]) : 12;
  const int codecs[] = {kTopK, kThreshold, kQSGD, kSign, kEFSign, kDense, kTernGrad, kNatural, kU8bit, kOneBit, kFP16, kRandomK, kQSGDX};
  for (int codec : codecs) {
    for (long long n : {1ll, 127ll, 4099ll}) {
      const int rc = run_codec(codec, world, n, steps);
      if (rc) { std::fprintf(stderr, "codec %d, %lld elements: failure %d\n", codec, n, rc); return 1; }
    }
  }
  for (int codec : {kQSGD, kNatural, kFP16, kDense})   // two-phase mode: reduce my chunk, encode again, gather
    for (long long n : {1ll, 127ll, 4099ll}) {
      const int rc = run_codec(codec, world, n, steps, true);
      if (rc) { std::fprintf(stderr, "two-phase codec %d, %lld elements: failure %d\n", codec, n, rc); return 1; }
    }
  if (const int rc = run_lowrank(world, steps)) { std::fprintf(stderr, "low-rank exchange: failure %d\n", rc); return 1; }
  if (const int rc = run_timeout()) { std::fprintf(stderr, "time-out scenario: failure %d\n", rc); return 1; }
  if (const int rc = run_shm()) { std::fprintf(stderr, "shared-memory calls: failure %d\n", rc); return 1; }
  std::printf("host protocol: %d ranks x %d steps x 13 codecs x 3 sizes, the two-phase mode and the low-rank exchange ok, time-out reported\n", world, steps);
  return 0;
}
