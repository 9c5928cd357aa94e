// Host-thread model of the two lock-free protocols of the runtime, meant to be built with
// -fsanitize=thread (tests/test_host_protocols.py does that):
//
//  1. the shared-memory SPSC ring of rt_host.cpp (the real code, included below): one producer
//     and one consumer thread move N messages through a small ring and check order and content;
//  2. the epoch/flag barrier of peer_rt.cu restated with std::atomic (release store of the epoch
//     into every peer's flag slot, acquire loads until every peer's slot reaches it): P threads
//     alternate "write my block, barrier, read everyone's block, barrier" and every read must see
//     the value of the current round.  A data race or a missing release/acquire pair is reported
//     by ThreadSanitizer; a logic error by the checks (exit code 1).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "../rt_host.cpp"

namespace {

int ring_test(int n_msgs) {
  char name[64];
  snprintf(name, sizeof(name), "/omni_tsan_ring_%d", (int)getpid());
  void* prod = omni_ring_open(name, 1, 64, 8);
  if (!prod) { fprintf(stderr, "ring create failed\n"); return 1; }
  void* cons = omni_ring_open(name, 0, 0, 0);
  if (!cons) { fprintf(stderr, "ring attach failed\n"); return 1; }
  int bad = 0;
  std::thread tp([&] {
    for (int i = 0; i < n_msgs; ++i) {
      uint32_t msg[4] = {(uint32_t)i, (uint32_t)i * 3u, 0xabcdu, (uint32_t)(i % 7)};
      const uint32_t len = 4 + 4 * (i % 4);
      while (omni_ring_push(prod, msg, len) == -1) std::this_thread::yield();
    }
  });
  std::thread tc([&] {
    for (int i = 0; i < n_msgs; ++i) {
      uint32_t msg[16];
      int len;
      while ((len = omni_ring_pop(cons, msg, sizeof(msg))) == -1) std::this_thread::yield();
      if (len != 4 + 4 * (i % 4) || msg[0] != (uint32_t)i) ++bad;
      if (len >= 8 && msg[1] != (uint32_t)i * 3u) ++bad;
    }
  });
  tp.join();
  tc.join();
  if (omni_ring_size(cons) != 0) ++bad;
  omni_ring_close(cons);
  omni_ring_close(prod);
  return bad;
}

struct Rank {
  std::vector<std::atomic<unsigned long long>> flags;   // flags[j]: written by rank j only
  unsigned long long epoch = 0;
  std::vector<int> block;                               // plain (non-atomic) payload
  explicit Rank(int P) : flags(P), block(64, -1) {
    for (auto& f : flags) f.store(0);
  }
};

// returns false when the wait ran out (bounded, like the device kernel)
bool barrier(std::vector<Rank*>& ranks, int me, long spin_limit) {
  Rank& r = *ranks[me];
  const unsigned long long e = ++r.epoch;
  const int P = (int)ranks.size();
  for (int j = 0; j < P; ++j)
    if (j != me) ranks[j]->flags[me].store(e, std::memory_order_release);
  for (int j = 0; j < P; ++j) {
    if (j == me) continue;
    long it = 0;
    while (r.flags[j].load(std::memory_order_acquire) < e) {
      if (++it > spin_limit) return false;
      std::this_thread::yield();
    }
  }
  return true;
}

int barrier_test(int P, int rounds) {
  std::vector<Rank*> ranks;
  for (int i = 0; i < P; ++i) ranks.push_back(new Rank(P));
  std::atomic<int> bad{0};
  std::vector<std::thread> ts;
  for (int me = 0; me < P; ++me) {
    ts.emplace_back([&, me] {
      for (int round = 0; round < rounds; ++round) {
        for (auto& v : ranks[me]->block) v = round * 100 + me;        // "peer stores"
        if (!barrier(ranks, me, 50000000L)) { ++bad; return; }
        for (int j = 0; j < P; ++j)                                    // "peer loads"
          for (int v : ranks[j]->block)
            if (v != round * 100 + j) ++bad;
        if (!barrier(ranks, me, 50000000L)) { ++bad; return; }         // blocks may be overwritten
      }
    });
  }
  for (auto& t : ts) t.join();
  // a partner that never arrives: the wait gives up
  Rank lonely(2), ghost(2);
  std::vector<Rank*> two = {&lonely, &ghost};
  if (barrier(two, 0, 1000)) ++bad;
  for (auto* r : ranks) delete r;
  return bad.load();
}

}  // namespace

int main() {
  const int a = ring_test(20000);
  const int b = barrier_test(4, 300);
  printf("ring_errors=%d barrier_errors=%d\n", a, b);
  return (a || b) ? 1 : 0;
}
