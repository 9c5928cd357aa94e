// One-way arrival signals between the ranks of a peer-memory group, consumed INSIDE the kernel
// that needs the data (no barrier kernel between producer and consumer).
//
// Producer kernel (writes into peers' buffers: the scatter epilogues of the GEMM and attention
// kernels).  Every CTA, once all of its peer stores are issued and ordered (CTA barrier, then a
// system-scope fence by one thread), counts itself on a LOCAL counter; the CTA that completes the
// count adds 1 to the arrival counter of every rank of the group (its own included) with
// system-scope atomics.  One launch therefore contributes exactly 1 to every rank's counter,
// whatever its grid size.
//
// Consumer kernel (reads what the peers wrote: q/k norm + rope after the QKV exchange, the
// out-projection GEMM after the attention exchange).  One thread per CTA reads the consumer's
// `epoch` word (uses completed so far; stable while the kernel runs), spins with ld.acquire.sys
// until the arrival counter reaches (epoch + 1) * per_use, and releases the CTA.  On exit every
// CTA counts itself; the last one resets the exit count and bumps the epoch, so the same launch
// can be replayed from a CUDA graph.  The spin is bounded: after `timeout_ns` the waiter writes
// ERR_WAIT_PEER to the status word, raises the CTA's abort flag (if it has one) and carries on,
// so the kernel always terminates.
//
// The reference has no counterpart: its exchanges are NCCL all-to-all calls between kernels
// (vllm_omni/diffusion/distributed/comm.py:16-207).
#pragma once
#include "ptx_sm100.cuh"

namespace omni {

constexpr int SIGNAL_MAX_PEERS = 16;

struct PeerSignal {
  unsigned long long* counters[SIGNAL_MAX_PEERS];  // arrival counter on every rank (index = rank in group)
  unsigned int* done;                              // local: CTAs of this launch that finished
  int n;                                           // ranks in the group; 0 = no signalling
};

struct PeerWait {
  const unsigned long long* counter;  // this rank's arrival counter; nullptr = no wait
  unsigned long long* epoch;          // local: [0] uses completed, [1] CTAs of this launch that left
  unsigned long long per_use;         // arrivals that make one use complete (producer launches x ranks)
  unsigned long long timeout_ns;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Call from ONE thread of the CTA after a CTA-wide barrier that follows the CTA's last peer store.
__device__ __forceinline__ void peer_signal_cta_done(const PeerSignal& s, unsigned int total_ctas) {
  if (s.n <= 0) return;
  __threadfence_system();
  const unsigned int prev = atomicAdd_system(s.done, 1u);
  if (prev == total_ctas - 1u) {
    *s.done = 0u;                       // next launch starts from zero (kernel boundary orders it)
    __threadfence_system();             // every counted CTA's stores are ordered before the arrivals
    for (int i = 0; i < s.n; ++i) atomicAdd_system(s.counters[i], 1ull);
  }
}

// Call from ONE thread of the CTA before the CTA touches peer-written data; follow with a CTA
// barrier (or an mbarrier hand-off) for the other threads.  Returns false on timeout.
__device__ __forceinline__ bool peer_wait_arrivals(const PeerWait& w, volatile int* s_abort, int* status) {
  if (w.counter == nullptr) return true;
  const unsigned long long target = (*(volatile unsigned long long*)w.epoch + 1ull) * w.per_use;
  if (ld_acquire_sys_u64(w.counter) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (unsigned int it = 1;; ++it) {
    if (ld_acquire_sys_u64(w.counter) >= target) return true;
    if ((it & 0x3f) == 0) {
      if (s_abort && *s_abort) return false;
      if (globaltimer_ns() - t0 > w.timeout_ns) {
        if (s_abort) *s_abort = 1;
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

// Call from ONE thread of the CTA when the CTA is done (after its last read of peer-written data).
__device__ __forceinline__ void peer_wait_cta_exit(const PeerWait& w, unsigned int total_ctas) {
  if (w.counter == nullptr) return;
  const unsigned long long e = *(volatile unsigned long long*)w.epoch;
  const unsigned long long prev = atomicAdd(w.epoch + 1, 1ull);
  if (prev == (unsigned long long)total_ctas - 1ull) {
    w.epoch[1] = 0ull;
    w.epoch[0] = e + 1ull;
    __threadfence();
  }
}

// Host-side C mirror of the two structs, as the entry points take them (pointers may be null).
struct OmniSync {
  void* signal_counters[SIGNAL_MAX_PEERS];
  void* signal_done;
  int signal_n;
  const void* wait_counter;
  void* wait_epoch;
  unsigned long long wait_per_use;
  unsigned long long wait_timeout_ns;
};

inline void unpack_sync(const OmniSync* s, PeerSignal& sig, PeerWait& wt) {
  sig.n = 0; sig.done = nullptr;
  for (int i = 0; i < SIGNAL_MAX_PEERS; ++i) sig.counters[i] = nullptr;
  wt.counter = nullptr; wt.epoch = nullptr; wt.per_use = 0; wt.timeout_ns = 0;
  if (!s) return;
  if (s->signal_n > 0 && s->signal_n <= SIGNAL_MAX_PEERS && s->signal_done) {
    sig.n = s->signal_n;
    sig.done = static_cast<unsigned int*>(s->signal_done);
    for (int i = 0; i < s->signal_n; ++i) sig.counters[i] = static_cast<unsigned long long*>(s->signal_counters[i]);
  }
  if (s->wait_counter && s->wait_epoch && s->wait_per_use) {
    wt.counter = static_cast<const unsigned long long*>(s->wait_counter);
    wt.epoch = static_cast<unsigned long long*>(s->wait_epoch);
    wt.per_use = s->wait_per_use;
    wt.timeout_ns = s->wait_timeout_ns ? s->wait_timeout_ns : WAIT_LIMIT_NS;
  }
}

}  // namespace omni
