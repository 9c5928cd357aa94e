// Host-side runtime pieces that the AR engine calls on its critical path (no CUDA here):
//
//  * block allocator for the paged KV cache: free-list stack with reference counts
//    (prefix sharing), O(1) alloc/free, used by engine/kv_cache_manager.py
//  * SPSC byte ring over shared memory (POSIX shm + futex-free polling) used as the control
//    plane between an engine process and its worker processes: fixed-size slots with a
//    length header, sequence counters for lock-free publish/consume.
//
// The reference takes both from vLLM (KVCacheManager, shm MessageQueue).
#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

struct BlockAllocator {
  std::vector<int32_t> free_list;
  std::vector<int32_t> refcnt;
  std::mutex mu;
};

struct RingHeader {
  std::atomic<uint64_t> head;   // next slot to write
  std::atomic<uint64_t> tail;   // next slot to read
  uint32_t slot_bytes;
  uint32_t num_slots;
};

struct Ring {
  RingHeader* hdr;
  uint8_t* data;
  size_t map_bytes;
  int fd;
  bool owner;
  char name[128];
};

}  // namespace

extern "C" {

// ------------------------------------------------------------------ block allocator
void* omni_balloc_create(int num_blocks) {
  auto* a = new BlockAllocator();
  a->refcnt.assign(num_blocks, 0);
  a->free_list.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) a->free_list.push_back(i);   // block 0 is handed out first
  return a;
}
void omni_balloc_destroy(void* h) { delete static_cast<BlockAllocator*>(h); }
int omni_balloc_num_free(void* h) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> lk(a->mu);
  return (int)a->free_list.size();
}
// Allocates n blocks into out[]; returns 0, or -1 (and allocates nothing) when fewer are free.
int omni_balloc_alloc(void* h, int n, int32_t* out) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> lk(a->mu);
  if ((int)a->free_list.size() < n) return -1;
  for (int i = 0; i < n; ++i) {
    const int32_t b = a->free_list.back();
    a->free_list.pop_back();
    a->refcnt[b] = 1;
    out[i] = b;
  }
  return 0;
}
// Adds a reference (prefix sharing).  Returns the new count or -1 for a block that is free.
int omni_balloc_ref(void* h, int block) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> lk(a->mu);
  if (block < 0 || block >= (int)a->refcnt.size() || a->refcnt[block] <= 0) return -1;
  return ++a->refcnt[block];
}
// Drops one reference from each block; blocks whose count reaches 0 return to the free list.
// Returns the number of blocks actually freed, or -1 on a double free.
int omni_balloc_free(void* h, int n, const int32_t* blocks) {
  auto* a = static_cast<BlockAllocator*>(h);
  std::lock_guard<std::mutex> lk(a->mu);
  int freed = 0;
  for (int i = 0; i < n; ++i) {
    const int32_t b = blocks[i];
    if (b < 0 || b >= (int)a->refcnt.size() || a->refcnt[b] <= 0) return -1;
    if (--a->refcnt[b] == 0) {
      a->free_list.push_back(b);
      ++freed;
    }
  }
  return freed;
}

// ------------------------------------------------------------------------ shm ring
void* omni_ring_open(const char* name, int create, uint32_t slot_bytes, uint32_t num_slots) {
  int fd = shm_open(name, create ? (O_CREAT | O_RDWR | O_EXCL) : O_RDWR, 0600);
  if (fd < 0) return nullptr;
  size_t bytes = sizeof(RingHeader) + (size_t)slot_bytes * num_slots;
  if (create) {
    if (ftruncate(fd, (off_t)bytes) != 0) { close(fd); shm_unlink(name); return nullptr; }
  } else {
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); return nullptr; }
    bytes = (size_t)st.st_size;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) { close(fd); if (create) shm_unlink(name); return nullptr; }
  auto* r = new Ring();
  r->hdr = static_cast<RingHeader*>(p);
  r->data = static_cast<uint8_t*>(p) + sizeof(RingHeader);
  r->map_bytes = bytes;
  r->fd = fd;
  r->owner = create != 0;
  strncpy(r->name, name, sizeof(r->name) - 1);
  if (create) {
    r->hdr->head.store(0);
    r->hdr->tail.store(0);
    r->hdr->slot_bytes = slot_bytes;
    r->hdr->num_slots = num_slots;
  }
  return r;
}
void omni_ring_close(void* h) {
  auto* r = static_cast<Ring*>(h);
  munmap(r->hdr, r->map_bytes);
  close(r->fd);
  if (r->owner) shm_unlink(r->name);
  delete r;
}
uint32_t omni_ring_slot_bytes(void* h) { return static_cast<Ring*>(h)->hdr->slot_bytes - 4; }
// 0 = ok, -1 = ring full, -2 = message too large
int omni_ring_push(void* h, const void* msg, uint32_t len) {
  auto* r = static_cast<Ring*>(h);
  const uint32_t sb = r->hdr->slot_bytes;
  if (len + 4 > sb) return -2;
  const uint64_t head = r->hdr->head.load(std::memory_order_relaxed);
  const uint64_t tail = r->hdr->tail.load(std::memory_order_acquire);
  if (head - tail >= r->hdr->num_slots) return -1;
  uint8_t* slot = r->data + (size_t)(head % r->hdr->num_slots) * sb;
  memcpy(slot, &len, 4);
  memcpy(slot + 4, msg, len);
  r->hdr->head.store(head + 1, std::memory_order_release);
  return 0;
}
// returns the message length, -1 when empty, -2 when `cap` is too small (message stays queued)
int omni_ring_pop(void* h, void* out, uint32_t cap) {
  auto* r = static_cast<Ring*>(h);
  const uint64_t tail = r->hdr->tail.load(std::memory_order_relaxed);
  const uint64_t head = r->hdr->head.load(std::memory_order_acquire);
  if (tail == head) return -1;
  const uint8_t* slot = r->data + (size_t)(tail % r->hdr->num_slots) * r->hdr->slot_bytes;
  uint32_t len;
  memcpy(&len, slot, 4);
  if (len > cap) return -2;
  memcpy(out, slot + 4, len);
  r->hdr->tail.store(tail + 1, std::memory_order_release);
  return (int)len;
}
int omni_ring_size(void* h) {
  auto* r = static_cast<Ring*>(h);
  return (int)(r->hdr->head.load(std::memory_order_acquire) - r->hdr->tail.load(std::memory_order_acquire));
}

}  // extern "C"
