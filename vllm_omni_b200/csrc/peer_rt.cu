// Peer-memory runtime for the fused compute+collective kernels.
//
// One process per GPU.  Every rank allocates an arena with cudaMalloc, exports it as a CUDA
// IPC handle, and maps the arenas of all peers of its group, so that kernels can store to /
// load from a peer's memory over NVLink with ordinary global accesses.  (The reference has no
// counterpart: it moves everything through NCCL calls between kernels,
// vllm_omni/diffusion/distributed/comm.py.)
//
// Synchronisation is a flag page per rank: flag[j] on rank i is written only by rank j and
// holds the number of barriers rank j has entered.  omni_peer_barrier:
//   1. __threadfence_system(): this rank's earlier stores (peer stores included) are ordered
//      before the flag stores,
//   2. bumps a device-resident epoch counter (so the same launch can be replayed from a CUDA
//      graph) and stores the new epoch into flag[my_rank] of every peer (st.release.sys),
//   3. spins (ld.acquire.sys) until every peer's flag in the local page reaches the epoch.
// The spin is bounded: after `timeout_ns` the kernel writes ERR_WAIT_PEER to the status word
// and returns, leaving the context usable; the host turns that into an exception.
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  unsigned long long* flags[MAX_PEERS];  // flag page of every rank (index = rank in group)
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__global__ void peer_barrier_kernel(PeerPtrs peers, int rank, int world, unsigned long long* epoch_counter,
                                    unsigned long long timeout_ns, int* status) {
  __shared__ unsigned long long s_epoch;
  __threadfence_system();
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    *epoch_counter = s_epoch;
  }
  __syncthreads();
  const unsigned long long epoch = s_epoch;
  const int j = threadIdx.x;
  if (j < world && j != rank) {
    st_release_sys(peers.flags[j] + rank, epoch);
    const unsigned long long* mine = peers.flags[rank] + j;
    const unsigned long long t0 = globaltimer_ns();
    unsigned it = 0;
    while (ld_acquire_sys(mine) < epoch) {
      if ((++it & 0x3f) == 0 && globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, ERR_WAIT_PEER);
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
}

// Flat copy into (or out of) a peer-mapped buffer with ordinary 16-byte loads and stores: every
// warp instruction moves 512 contiguous bytes, so the NVLink packets are full.  Used by the
// device-to-device stage connector to push a payload into the consumer stage's arena.
__global__ void __launch_bounds__(256)
peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n16, unsigned char* __restrict__ dst_tail,
                 const unsigned char* __restrict__ src_tail, int tail) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

// Pitched copy: `rows` segments of `row16` 16-byte words each (K and V of every row of a packed
// [rows, q | k | v] buffer, for example), either side may be a peer mapping.  A warp moves 512
// contiguous bytes of one segment per instruction.
__global__ void __launch_bounds__(256)
peer_copy_2d_kernel(unsigned char* __restrict__ dst, size_t dst_pitch, const unsigned char* __restrict__ src, size_t src_pitch,
                    int row16, long rows) {
  // blockIdx.y walks the segments, blockIdx.x the 16-byte words of a segment; four independent 16-byte loads per
  // thread are in flight before the first store (remote loads have microseconds of latency)
  for (long r = blockIdx.y; r < rows; r += gridDim.y) {
    const uint4* s = reinterpret_cast<const uint4*>(src + r * src_pitch);
    uint4* d = reinterpret_cast<uint4*>(dst + r * dst_pitch);
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4; c < row16; c += gridDim.x * blockDim.x * 4) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < row16) v[j] = s[c + j];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < row16) d[c + j] = v[j];
    }
  }
}

}  // namespace omni

using namespace omni;

// Pitches and row_bytes in bytes, all multiples of 16; dst / src 16-byte aligned.
extern "C" int omni_peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                                 long rows, void* stream) {
  if (rows <= 0 || row_bytes == 0) return RC_OK;
  if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (dst_pitch & 15) ||
      (src_pitch & 15) || (row_bytes & 15) || row_bytes > dst_pitch || row_bytes > src_pitch || (row_bytes >> 4) > 0x7fffffff)
    return RC_BAD_ARG;
  const int row16 = (int)(row_bytes >> 4);
  // about 16 blocks per SM in total: few long segments spread over blockIdx.x, many short ones over blockIdx.y
  const long budget = 148 * 16;
  long gx = (row16 + 1023) / 1024;                    // 256 threads x 4 words per block
  long gy = rows < 65535 ? rows : 65535;
  if (gx * gy > budget) {
    if (gy >= budget) { gx = 1; gy = budget; }
    else gx = (budget + gy - 1) / gy < gx ? (budget + gy - 1) / gy : gx;
  }
  peer_copy_2d_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, (cudaStream_t)stream>>>(
      static_cast<unsigned char*>(dst), dst_pitch, static_cast<const unsigned char*>(src), src_pitch, row16, rows);
  return (int)cudaGetLastError();
}

// dst / src: device pointers (either may be a peer mapping), both 16-byte aligned.
extern "C" int omni_peer_copy(void* dst, const void* src, size_t nbytes, void* stream) {
  if (nbytes == 0) return RC_OK;
  if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return RC_BAD_ARG;
  const size_t n16 = nbytes >> 4;
  const int tail = (int)(nbytes & 15);
  size_t blocks = (n16 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks == 0) blocks = 1;
  peer_copy_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16, static_cast<unsigned char*>(dst) + (n16 << 4),
      static_cast<const unsigned char*>(src) + (n16 << 4), tail);
  return (int)cudaGetLastError();
}

extern "C" int omni_peer_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

extern "C" int omni_peer_free(void* p) { return (int)cudaFree(p); }

// handle: 64 bytes
extern "C" int omni_peer_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

extern "C" int omni_peer_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}

extern "C" int omni_peer_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

extern "C" int omni_ipc_handle_size(void) { return (int)sizeof(cudaIpcMemHandle_t); }

// flag_pages: `world` device pointers (this rank's own page at index `rank`), each at least
// `world` u64 entries; epoch_counter: a device u64 owned by this rank.
extern "C" int omni_peer_barrier(void* const* flag_pages, int rank, int world, void* epoch_counter,
                                 unsigned long long timeout_ns, int* status, void* stream) {
  if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) return RC_BAD_ARG;
  if (world == 1) return RC_OK;
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.flags[i] = i < world ? (unsigned long long*)flag_pages[i] : nullptr;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pp, rank, world, (unsigned long long*)epoch_counter,
                                                          timeout_ns, status);
  return (int)cudaGetLastError();
}
