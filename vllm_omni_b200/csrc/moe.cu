// K10: mixture-of-experts routing, dispatch and combine around the grouped tcgen05 GEMM.
//
//   omni_moe_route     softmax over expert logits, top-k, optional renormalisation
//   omni_moe_plan      per-expert counts -> segment offsets padded to 128 rows (the GEMM's M
//                      tile), the expert of every M tile, and the row of every (token, k) pair
//   omni_moe_dispatch  copy token rows into the expert-major padded buffer
//   omni_moe_combine   out[t] = sum_k w[t,k] * y[row(t,k)]  (+ optional residual / shared expert)
//
// Padding each expert segment to the 128-row MMA tile keeps every GEMM tile inside one expert,
// so the expert GEMMs are ONE launch of the grouped kernel (gemm_sm100.cu) with a per-tile
// expert index.  The reference reaches vLLM's Triton fused_moe or a Python loop over experts
// (vllm_omni/model_executor/models/qwen3_omni/qwen3_moe.py).
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

constexpr int MOE_TILE = 128;

// Limits for the checked build (OMNI_IN_BOUNDS in ptx_sm100.cuh; 0 = unknown / unchecked), set by the host
// through omni_moe_set_bounds and passed to the kernels by value: the rows the expert-major buffers hold.
struct MoeBounds {
  long max_rows;
  int* status;
};
static MoeBounds g_moe_bounds = {0, nullptr};
enum { KID_MOE_PLAN = 3, KID_MOE_DISPATCH = 4, KID_MOE_COMBINE = 5 };

// one warp per token; E <= 256 (8 per lane), k <= 16
__global__ void __launch_bounds__(256)
moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int T, int E, int k, int renorm,
                 int* __restrict__ ids, float* __restrict__ weights) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + i * 32;
    v[i] = e < E ? __bfloat162float(logits[(size_t)t * ld + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { v[i] = v[i] == -INFINITY ? 0.f : __expf(v[i] - mx); sum += v[i]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
  float picked = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + i * 32;
      if (v[i] > best || (v[i] == best && e < bi)) { best = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { ids[(size_t)t * k + j] = bi; weights[(size_t)t * k + j] = best * inv; }
    picked += best * inv;
    if ((bi & 31) == lane) v[bi >> 5] = -1.f;   // remove the winner
  }
  if (renorm && lane == 0) {
    const float r = 1.0f / fmaxf(picked, 1e-20f);
    for (int j = 0; j < k; ++j) weights[(size_t)t * k + j] *= r;
  }
}

// single CTA: histogram, padded prefix sum, tile->expert table, (token,k)->row map.
// counts/cursor live in shared memory (E <= 1024).
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int E, int e_lo, int e_hi, int max_tiles,
                int* __restrict__ row_of_pair, int* __restrict__ tile_expert, int* __restrict__ offsets,
                int* __restrict__ n_rows_out, MoeBounds bd) {
  __shared__ int cnt[1024];
  __shared__ int off[1025];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (!OMNI_IN_BOUNDS(e >= 0 && e < E, bd.status, KID_MOE_PLAN)) continue;
    if (e >= e_lo && e < e_hi) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = acc;
      acc += (cnt[e] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    }
    off[E] = acc;
    *n_rows_out = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
    // expert owning row tile*128: the last e with off[e] <= row (binary search)
    const int row = tile * MOE_TILE;
    int ex = -1;
    if (row < off[E]) {
      int lo = 0, hi = E - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      ex = lo;
    }
    tile_expert[tile] = ex;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;   // reuse as cursors
  __syncthreads();
  // deterministic placement: pairs are placed in index order per expert by one thread per expert
  // when the batch is small, otherwise by atomics (order inside an expert does not affect results)
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    row_of_pair[i] = (e >= e_lo && e < e_hi) ? off[e] + atomicAdd(&cnt[e], 1) : -1;
  }
}

// Plan without padding: the rows of expert e are [off[e], off[e] + cnt[e]); expert e owns ceil(cnt[e] / 128)
// M tiles; tile t = (expert, first row, rows <= 128).  Unused tiles get expert -1.
__global__ void __launch_bounds__(1024)
moe_plan_compact_kernel(const int* __restrict__ ids, int n_pairs, int E, int e_lo, int e_hi, int max_tiles,
                        int* __restrict__ row_of_pair, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                        int* __restrict__ tile_rows, int* __restrict__ n_rows_out, MoeBounds bd) {
  __shared__ int cnt[1024];
  __shared__ int off[1025];
  __shared__ int toff[1025];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (!OMNI_IN_BOUNDS(e >= 0 && e < E, bd.status, KID_MOE_PLAN)) continue;
    if (e >= e_lo && e < e_hi) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, tacc = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = acc;
      toff[e] = tacc;
      acc += cnt[e];
      tacc += (cnt[e] + MOE_TILE - 1) / MOE_TILE;
    }
    off[E] = acc;
    toff[E] = tacc;
    *n_rows_out = acc;
  }
  __syncthreads();
  for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
    int ex = -1, r0 = 0, nr = 0;
    if (tile < toff[E]) {
      int lo = 0, hi = E - 1;            // the last e with toff[e] <= tile that owns tiles
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (toff[mid] <= tile) lo = mid; else hi = mid - 1;
      }
      ex = lo;
      const int within = tile - toff[ex];
      r0 = off[ex] + within * MOE_TILE;
      nr = min(MOE_TILE, cnt[ex] - within * MOE_TILE);
    }
    tile_expert[tile] = ex;
    tile_row0[tile] = r0;
    tile_rows[tile] = nr;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;   // reuse as cursors
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    row_of_pair[i] = (e >= e_lo && e < e_hi) ? off[e] + atomicAdd(&cnt[e], 1) : -1;
  }
}

// x: [T, D] (pitch ldx) -> xp[row_of_pair[t*k+j], :] ; rows not written stay as they are (the GEMM
// output rows of padding are never read back)
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const int* __restrict__ row_of_pair, int n_pairs,
                    int k, int D, __nv_bfloat16* __restrict__ xp, MoeBounds bd) {
  const int chunks = D >> 3;
  const long total = (long)n_pairs * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int p = (int)(i / chunks);
    const int c = (int)(i % chunks) * 8;
    const int r = row_of_pair[p];
    if (r < 0) continue;
    if (!OMNI_IN_BOUNDS(bd.max_rows == 0 || r < bd.max_rows, bd.status, KID_MOE_DISPATCH)) continue;
    *reinterpret_cast<uint4*>(xp + (size_t)r * D + c) = *reinterpret_cast<const uint4*>(x + (size_t)(p / k) * ldx + c);
  }
}

// out[t, :] = (residual[t, :]) + sum_j w[t,j] * y[row(t,j), :]; pairs with row < 0 (experts of
// another rank) contribute nothing.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_pair,
                   const float* __restrict__ weights, int T, int k, int D, const __nv_bfloat16* __restrict__ residual,
                   long ldr, __nv_bfloat16* __restrict__ out, long ldo, MoeBounds bd) {
  const int chunks = D >> 3;
  const long total = (long)T * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks);
    const int c = (int)(i % chunks) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + (size_t)t * ldr + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = cc.x; acc[5] = cc.y; acc[6] = d.x; acc[7] = d.y;
    }
    for (int j = 0; j < k; ++j) {
      const int r = row_of_pair[(size_t)t * k + j];
      if (r < 0) continue;
      if (!OMNI_IN_BOUNDS(bd.max_rows == 0 || r < bd.max_rows, bd.status, KID_MOE_COMBINE)) continue;
      const float w = weights[(size_t)t * k + j];
      const uint4 u = *reinterpret_cast<const uint4*>(y + (size_t)r * D + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
      acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * d.x; acc[7] += w * d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * ldo + c) = o;
  }
}

// Expert-parallel combine: the weighted sum of THIS rank's experts for token t is a partial result;
// it is stored straight into the slot this rank owns on the rank that owns token t's row block
// (peer_out[t / rows_per_owner], local row t % rows_per_owner, pitch D), so the cross-rank sum needs
// no separate all-reduce of a [T, D] tensor: a local reduce kernel finishes it (tp_reduce.cu).
struct MoePeers {
  __nv_bfloat16* out[16];
};
__global__ void __launch_bounds__(256)
moe_combine_scatter_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_pair,
                           const float* __restrict__ weights, int T, int k, int D, int rows_per_owner, MoePeers peers,
                           MoeBounds bd) {
  const int chunks = D >> 3;
  const long total = (long)T * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks);
    const int c = (int)(i % chunks) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int r = row_of_pair[(size_t)t * k + j];
      if (r < 0) continue;
      if (!OMNI_IN_BOUNDS(bd.max_rows == 0 || r < bd.max_rows, bd.status, KID_MOE_COMBINE)) continue;
      const float w = weights[(size_t)t * k + j];
      const uint4 u = *reinterpret_cast<const uint4*>(y + (size_t)r * D + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
      acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * d.x; acc[7] += w * d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    const int owner = t / rows_per_owner;
    *reinterpret_cast<uint4*>(peers.out[owner] + (size_t)(t - owner * rows_per_owner) * D + c) = o;
  }
}

}  // namespace omni

using namespace omni;

// 1 when this library was compiled with -DOMNI_BOUNDS_CHECK
extern "C" int omni_moe_bounds_check_enabled(void) {
#ifdef OMNI_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" void omni_moe_set_bounds(long max_rows, int* status) {
  g_moe_bounds.max_rows = max_rows;
  g_moe_bounds.status = status;
}

extern "C" int omni_moe_combine_scatter(const void* y, const int* row_of_pair, const float* weights, int T, int k, int D,
                                        int rows_per_owner, void* const* peer_out, void* stream) {
  if (T <= 0) return RC_OK;
  if ((D & 7) || rows_per_owner <= 0 || peer_out == nullptr) return RC_BAD_ARG;
  const int owners = (T + rows_per_owner - 1) / rows_per_owner;
  if (owners > 16) return RC_BAD_ARG;
  MoePeers peers;
  for (int i = 0; i < 16; ++i) peers.out[i] = i < owners ? static_cast<__nv_bfloat16*>(peer_out[i]) : nullptr;
  long blocks = ((long)T * (D >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  moe_combine_scatter_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, row_of_pair, weights, T, k, D, rows_per_owner, peers, g_moe_bounds);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_route(const void* logits, int ld, int T, int E, int k, int renorm, int* ids, float* weights,
                              void* stream) {
  if (T <= 0) return RC_OK;
  if (E > 256 || k > 16 || k > E) return RC_BAD_ARG;
  moe_route_kernel<<<(T + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, T, E, k, renorm, ids, weights);
  return (int)cudaGetLastError();
}

// Experts [e_lo, e_hi) are local (expert parallelism); others get row -1.
// max_tiles: capacity of tile_expert = ceil((n_pairs + E*127) / 128).
extern "C" int omni_moe_plan(const int* ids, int n_pairs, int E, int e_lo, int e_hi, int max_tiles, int* row_of_pair,
                             int* tile_expert, int* offsets, int* n_rows_out, void* stream) {
  if (E > 1024) return RC_BAD_ARG;
  moe_plan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, n_pairs, E, e_lo, e_hi, max_tiles, row_of_pair, tile_expert, offsets, n_rows_out,
                                                        g_moe_bounds);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_plan_compact(const int* ids, int n_pairs, int E, int e_lo, int e_hi, int max_tiles, int* row_of_pair,
                                     int* tile_expert, int* tile_row0, int* tile_rows, int* n_rows_out, void* stream) {
  if (E > 1024) return RC_BAD_ARG;
  moe_plan_compact_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, n_pairs, E, e_lo, e_hi, max_tiles, row_of_pair, tile_expert,
                                                                tile_row0, tile_rows, n_rows_out, g_moe_bounds);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_dispatch(const void* x, long ldx, const int* row_of_pair, int n_pairs, int k, int D, void* xp,
                                 void* stream) {
  if (n_pairs <= 0) return RC_OK;
  if (D & 7) return RC_BAD_ARG;
  long blocks = ((long)n_pairs * (D >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  moe_dispatch_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, row_of_pair, n_pairs, k, D, (__nv_bfloat16*)xp,
                                                                          g_moe_bounds);
  return (int)cudaGetLastError();
}

extern "C" int omni_moe_combine(const void* y, const int* row_of_pair, const float* weights, int T, int k, int D,
                                const void* residual, long ldr, void* out, long ldo, void* stream) {
  if (T <= 0) return RC_OK;
  if (D & 7) return RC_BAD_ARG;
  long blocks = ((long)T * (D >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  moe_combine_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, row_of_pair, weights, T, k, D, (const __nv_bfloat16*)residual, ldr, (__nv_bfloat16*)out, ldo,
      g_moe_bounds);
  return (int)cudaGetLastError();
}
