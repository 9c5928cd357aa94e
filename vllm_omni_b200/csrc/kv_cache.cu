// K11 (part 1) and K13: paged KV cache kernels for the AR engine.
//
// Cache layout per layer: K and V pages  [num_blocks, block_size, Hkv, D]  (bf16), one
// contiguous buffer each.  A sequence owns a list of page ids (its block table).
//
//   omni_kv_write      scatter this step's K/V rows into their pages (slot mapping)
//   omni_kv_gather     pages -> contiguous [T, Hkv, D] (context for chunked prefill; KV
//                      hand-off to another stage: the destination may be peer memory)
//   omni_paged_decode  one query token per sequence against its paged KV, GQA, split over
//                      the context with a second pass that merges the partial results (CUDA-core
//                      fallback; the tensor-core paged attention lives in attention_sm100.cu)
//
// The reference reaches vLLM's FlashAttention / FlashInfer backends for these
// (vllm_omni/worker/gpu_model_runner.py:37) and extracts KV for hand-off with eager index +
// .cpu() (vllm_omni/distributed/omni_connectors/kv_transfer_manager.py:217-276).
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

// Limits for the checked build (see OMNI_IN_BOUNDS in ptx_sm100.cuh): 0 = unknown / unchecked.  Set by the
// host through omni_kv_set_bounds before the launches of a step; passed to the kernels by value.
struct KvBounds {
  long num_slots;   // pages x page size of the cache the slot mapping addresses
  int num_blocks;   // pages of the cache the block tables address
  int* status;      // device status word
};
static KvBounds g_kv_bounds = {0, 0, nullptr};
enum { KID_KV_WRITE = 1, KID_KV_GATHER = 2 };

// ---------------------------------------------------------------------------- write
// k, v: [T, Hkv, D] with row pitch ld (elements); slot[t] = block * block_size + offset, <0 skips.
__global__ void __launch_bounds__(256)
kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long ldk, long ldv,
                __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, const int* __restrict__ slot, int T,
                int row_elems, KvBounds bd) {
  const int chunks = row_elems >> 3;  // 16-byte chunks per token
  const long total = (long)T * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks);
    const int c = (int)(i % chunks) * 8;
    const int s = slot[t];
    if (s < 0) continue;
    if (!OMNI_IN_BOUNDS(bd.num_slots == 0 || s < bd.num_slots, bd.status, KID_KV_WRITE)) continue;
    *reinterpret_cast<uint4*>(kc + (size_t)s * row_elems + c) = *reinterpret_cast<const uint4*>(k + (size_t)t * ldk + c);
    *reinterpret_cast<uint4*>(vc + (size_t)s * row_elems + c) = *reinterpret_cast<const uint4*>(v + (size_t)t * ldv + c);
  }
}

// --------------------------------------------------------------------------- gather
// out_k/out_v: [T, row_elems]; token t of the sequence lives in page block_table[t / bs].
__global__ void __launch_bounds__(256)
kv_gather_kernel(const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                 const int* __restrict__ block_table, int block_size, int T, int row_elems,
                 __nv_bfloat16* __restrict__ out_k, __nv_bfloat16* __restrict__ out_v, KvBounds bd) {
  const int chunks = row_elems >> 3;
  const long total = (long)T * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks);
    const int c = (int)(i % chunks) * 8;
    const int blk = block_table[t / block_size];
    if (!OMNI_IN_BOUNDS(blk >= 0 && (bd.num_blocks == 0 || blk < bd.num_blocks), bd.status, KID_KV_GATHER)) continue;
    const size_t s = (size_t)blk * block_size + (t % block_size);
    *reinterpret_cast<uint4*>(out_k + (size_t)t * row_elems + c) = *reinterpret_cast<const uint4*>(kc + s * row_elems + c);
    *reinterpret_cast<uint4*>(out_v + (size_t)t * row_elems + c) = *reinterpret_cast<const uint4*>(vc + s * row_elems + c);
  }
}

// --------------------------------------------------------------------- paged decode
// CUDA-core fallback for page shapes the tcgen05 path (attention_sm100.cu, omni_attn_fwd_paged)
// does not take.  grid = (num_seqs, Hkv, num_splits), 128 threads.  The CTA serves the
// G = H/Hkv query heads that share one KV head.  Half a warp owns one token (16 lanes x 8 dims,
// one 16-byte load per lane); scores of the G heads are reduced with butterfly shuffles inside the
// half-warp, then an online softmax keeps (m, l, acc[8]) per head; the 8 half-warp streams are
// merged through shared memory and the splits by a second kernel.
constexpr int PD_D = 128;
constexpr int PD_WARPS = 4;

template <int G>
__global__ void __launch_bounds__(PD_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long q_rs, const __nv_bfloat16* __restrict__ kc,
                    const __nv_bfloat16* __restrict__ vc, const int* __restrict__ block_tables, int max_blocks,
                    const int* __restrict__ seq_lens, int block_size, int Hkv, float scale_log2,
                    float* __restrict__ part_o, float* __restrict__ part_ml, int num_splits) {
  // Half a warp (16 lanes x 8 dims, one 16-byte load per lane) owns one token; a warp handles two
  // tokens per load instruction and two such instructions are in flight per iteration, so 8 half-
  // warps x 2 = 16 tokens of K and V are being fetched per CTA at any time.
  const int seq = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int l16 = lane & 15, sub = lane >> 4;
  const int grp = warp * 2 + sub;                 // 0..7: token stream of this half-warp
  constexpr int NG = PD_WARPS * 2;
  const int len = seq_lens[seq];
  const int per = (len + num_splits - 1) / num_splits;
  const int t0 = split * per, t1 = min(len, t0 + per);
  const int H = Hkv * G;
  float qv[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 u = *reinterpret_cast<const uint4*>(q + (size_t)seq * q_rs + (size_t)(hk * G + g) * PD_D + l16 * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      qv[g][2 * j] = f.x * scale_log2;
      qv[g][2 * j + 1] = f.y * scale_log2;
    }
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }
  const int* bt = block_tables + (size_t)seq * max_blocks;
  const size_t row = (size_t)Hkv * PD_D;
  // The trip count is the same for every thread of the CTA (the shuffles below name all 32
  // lanes, so the two half-warps must not leave the loop at different times); tokens past the
  // end of the split are loaded from a valid address and ignored.
  for (int tb0 = t0; tb0 < t1; tb0 += 2 * NG) {
    uint4 ku[2], vu[2];
    bool ok[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int t = tb0 + grp + u * NG;
      ok[u] = t < t1;
      const int tt = ok[u] ? t : t0;
      const size_t s = ((size_t)bt[tt / block_size] * block_size + (tt % block_size)) * row + (size_t)hk * PD_D + l16 * 8;
      ku[u] = *reinterpret_cast<const uint4*>(kc + s);
      vu[u] = *reinterpret_cast<const uint4*>(vc + s);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float kf[8], vf[8];
      {
        const uint32_t kw[4] = {ku[u].x, ku[u].y, ku[u].z, ku[u].w};
        const uint32_t vw[4] = {vu[u].x, vu[u].y, vu[u].z, vu[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16(kw[j]), b = unpack_bf16(vw[j]);
          kf[2 * j] = a.x; kf[2 * j + 1] = a.y; vf[2 * j] = b.x; vf[2 * j + 1] = b.y;
        }
      }
      float sc[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qv[g][e], kf[e], d);
        sc[g] = d;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], o);
      }
      if (ok[u]) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float mn = fmaxf(m[g], sc[g]);
          const float a = exp2f(m[g] - mn);
          const float p = exp2f(sc[g] - mn);
          l[g] = l[g] * a + p;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(acc[g][e], a, p * vf[e]);
          m[g] = mn;
        }
      }
    }
  }
  // merge the 8 half-warp streams through shared memory
  __shared__ float s_m[NG][G], s_l[NG][G];
  __shared__ float s_acc[NG][G][PD_D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (l16 == 0) { s_m[grp][g] = m[g]; s_l[grp][g] = l[g]; }
    *reinterpret_cast<float4*>(&s_acc[grp][g][l16 * 8]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    *reinterpret_cast<float4*>(&s_acc[grp][g][l16 * 8 + 4]) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * PD_D; idx += blockDim.x) {
    const int g = idx / PD_D, d = idx % PD_D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NG; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < NG; ++w) {
      const float a = s_m[w][g] == -INFINITY ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * a;
      o += s_acc[w][g][d] * a;
    }
    const size_t pidx = ((size_t)seq * H + hk * G + g) * num_splits + split;
    part_o[pidx * PD_D + d] = o;
    if (d == 0) { part_ml[pidx * 2] = mm; part_ml[pidx * 2 + 1] = ll; }
  }
}

// merge the splits: out[seq, h, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
__global__ void __launch_bounds__(PD_D)
paged_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int num_splits,
                          __nv_bfloat16* __restrict__ out, long o_rs, int H) {
  const int seq = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const size_t base = ((size_t)seq * H + h) * num_splits;
  float mm = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float ll = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float a = ms == -INFINITY ? 0.f : exp2f(ms - mm);
    ll += part_ml[(base + s) * 2 + 1] * a;
    o += part_o[(base + s) * PD_D + d] * a;
  }
  out[(size_t)seq * o_rs + (size_t)h * PD_D + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
}

}  // namespace omni

using namespace omni;

// 1 when this library was compiled with -DOMNI_BOUNDS_CHECK
extern "C" int omni_kv_bounds_check_enabled(void) {
#ifdef OMNI_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" void omni_kv_set_bounds(long num_slots, int num_blocks, int* status) {
  g_kv_bounds.num_slots = num_slots;
  g_kv_bounds.num_blocks = num_blocks;
  g_kv_bounds.status = status;
}

extern "C" int omni_kv_write(const void* k, const void* v, long ldk, long ldv, void* kc, void* vc,
                             const int* slot, int T, int row_elems, void* stream) {
  if (T <= 0) return RC_OK;
  if ((row_elems & 7) || (ldk & 7) || (ldv & 7)) return RC_BAD_ARG;
  const long total = (long)T * (row_elems >> 3);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  kv_write_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldk, ldv, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, slot, T, row_elems,
      g_kv_bounds);
  return (int)cudaGetLastError();
}

extern "C" int omni_kv_gather(const void* kc, const void* vc, const int* block_table, int block_size, int T,
                              int row_elems, void* out_k, void* out_v, void* stream) {
  if (T <= 0) return RC_OK;
  if ((row_elems & 7) || block_size <= 0) return RC_BAD_ARG;
  const long total = (long)T * (row_elems >> 3);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  kv_gather_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, block_table, block_size, T, row_elems,
      (__nv_bfloat16*)out_k, (__nv_bfloat16*)out_v, g_kv_bounds);
  return (int)cudaGetLastError();
}

// Scratch the caller provides: part_o  float[num_seqs * H * num_splits * 128],
//                              part_ml float[num_seqs * H * num_splits * 2].
extern "C" int omni_paged_decode(const void* q, long q_rs, const void* kc, const void* vc, const int* block_tables,
                                 int max_blocks, const int* seq_lens, int num_seqs, int block_size, int H, int Hkv,
                                 int D, float scale, int num_splits, float* part_o, float* part_ml, void* out,
                                 long o_rs, void* stream) {
  if (num_seqs <= 0) return RC_OK;
  if (D != PD_D || Hkv <= 0 || H % Hkv || num_splits < 1) return RC_BAD_ARG;
  const int G = H / Hkv;
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(num_seqs, Hkv, num_splits);
  cudaStream_t st = (cudaStream_t)stream;
  auto qq = (const __nv_bfloat16*)q; auto k = (const __nv_bfloat16*)kc; auto v = (const __nv_bfloat16*)vc;
#define OMNI_PD(GG) paged_decode_kernel<GG><<<grid, PD_WARPS * 32, 0, st>>>(qq, q_rs, k, v, block_tables, max_blocks, seq_lens, block_size, Hkv, sl2, part_o, part_ml, num_splits)
  switch (G) {
    case 1: OMNI_PD(1); break;
    case 2: OMNI_PD(2); break;
    case 4: OMNI_PD(4); break;
    case 8: OMNI_PD(8); break;
    default: return RC_BAD_ARG;
  }
#undef OMNI_PD
  paged_decode_merge_kernel<<<dim3(num_seqs, H), PD_D, 0, st>>>(part_o, part_ml, num_splits, (__nv_bfloat16*)out, o_rs, H);
  return (int)cudaGetLastError();
}
