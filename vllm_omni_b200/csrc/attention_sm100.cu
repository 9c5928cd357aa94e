// K4 / K11: flash-attention forward for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// softmax(Q K^T * scale) V over bf16 inputs (non-causal, or causal with a query offset for
// chunked prefill), head_dim 128, optional per-batch key lengths (padding mask), GQA, optional
// log-sum-exp output (used by the ring / peer-KV merge), K/V either contiguous or in a paged cache
// addressed through a block table, optional split of the KV range over several CTAs with a
// merge kernel.  Replaces the PyTorch SDPA call the reference makes on Blackwell
// (vllm_omni/diffusion/attention/backends/sdpa.py:82; its FlashAttention backend is gated
// off for compute capability >= 10, vllm_omni/platforms/cuda/platform.py:44-51) and the paged
// attention it takes from vLLM for the AR stages (vllm_omni/worker/gpu_model_runner.py:37).
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles (one tile when the
// rows end inside the first; decode maps the heads of a GQA group onto the rows of a tile).
//   warp 0        TMA producer: Q once, then K and V tiles through two 2-deep rings; with a paged
//                 cache one box per page, page ids read from the block table
//   warp 1        MMA issuer (one elected thread):
//                   S_t = Q_t K_j^T      (SS form, both operands K-major in shared memory)
//                   O_t += P_t V_j       (TS form: P_t read from TMEM, V_j MN-major in smem)
//   warps 4-7     softmax of tile 0, warps 8-11 softmax of tile 1.  One THREAD owns one query row
//                 (TMEM lane): a single tcgen05.ld pass brings the row's 128 scores into
//                 registers, the row maximum needs no exchange with other threads, exp2 runs in
//                 packed fp32 (a quarter of the exponentials on an FMA-pipe polynomial), bf16 P is
//                 written back with tcgen05.st over the S columns, then the final O / l epilogue
//                 (local stores, peer stores for the fused Ulysses exchange, or fp32 partials
//                 for split-KV)
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t (bf16, two keys per
// column) sits in columns [0,64) of S_t.  O is rescaled lazily: only when a row maximum grows by
// more than 2^8, so the steady state never touches O outside the MMAs.
// The MMA stream is software-pipelined (PV_t(j) is followed at once by S_t(j+1)) so that
// the tensor pipe works on one tile while the other tile's softmax runs.  Every wait is bounded.
#include <stdlib.h>

#include "host_util.h"
#include "ptx_sm100.cuh"
#include "peer_signal.cuh"

namespace omni {

constexpr int ATT_D = 128;    // the larger of the two head sizes (64 and 128) the kernel is built for
constexpr int ATT_BM = 128;   // rows per query tile
constexpr int ATT_BN = 128;   // keys per KV tile
constexpr int ATT_THREADS = 384;  // TMA, MMA, 2 idle warps, 2 x 4 softmax warps (one row per thread)
constexpr int ATT_HALF_BYTES = ATT_BM * 64 * 2;     // one 64-wide TMA box of 128 rows: 16 KiB
// per head size D: a tile is D / 64 boxes; the K and V rings are 2 deep at D = 128 and 4 deep at D = 64
template <int D> struct AttCfg {
  static constexpr int TILE_BYTES = ATT_BM * D * 2;
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int SMEM = 2 * TILE_BYTES /*Q*/ + 2 * STAGES * TILE_BYTES /*K, V*/ + 1024;
};

struct AttnOut {
  __nv_bfloat16* o;   // rows [0, split) of every batch
  __nv_bfloat16* o2;  // rows [split, Sq) (row index s - split); nullptr -> everything in o
  long o_bs, o_rs, o_hs;     // element strides: batch, row, head
  long o2_bs, o2_rs, o2_hs;
  int split;
  float* lse;  // [B, H, Sq] or nullptr
  // Fused reverse all-to-all (Ulysses): with n_peers > 1 query row s < split belongs to rank
  // s / rows_per_rank and is stored, as local row s % rows_per_rank, through o_peers[that rank];
  // rows >= split use rows_per_rank2 / o2_peers the same way.  The pointers are peer (NVLink)
  // or local addresses that already include this rank's head offset.
  int n_peers;
  int rows_per_rank, rows_per_rank2;
  __nv_bfloat16* o_peers[16];
  __nv_bfloat16* o2_peers[16];
  // Split-KV: with kv_splits > 1 CTA (qblk, split) covers a contiguous share of the KV tiles and
  // stores the unnormalised fp32 O row, its reference exponent m (log2 units) and row sum l at
  // index ((b * H + h) * Sq + row) * kv_splits + split; a merge kernel combines the shares.
  int kv_splits;
  float* part_o;    // [.., kv_splits, 128]
  float* part_ml;   // [.., kv_splits, 2]
  // Continuation of an attention over another set of keys (sequence-parallel K/V shards): with
  // prev_o set, the epilogue blends this launch's normalised rows with the earlier result by their
  // log-sum-exps, out = prev + sigmoid(lse - prev_lse) (this - prev), and stores the combined LSE.
  // prev_o may alias o (every element is read and written by the same thread).
  const __nv_bfloat16* prev_o;
  const float* prev_lse;   // [B, H, Sq], natural-log units
  long p_bs, p_rs, p_hs;
};

// C view of the continuation operands (all strides in elements)
struct AttnPrev {
  const void* o;
  const float* lse;
  long rs, hs, bs;
};

// eight accumulator values scaled by `sb`, plus eight earlier bf16 values scaled by `wp`
__device__ __forceinline__ uint4 blend8(const uint32_t* v, float sb, uint4 pv, float wp) {
  const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pv);
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 pf = __bfloat1622float2(p2[j]);
    ow[j] = pack_bf16(fmaf(__uint_as_float(v[2 * j]), sb, pf.x * wp), fmaf(__uint_as_float(v[2 * j + 1]), sb, pf.y * wp));
  }
  return o;
}

// Paged K/V: the tensor maps cover the page pool as [num_blocks * block_size, Hkv, 128] and token
// t of batch row b lives in page block_table[b * bt_stride + t / block_size].
struct AttnPaging {
  const int* block_table;   // nullptr = contiguous K/V
  int bt_stride;
  int block_size;           // a multiple of 8 that divides 128
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Packed pairs of fp32 in one 64-bit register (add/mul/fma.f32x2 issue once for two values).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t r, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for a pair, on the FMA and integer pipes: n = round(x), r = x - n in [-0.5, 0.5],
// 2^r by a degree-3 polynomial (relative error 7.5e-5, far inside bf16's 2^-9), and n added
// into the exponent field.  x is clamped at -126 so the exponent cannot wrap.
__device__ __forceinline__ uint64_t exp2_poly2(uint64_t x2) {
  float x0, x1;
  unpack2(x2, x0, x1);
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  x2 = pack2(x0, x1);
  const uint64_t fl = add2(x2, pack2(12582912.f, 12582912.f));          // 1.5 * 2^23: integer in the low bits
  const uint64_t n = add2(fl, pack2(-12582912.f, -12582912.f));
  const uint64_t r = fma2(n, pack2(-1.f, -1.f), x2);
  uint64_t p = fma2(pack2(0.0551716685f, 0.0551716685f), r, pack2(0.2426111251f, 0.2426111251f));
  p = fma2(p, r, pack2(0.6932609677f, 0.6932609677f));
  p = fma2(p, r, pack2(0.9999280572f, 0.9999280572f));
  float p0, p1, f0, f1;
  unpack2(p, p0, p1);
  unpack2(fl, f0, f1);
  p0 = __int_as_float(__float_as_int(p0) + (__float_as_int(f0) << 23));
  p1 = __int_as_float(__float_as_int(p1) + (__float_as_int(f1) << 23));
  return pack2(p0, p1);
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// NH = how many times per KV tile the softmax warps hand P over to the MMA warp (4: every 32 keys,
// 2: every 64 keys, 1: once): earlier hand-offs let P*V start while the later exponentials of the
// tile are still being computed, at the price of one tcgen05.wait::st per hand-off.  Measured on
// B2 S4352 H24 (one box, medians): 4 hand-offs 0.396 ms, 1 hand-off 0.409 ms; packed-bf16 MUFU
// exponentials and polynomial shares of 0, 1/8, 3/8 and 1/2 were within 1 % of, or slower than,
// fp32 MUFU with a quarter of the pairs on the FMA-pipe polynomial.
template <int NH, int HD>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, AttnOut out, int Sq, int Skv, int H, int Hkv,
                const int* __restrict__ kv_lens, float scale_log2, int causal, int q_offset, AttnPaging pg,
                PeerSignal sig, int* status) {
  constexpr int ATT_TILE_BYTES = AttCfg<HD>::TILE_BYTES;
  constexpr int KV_STAGES = AttCfg<HD>::STAGES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, k_full[4], k_empty[4], v_full[4], v_empty[4];
  __shared__ __align__(8) uint64_t s_full[2], p_full[2][4], o_done[2];   // p_full: per 32-key chunk of P
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int splits = out.kv_splits > 1 ? out.kv_splits : 1;
  const int qblk = blockIdx.x / splits, split = blockIdx.x - qblk * splits;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (H / Hkv);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;                         // 2 tiles
  const uint32_t sK = smem_base + 2 * ATT_TILE_BYTES;                    // KV_STAGES tiles
  const uint32_t sV = smem_base + (2 + KV_STAGES) * ATT_TILE_BYTES;      // KV_STAGES tiles
  const int kv_len = kv_lens ? min(kv_lens[b], Skv) : Skv;
  // causal: query row s sees keys [0, s + q_offset]; the CTA only visits tiles its last row sees
  const int kv_cta = causal ? min(kv_len, qblk * 2 * ATT_BM + 2 * ATT_BM + q_offset) : kv_len;
  const int n_kv_all = (kv_cta + ATT_BN - 1) / ATT_BN;
  const int per_split = (n_kv_all + splits - 1) / splits;
  const int j0 = min(n_kv_all, split * per_split);       // this CTA's KV tiles: [j0, j0 + n_kv)
  const int n_kv = min(n_kv_all, j0 + per_split) - j0;
  // query tiles in use: the second one is skipped when this block's rows end inside the first
  const int n_qt = (Sq - qblk * 2 * ATT_BM > ATT_BM) ? 2 : 1;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&k_empty[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      mbar_init(smem_u32(&v_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_full[i]), 1);
      for (int c = 0; c < 4; ++c) mbar_init(smem_u32(&p_full[i][c]), 4);   // one arrival per softmax warp
      mbar_init(smem_u32(&o_done[i]), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one() && n_kv > 0) {
      const uint32_t qb = smem_u32(&q_full);
      mbar_expect_tx(qb, 2 * ATT_TILE_BYTES);
      for (int t = 0; t < 2; ++t) {
        const int s0 = qblk * 2 * ATT_BM + t * ATT_BM;
#pragma unroll
        for (int x = 0; x < HD / 64; ++x)
          tma_load_4d(sQ + t * ATT_TILE_BYTES + x * ATT_HALF_BYTES, &tmQ, qb, 64 * x, s0, h, b);
      }
      const int* bt = pg.block_table ? pg.block_table + (long)b * pg.bt_stride : nullptr;
      const int last_page = bt ? max(0, (kv_len + pg.block_size - 1) / pg.block_size - 1) : 0;
      const int pages_per_tile = bt ? ATT_BN / pg.block_size : 0;
      const uint32_t page_bytes = bt ? (uint32_t)pg.block_size * 128u : 0u;   // per 64-wide half
      for (int jj = 0; jj < n_kv; ++jj) {
        const int j = j0 + jj;
        const int st = jj % KV_STAGES;
        const uint32_t ph = (jj / KV_STAGES) & 1;
        mbar_wait(smem_u32(&k_empty[st]), ph ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
        const uint32_t kb = smem_u32(&k_full[st]);
        mbar_expect_tx(kb, ATT_TILE_BYTES);
        if (bt) {
          // one box of block_size rows per page; pages past the sequence's last one re-read the
          // last page (finite data that the key mask discards)
          for (int i = 0; i < pages_per_tile; ++i) {
            const int page = bt[min(j * pages_per_tile + i, last_page)];
#pragma unroll
            for (int x = 0; x < HD / 64; ++x)
              tma_load_4d(sK + st * ATT_TILE_BYTES + x * ATT_HALF_BYTES + i * page_bytes, &tmK, kb, 64 * x,
                          page * pg.block_size, hkv, 0);
          }
        } else {
#pragma unroll
          for (int x = 0; x < HD / 64; ++x)
            tma_load_4d(sK + st * ATT_TILE_BYTES + x * ATT_HALF_BYTES, &tmK, kb, 64 * x, j * ATT_BN, hkv, b);
        }
        mbar_wait(smem_u32(&v_empty[st]), ph ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
        const uint32_t vb = smem_u32(&v_full[st]);
        mbar_expect_tx(vb, ATT_TILE_BYTES);
        if (bt) {
          for (int i = 0; i < pages_per_tile; ++i) {
            const int page = bt[min(j * pages_per_tile + i, last_page)];
#pragma unroll
            for (int x = 0; x < HD / 64; ++x)
              tma_load_4d(sV + st * ATT_TILE_BYTES + x * ATT_HALF_BYTES + i * page_bytes, &tmV, vb, 64 * x,
                          page * pg.block_size, hkv, 0);
          }
        } else {
#pragma unroll
          for (int x = 0; x < HD / 64; ++x)
            tma_load_4d(sV + st * ATT_TILE_BYTES + x * ATT_HALF_BYTES, &tmV, vb, 64 * x, j * ATT_BN, hkv, b);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one() && n_kv > 0) {
      constexpr uint32_t idesc_qk = umma_idesc(ATT_BM, ATT_BN, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(ATT_BM, HD, 1, 1, 0, 1);  // V is MN-major, N = head size
      // The issuing thread is a serial resource: the shared-memory descriptors are built ONCE; a
      // tile, a ring stage or a K step is a constant added to the 14-bit address field (16-byte units).
      constexpr uint64_t TILE16 = ATT_TILE_BYTES >> 4, HALF16 = ATT_HALF_BYTES >> 4;
      const uint64_t dQ = umma_desc_kmajor_sw128(sQ);
      const uint64_t dK = umma_desc_kmajor_sw128(sK);
      const uint64_t dV = umma_desc_sw128(sV, ATT_HALF_BYTES, 1024);
      auto issue_s = [&](int t, int st) {
        const uint32_t d = tmem_base + t * 128;
        const uint64_t a0 = dQ + (uint64_t)t * TILE16, b0 = dK + (uint64_t)st * TILE16;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t off = (uint64_t)((k >> 2) * HALF16 + (k & 3) * 2);   // 16 bf16 = 32 bytes along K
          mma_f16_ss(d, a0 + off, b0 + off, idesc_qk, k == 0 ? 0u : 1u);
        }
      };
      // P*V for the 32 keys of chunk c (two K=16 steps); the chunks of one KV tile are issued as the
      // softmax warps hand them over, so the tensor pipe starts on P*V while later exponentials
      // of the same tile are still being computed
      auto issue_pv_chunk = [&](int t, uint64_t v0, uint32_t first, int c) {
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t p = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int k = 2 * c + kk;
          // 16 keys = two 8-row groups of 1024 B (2048 B per K step); the two 64-wide halves of D are
          // ATT_HALF_BYTES apart (the descriptor's leading-dimension offset).  P of keys
          // [16k, 16k + 16) sits in columns [8k, 8k + 8) of the S block.
          mma_f16_ts(d, p + k * 8, v0 + (uint64_t)(k * 128), idesc_pv, k == 0 ? first : 1u);
        }
      };
      mbar_wait(smem_u32(&q_full), 0, &s_abort, status, ERR_WAIT_FULL);
      mbar_wait(smem_u32(&k_full[0]), 0, &s_abort, status, ERR_WAIT_FULL);
      tc_fence_after_sync();
      for (int t = 0; t < n_qt; ++t) {
        issue_s(t, 0);
        tc_commit(smem_u32(&s_full[t]));
      }
      tc_commit(smem_u32(&k_empty[0]));
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const bool more = j + 1 < n_kv;
        const int st1 = (j + 1) % KV_STAGES;
        mbar_wait(smem_u32(&v_full[st]), ph, &s_abort, status, ERR_WAIT_FULL);
        if (more) mbar_wait(smem_u32(&k_full[st1]), ((j + 1) / KV_STAGES) & 1, &s_abort, status, ERR_WAIT_FULL);
        const uint64_t v0 = dV + (uint64_t)st * TILE16;
        const uint32_t first = j != 0 ? 1u : 0u;      // the first P*V of a tile overwrites O
        for (int t = 0; t < n_qt; ++t) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            mbar_wait(smem_u32(&p_full[t][c]), j & 1, &s_abort, status, ERR_WAIT_SOFTMAX);
            tc_fence_after_sync();
            issue_pv_chunk(t, v0, first, c);
          }
          if (more) {
            issue_s(t, st1);
            tc_commit(smem_u32(&s_full[t]));
          } else {
            tc_commit(smem_u32(&o_done[t]));
          }
        }
        tc_commit(smem_u32(&v_empty[st]));
        if (more) tc_commit(smem_u32(&k_empty[st1]));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------- softmax + epilogue
    // Four warps per query tile; warp (warp % 4) owns TMEM lanes [32 (warp % 4), +32), i.e. one
    // thread per query row, all 128 keys of the KV tile.
    const int t = (warp - 4) >> 2;       // query tile of this warp
    const int q = warp & 3;              // TMEM lane quadrant this warp may access
    const int row_in_tile = q * 32 + lane;
    const int srow = qblk * 2 * ATT_BM + t * ATT_BM + row_in_tile;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + t * 128;           // P overwrites the first 64 of these
    const uint32_t tO = tmem_base + lane_addr + 256 + t * 128;
    const uint64_t scale2 = pack2(scale_log2, scale_log2);
    float m = -INFINITY;  // running maximum in log2 units that P and l are relative to
    uint64_t l2a = 0ull, l2b = 0ull;     // four partial row sums (two packed pairs)
    // A tile that is not in use has no work at all; a warp whose 32 rows all lie past the last
    // query row (decode: a handful of real rows per tile) only keeps the barrier protocol going.
    // Its rows of S come from zero-filled Q rows, so the stale bits the P*V MMA reads as their P
    // are zeros, and nothing of those rows is stored.
    const bool tile_used = t < n_qt;
    const bool rows_used = tile_used && (srow - lane) < Sq;
    for (int j = 0; tile_used && j < n_kv; ++j) {
      mbar_wait(smem_u32(&s_full[t]), j & 1, &s_abort, status, ERR_WAIT_FULL);
      if (!rows_used) {
        if (lane == 0)
          for (int c = 0; c < 4; ++c) mbar_arrive(smem_u32(&p_full[t][c]));
        continue;
      }
      tc_fence_after_sync();
      const int row_limit = causal ? min(kv_len, srow + q_offset + 1) : kv_len;
      const int valid = row_limit - (j0 + j) * ATT_BN;   // keys of this tile this row may see
      const bool any_masked = __any_sync(0xffffffffu, valid < ATT_BN);
      // the whole row of scores in registers: one TMEM pass
      uint32_t v0[32], v1[32], v2[32], v3[32];
      auto load_scores = [&]() {
        tmem_ld_32x32(tS, v0);
        tmem_ld_32x32(tS + 32, v1);
        tmem_ld_32x32(tS + 64, v2);
        tmem_ld_32x32(tS + 96, v3);
        tmem_wait_ld();
        if (any_masked) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            if (e >= valid) v0[e] = 0xff800000u;  // -inf
            if (e + 32 >= valid) v1[e] = 0xff800000u;
            if (e + 64 >= valid) v2[e] = 0xff800000u;
            if (e + 96 >= valid) v3[e] = 0xff800000u;
          }
        }
      };
      load_scores();
      float mx;
      {
        float m0 = __uint_as_float(v0[0]), m1 = __uint_as_float(v1[0]);
        float m2 = __uint_as_float(v2[0]), m3 = __uint_as_float(v3[0]);
#pragma unroll
        for (int e = 1; e < 31; e += 2) {
          m0 = max3(m0, __uint_as_float(v0[e]), __uint_as_float(v0[e + 1]));
          m1 = max3(m1, __uint_as_float(v1[e]), __uint_as_float(v1[e + 1]));
          m2 = max3(m2, __uint_as_float(v2[e]), __uint_as_float(v2[e + 1]));
          m3 = max3(m3, __uint_as_float(v3[e]), __uint_as_float(v3[e + 1]));
        }
        m0 = fmaxf(m0, __uint_as_float(v0[31]));
        m1 = fmaxf(m1, __uint_as_float(v1[31]));
        m2 = fmaxf(m2, __uint_as_float(v2[31]));
        m3 = fmaxf(m3, __uint_as_float(v3[31]));
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * scale_log2;
      }
      const float m_new = fmaxf(m, mx);
      // lazy rescale, decided per warp because tcgen05.ld/st are warp-wide
      const bool grow = m_new > m + 8.0f;
      if (j == 0) {
        m = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        const float alpha = ex2(m - m_new);
        const uint64_t alpha2 = pack2(alpha, alpha);
        l2a = mul2(l2a, alpha2);
        l2b = mul2(l2b, alpha2);
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
          tmem_st_32x32(tO + c * 32, v);
        }
        tmem_wait_st();
        m = m_new;
        load_scores();   // rare path: the scores were dropped to make room for the O chunks; read them again
      }
      // P = exp2(S * scale - m) as packed bf16 over the first 64 columns of the S block.  One pair
      // in four goes through a degree-3 polynomial on the FMA pipe instead of the MUFU unit,
      // which is otherwise as busy as the tensor pipe at head_dim 128.
      const float m_use = m == -INFINITY ? 0.f : m;
      const uint64_t negm2 = pack2(-m_use, -m_use);
      auto softmax_chunk = [&](uint32_t (&v)[32], int c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const uint64_t x2 = fma2(pack2(__uint_as_float(v[e]), __uint_as_float(v[e + 1])), scale2, negm2);
          float p0, p1;
          uint64_t p2;
          if ((e & 6) == 6) {
            p2 = exp2_poly2(x2);
            unpack2(p2, p0, p1);
          } else {
            unpack2(x2, p0, p1);
            p0 = ex2(p0);
            p1 = ex2(p1);
            p2 = pack2(p0, p1);
          }
          if (e & 2) l2b = add2(l2b, p2); else l2a = add2(l2a, p2);
          pk[e >> 1] = pack_bf16(p0, p1);
        }
        tmem_st_32x16(tS + c * 16, pk);
        if (((c + 1) * NH) % 4 == 0) {
          // hand the keys finished so far to the MMA warp: every lane's stores are complete, then
          // ONE lane arrives for the warp (128 separate arrivals would serialise on the barrier)
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0)
            for (int cc = c + 1 - 4 / NH; cc <= c; ++cc) mbar_arrive(smem_u32(&p_full[t][cc]));
        }
      };
      softmax_chunk(v0, 0);
      softmax_chunk(v1, 1);
      softmax_chunk(v2, 2);
      softmax_chunk(v3, 3);
    }
    // epilogue: O / l -> bf16
    if (rows_used) {
      float l;
      {
        float a0, a1, b0, b1;
        unpack2(l2a, a0, a1);
        unpack2(l2b, b0, b1);
        l = (a0 + a1) + (b0 + b1);
      }
      if (n_kv > 0) {
        mbar_wait(smem_u32(&o_done[t]), 0, &s_abort, status, ERR_WAIT_PV);
        tc_fence_after_sync();
      }
      if (out.kv_splits > 1) {
        // split-KV share: unnormalised O, reference exponent and row sum for the merge kernel
        const long pidx = (((long)b * H + h) * Sq + srow) * out.kv_splits + split;
        if (srow < Sq) {
          out.part_ml[pidx * 2] = n_kv > 0 ? m : -INFINITY;
          out.part_ml[pidx * 2 + 1] = l;
        }
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          if (n_kv > 0) {
            tmem_ld_32x32(tO + c * 32, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          if (srow < Sq) {
            float4* dst = reinterpret_cast<float4*>(out.part_o + pidx * HD + c * 32);
#pragma unroll
            for (int g = 0; g < 8; ++g)
              dst[g] = make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]),
                                   __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
          }
        }
      } else {
        float inv_l = l > 0.f ? 1.0f / l : 0.f;
        float lse_row = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        float wp = 0.f;                          // weight of the earlier result (continuation launches)
        const __nv_bfloat16* prow = nullptr;
        if (out.prev_o != nullptr && srow < Sq) {
          const float lp = out.prev_lse[((long)b * H + h) * Sq + srow];
          prow = out.prev_o + (long)b * out.p_bs + (long)srow * out.p_rs + (long)h * out.p_hs;
          if (!(l > 0.f)) {                      // no key seen here: the earlier result stands
            wp = 1.f;
            lse_row = lp;
          } else if (lp != -INFINITY) {
            const float d = lse_row - lp;
            const float wb = 1.0f / (1.0f + __expf(-d));
            wp = 1.0f - wb;
            inv_l *= wb;
            lse_row = fmaxf(lse_row, lp) + log1pf(__expf(-fabsf(d)));
          }
        }
        if (srow < Sq && out.lse) out.lse[((long)b * H + h) * Sq + srow] = lse_row;
        if (out.n_peers > 1) {
          // Fused exchange: rows go to their owner ranks over NVLink.  A store from the thread that
          // owns the row would put 32 separate 16-byte writes on the link per instruction, so the
          // warp's 32 rows pass through shared memory (the Q tile of this query tile is no longer
          // read once o_done has fired), 64 columns at a time, and leave as whole 128-byte row
          // segments: 8 lanes per row, 4 rows per store instruction.
          const uint32_t stg = sQ + t * ATT_TILE_BYTES + q * 4096;
          const int k = lane & 7;
          const int row_base = qblk * 2 * ATT_BM + t * ATT_BM + q * 32;
#pragma unroll 1
          for (int hf = 0; hf < HD / 64; ++hf) {
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
              uint32_t v[32];
              if (n_kv > 0) {
                tmem_ld_32x32(tO + hf * 64 + c * 32, v);
                tmem_wait_ld();
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = 0u;
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 o;
                if (prow) {
                  o = blend8(v + g * 8, inv_l, *reinterpret_cast<const uint4*>(prow + hf * 64 + c * 32 + g * 8), wp);
                } else {
                  o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
                  o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
                  o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
                  o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
                }
                const int kk = c * 4 + g;
                st_shared_v4(stg + lane * 128 + ((kk ^ (lane & 7)) << 4), o);
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              const int sr = row_base + r;
              if (sr < Sq) {
                __nv_bfloat16* dst;
                if (sr >= out.split) {
                  const int t2 = sr - out.split;
                  const int owner = t2 / out.rows_per_rank2;
                  dst = out.o2_peers[owner] + (long)b * out.o2_bs + (long)(t2 - owner * out.rows_per_rank2) * out.o2_rs + (long)h * out.o2_hs;
                } else {
                  const int owner = sr / out.rows_per_rank;
                  dst = out.o_peers[owner] + (long)b * out.o_bs + (long)(sr - owner * out.rows_per_rank) * out.o_rs + (long)h * out.o_hs;
                }
                const uint4 val = ld_shared_v4(stg + r * 128 + ((k ^ (r & 7)) << 4));
                *reinterpret_cast<uint4*>(dst + hf * 64 + k * 8) = val;
              }
            }
            __syncwarp();
          }
        } else {
          __nv_bfloat16* orow = nullptr;
          if (srow < Sq) {
            if (out.o2 && srow >= out.split)
              orow = out.o2 + (long)b * out.o2_bs + (long)(srow - out.split) * out.o2_rs + (long)h * out.o2_hs;
            else
              orow = out.o + (long)b * out.o_bs + (long)srow * out.o_rs + (long)h * out.o_hs;
          }
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t v[32];
            if (n_kv > 0) {
              tmem_ld_32x32(tO + c * 32, v);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] = 0u;
            }
            if (orow) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 o;
                if (prow) {
                  o = blend8(v + g * 8, inv_l, *reinterpret_cast<const uint4*>(prow + c * 32 + g * 8), wp);
                } else {
                  o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
                  o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
                  o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
                  o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
                }
                *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  // every peer store of this CTA was issued before the barrier above
  if (threadIdx.x == 0) peer_signal_cta_done(sig, gridDim.x * gridDim.y * gridDim.z);
  if (s_abort) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// out[b, row, h, :] = sum_s 2^(m_s - m*) O_s / sum_s 2^(m_s - m*) l_s over the split-KV shares
__global__ void __launch_bounds__(ATT_D)      // launched with D (64 or 128) threads
attn_merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                         __nv_bfloat16* __restrict__ o, long o_bs, long o_rs, long o_hs, float* __restrict__ lse,
                         int H, int Sq) {
  const long r = blockIdx.x;            // (b * H + h) * Sq + row
  const int d = threadIdx.x;
  const int row = (int)(r % Sq);
  const int h = (int)((r / Sq) % H);
  const long b = r / ((long)Sq * H);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(r * splits + s) * 2]);
  float ll = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(r * splits + s) * 2];
    const float a = ms == -INFINITY ? 0.f : exp2f(ms - mm);
    ll += part_ml[(r * splits + s) * 2 + 1] * a;
    acc += part_o[(r * splits + s) * blockDim.x + d] * a;
  }
  o[b * o_bs + (long)row * o_rs + (long)h * o_hs + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  if (lse && d == 0) lse[r] = ll > 0.f ? (mm + log2f(ll)) * 0.6931471805599453f : -INFINITY;
}

static int make_qkv_tmap(CUtensorMap* tm, const void* p, int S, int Hn, int B, long rs, long hs, long bs,
                         int box_rows = ATT_BM, int D = ATT_D) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return RC_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(p) & 15) || (rs & 7) || (hs & 7) || (bs & 7)) return RC_BAD_ARG;
  cuuint64_t gdim[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)Hn, (cuuint64_t)B};
  cuuint64_t gstr[3] = {(cuuint64_t)rs * 2, (cuuint64_t)hs * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(p), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RC_OK : RC_TMAP;
}

static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, AttnOut& out, int B, int H,
                       int Hkv, int Sq, int Skv, const int* kv_lens, float scale, int causal, int q_offset,
                       const AttnPaging& pg, int* status, cudaStream_t stream, const OmniSync* sync = nullptr,
                       int D = ATT_D) {
  // OMNI_ATTN_HANDOFFS (4 | 2 | 1): tuning switch, see attn_fwd_kernel
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, AttnOut, int, int, int, int, const int*,
                           float, int, int, AttnPaging, PeerSignal, int*);
  static KernelFn fns[2] = {nullptr, nullptr};     // [0]: head size 64, [1]: head size 128
  const int di = D == 64 ? 0 : 1;
  if (fns[di] == nullptr) {
    const char* ev = getenv("OMNI_ATTN_HANDOFFS");
    const int want = ev ? atoi(ev) : 4;
    KernelFn f;
    if (di == 0) f = want == 1 ? attn_fwd_kernel<1, 64> : (want == 2 ? attn_fwd_kernel<2, 64> : attn_fwd_kernel<4, 64>);
    else f = want == 1 ? attn_fwd_kernel<1, 128> : (want == 2 ? attn_fwd_kernel<2, 128> : attn_fwd_kernel<4, 128>);
    fns[di] = f;
  }
  static unsigned long long prepared[2] = {0, 0};
  if (int e = ensure_dynamic_smem((const void*)fns[di], di == 0 ? AttCfg<64>::SMEM : AttCfg<128>::SMEM, prepared[di])) return e;
  const int splits = out.kv_splits > 1 ? out.kv_splits : 1;
  dim3 grid(((Sq + 2 * ATT_BM - 1) / (2 * ATT_BM)) * splits, H, B);
  const float scale_log2 = scale * 1.4426950408889634f;
  PeerSignal sig;
  PeerWait unused;
  unpack_sync(sync, sig, unused);
  fns[di]<<<grid, ATT_THREADS, di == 0 ? AttCfg<64>::SMEM : AttCfg<128>::SMEM, stream>>>(
      tq, tk, tv, out, Sq, Skv, H, Hkv, kv_lens, scale_log2, causal, q_offset, pg, sig, status);
  return (int)cudaGetLastError();
}

}  // namespace omni

// Strides are in elements: *_rs between consecutive sequence positions, *_hs between heads,
// *_bs between batches; head_dim (128) is contiguous.  o2/split route query rows >= split
// of every batch to a second tensor (used to hand text and image rows to their own
// projections).  kv_lens: optional int32[B] valid key counts.  lse: optional fp32 [B,H,Sq].
// `sync` (may be null): the arrival this launch reports to the group once its peer stores are out
// (see peer_signal.cuh); only the signalling half is used.
extern "C" int omni_attn_fwd_cont(const void* q, long q_rs, long q_hs, long q_bs, const void* k, long k_rs,
                                  long k_hs, long k_bs, const void* v, long v_rs, long v_hs, long v_bs,
                                  void* o, long o_rs, long o_hs, long o_bs, void* o2, long o2_rs, long o2_hs,
                                  long o2_bs, int split, float* lse, int B, int H, int Hkv, int Sq, int Skv,
                                  int D, const int* kv_lens, float scale, int causal, int q_offset, int n_peers,
                                  int rows_per_rank,
                                  int rows_per_rank2, void* const* o_peers, void* const* o2_peers,
                                  const omni::AttnPrev* prev, const omni::OmniSync* sync, int* status, void* stream);

extern "C" int omni_attn_fwd_sync(const void* q, long q_rs, long q_hs, long q_bs, const void* k, long k_rs,
                                  long k_hs, long k_bs, const void* v, long v_rs, long v_hs, long v_bs,
                                  void* o, long o_rs, long o_hs, long o_bs, void* o2, long o2_rs, long o2_hs,
                                  long o2_bs, int split, float* lse, int B, int H, int Hkv, int Sq, int Skv,
                                  int D, const int* kv_lens, float scale, int causal, int q_offset, int n_peers,
                                  int rows_per_rank,
                                  int rows_per_rank2, void* const* o_peers, void* const* o2_peers,
                                  const omni::OmniSync* sync, int* status, void* stream) {
  return omni_attn_fwd_cont(q, q_rs, q_hs, q_bs, k, k_rs, k_hs, k_bs, v, v_rs, v_hs, v_bs, o, o_rs, o_hs, o_bs, o2,
                            o2_rs, o2_hs, o2_bs, split, lse, B, H, Hkv, Sq, Skv, D, kv_lens, scale, causal, q_offset,
                            n_peers, rows_per_rank, rows_per_rank2, o_peers, o2_peers, nullptr, sync, status, stream);
}

// `prev` (may be null): result and LSE of an attention of the same queries over other keys; this
// launch's output is the combination of both (see AttnOut::prev_o).  Needs `lse` when the caller
// goes on combining.
extern "C" int omni_attn_fwd_cont(const void* q, long q_rs, long q_hs, long q_bs, const void* k, long k_rs,
                                  long k_hs, long k_bs, const void* v, long v_rs, long v_hs, long v_bs,
                                  void* o, long o_rs, long o_hs, long o_bs, void* o2, long o2_rs, long o2_hs,
                                  long o2_bs, int split, float* lse, int B, int H, int Hkv, int Sq, int Skv,
                                  int D, const int* kv_lens, float scale, int causal, int q_offset, int n_peers,
                                  int rows_per_rank,
                                  int rows_per_rank2, void* const* o_peers, void* const* o2_peers,
                                  const omni::AttnPrev* prev, const omni::OmniSync* sync, int* status, void* stream) {
  using namespace omni;
  if ((D != 64 && D != 128) || H <= 0 || Hkv <= 0 || (H % Hkv) || B <= 0) return RC_BAD_ARG;
  if (prev && (prev->o == nullptr || prev->lse == nullptr || (prev->rs & 7) || (prev->hs & 7) || (prev->bs & 7) ||
               (reinterpret_cast<uintptr_t>(prev->o) & 15)))
    return RC_BAD_ARG;
  if (Sq <= 0) return RC_OK;
  if ((o_rs & 7) || (o_hs & 7) || (o_bs & 7) || (o2_rs & 7) || (o2_hs & 7) || (o2_bs & 7)) return RC_BAD_ARG;
  CUtensorMap tq, tk, tv;
  int rc = make_qkv_tmap(&tq, q, Sq, H, B, q_rs, q_hs, q_bs, ATT_BM, D);
  if (rc) return rc;
  rc = make_qkv_tmap(&tk, k, Skv, Hkv, B, k_rs, k_hs, k_bs, ATT_BM, D);
  if (rc) return rc;
  rc = make_qkv_tmap(&tv, v, Skv, Hkv, B, v_rs, v_hs, v_bs, ATT_BM, D);
  if (rc) return rc;
  AttnOut out;
  out.o = (__nv_bfloat16*)o; out.o2 = (__nv_bfloat16*)o2;
  out.o_bs = o_bs; out.o_rs = o_rs; out.o_hs = o_hs;
  out.o2_bs = o2_bs; out.o2_rs = o2_rs; out.o2_hs = o2_hs;
  out.split = split; out.lse = lse;
  out.n_peers = 0; out.rows_per_rank = 1; out.rows_per_rank2 = 1;
  for (int i = 0; i < 16; ++i) { out.o_peers[i] = nullptr; out.o2_peers[i] = nullptr; }
  if (n_peers > 1) {
    if (n_peers > 16 || rows_per_rank <= 0 || o_peers == nullptr) return RC_BAD_ARG;
    if (split < Sq && (rows_per_rank2 <= 0 || o2_peers == nullptr)) return RC_BAD_ARG;
    out.n_peers = n_peers; out.rows_per_rank = rows_per_rank; out.rows_per_rank2 = rows_per_rank2 > 0 ? rows_per_rank2 : 1;
    for (int i = 0; i < n_peers; ++i) {
      out.o_peers[i] = (__nv_bfloat16*)o_peers[i];
      out.o2_peers[i] = o2_peers ? (__nv_bfloat16*)o2_peers[i] : nullptr;
    }
  }
  out.kv_splits = 1; out.part_o = nullptr; out.part_ml = nullptr;
  out.prev_o = nullptr; out.prev_lse = nullptr; out.p_bs = out.p_rs = out.p_hs = 0;
  if (prev) {
    out.prev_o = static_cast<const __nv_bfloat16*>(prev->o); out.prev_lse = prev->lse;
    out.p_rs = prev->rs; out.p_hs = prev->hs; out.p_bs = prev->bs;
  }
  AttnPaging pg = {nullptr, 0, 0};
  return launch_attn(tq, tk, tv, out, B, H, Hkv, Sq, Skv, kv_lens, scale, causal, q_offset, pg, status,
                     (cudaStream_t)stream, sync, D);
}

extern "C" int omni_attn_fwd(const void* q, long q_rs, long q_hs, long q_bs, const void* k, long k_rs,
                             long k_hs, long k_bs, const void* v, long v_rs, long v_hs, long v_bs,
                             void* o, long o_rs, long o_hs, long o_bs, void* o2, long o2_rs, long o2_hs,
                             long o2_bs, int split, float* lse, int B, int H, int Hkv, int Sq, int Skv,
                             int D, const int* kv_lens, float scale, int causal, int q_offset, int n_peers,
                             int rows_per_rank,
                             int rows_per_rank2, void* const* o_peers, void* const* o2_peers, int* status,
                             void* stream) {
  return omni_attn_fwd_sync(q, q_rs, q_hs, q_bs, k, k_rs, k_hs, k_bs, v, v_rs, v_hs, v_bs, o, o_rs, o_hs, o_bs, o2,
                            o2_rs, o2_hs, o2_bs, split, lse, B, H, Hkv, Sq, Skv, D, kv_lens, scale, causal, q_offset,
                            n_peers, rows_per_rank, rows_per_rank2, o_peers, o2_peers, nullptr, status, stream);
}

// Attention over a paged KV cache.  k_pool / v_pool: [num_blocks, block_size, Hkv, 128] bf16;
// block_table: int32 [B, bt_stride] page ids; kv_lens: int32 [B] tokens per row.  Queries are
// addressed by strides exactly as in omni_attn_fwd, which covers both uses:
//   chunked prefill   q [T, H, 128] of one sequence: B = 1, Sq = T, causal with
//                     q_offset = kv_len - T
//   GQA decode        one token per sequence: the G = H / Hkv heads that share a KV head are the
//                     ROWS of a query tile (Sq = G, "heads" = Hkv, q_rs = 128, q_hs = G * 128,
//                     q_bs = token pitch), so one MMA serves the whole group
// kv_splits > 1 spreads the KV tiles of a row block over that many CTAs; part_o
// (float [B*H*Sq*kv_splits*128]) and part_ml (float [B*H*Sq*kv_splits*2]) are scratch.
extern "C" int omni_attn_fwd_paged(const void* q, long q_rs, long q_hs, long q_bs, const void* k_pool,
                                   const void* v_pool, int num_blocks, int block_size, const int* block_table,
                                   int bt_stride, void* o, long o_rs, long o_hs, long o_bs, float* lse, int B, int H,
                                   int Hkv, int Sq, int max_kv, const int* kv_lens, float scale, int causal,
                                   int q_offset, int kv_splits, float* part_o, float* part_ml, int* status,
                                   void* stream) {
  using namespace omni;
  if (H <= 0 || Hkv <= 0 || (H % Hkv) || B <= 0 || block_table == nullptr || kv_lens == nullptr) return RC_BAD_ARG;
  if (block_size < 8 || (block_size & 7) || (ATT_BN % block_size) || num_blocks <= 0) return RC_BAD_ARG;
  if (Sq <= 0 || max_kv <= 0) return RC_OK;
  if ((o_rs & 7) || (o_hs & 7) || (o_bs & 7)) return RC_BAD_ARG;
  if (kv_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return RC_BAD_ARG;
  CUtensorMap tq, tk, tv;
  int rc = make_qkv_tmap(&tq, q, Sq, H, B, q_rs, q_hs, q_bs);
  if (rc) return rc;
  const long pool_rows = (long)num_blocks * block_size;
  rc = make_qkv_tmap(&tk, k_pool, (int)pool_rows, Hkv, 1, (long)Hkv * ATT_D, ATT_D, pool_rows * Hkv * ATT_D, block_size);
  if (rc) return rc;
  rc = make_qkv_tmap(&tv, v_pool, (int)pool_rows, Hkv, 1, (long)Hkv * ATT_D, ATT_D, pool_rows * Hkv * ATT_D, block_size);
  if (rc) return rc;
  AttnOut out;
  out.o = (__nv_bfloat16*)o; out.o2 = nullptr;
  out.o_bs = o_bs; out.o_rs = o_rs; out.o_hs = o_hs;
  out.o2_bs = 0; out.o2_rs = 0; out.o2_hs = 0;
  out.split = Sq; out.lse = kv_splits > 1 ? nullptr : lse;
  out.n_peers = 0; out.rows_per_rank = 1; out.rows_per_rank2 = 1;
  for (int i = 0; i < 16; ++i) { out.o_peers[i] = nullptr; out.o2_peers[i] = nullptr; }
  out.kv_splits = kv_splits > 1 ? kv_splits : 1;
  out.part_o = part_o; out.part_ml = part_ml;
  out.prev_o = nullptr; out.prev_lse = nullptr; out.p_bs = out.p_rs = out.p_hs = 0;
  AttnPaging pg = {block_table, bt_stride, block_size};
  cudaStream_t st = (cudaStream_t)stream;
  rc = launch_attn(tq, tk, tv, out, B, H, Hkv, Sq, max_kv, kv_lens, scale, causal, q_offset, pg, status, st);
  if (rc || kv_splits <= 1) return rc;
  attn_merge_splits_kernel<<<(unsigned)((long)B * H * Sq), ATT_D, 0, st>>>(part_o, part_ml, kv_splits, (__nv_bfloat16*)o,
                                                                         o_bs, o_rs, o_hs, lse, H, Sq);
  return (int)cudaGetLastError();
}
