// K1-fp8: block-scaled fp8 (e4m3) GEMM on tcgen05 for sm_100a.
//
//   C[M,N] (bf16) = epilogue( sum_kb  sa[m, kb] * sw[n/128, kb] * (A8[m, kb-block] . W8[n, kb-block]) )
//
// A8 [M,K] and W8 [N,K] are e4m3, K-major.  Scales are fp32 over 128-element blocks of K: one per
// activation row and K block (sa [M, K/128]), one per 128 x 128 weight block (sw [N/128, K/128]) —
// the "weight_block_size = [128, 128], dynamic per-token-group activation" scheme the reference
// reaches through vLLM's Fp8Config (vllm_omni/diffusion/quantization/fp8.py).
//
// Per 128-wide K block the MMA issuer runs four tcgen05.mma kind::f8f6f4 (M=128, N=128, K=32)
// into one of four TMEM partial buffers; eight promotion warps (two per TMEM lane quadrant, 64
// columns each) pull the partial with tcgen05.ld, multiply by sa * sw and accumulate in fp32
// registers, so the block scales are applied exactly where they belong (between K blocks) while
// the tensor pipe already works on the next block.  The final epilogue (bias, activation,
// gate, residual) is the same as the bf16 kernel's.  All waits are bounded.
#include <cuda_fp8.h>

#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;   // BK bytes = 128 = one swizzle row
constexpr int F8_STAGES = 6;
constexpr int F8_SLOTS = 4;                             // TMEM partial buffers (4 x 128 columns)
constexpr int F8_THREADS = 320;
constexpr int F8_A_BYTES = F8_BM * F8_BK, F8_B_BYTES = F8_BN * F8_BK;
constexpr int F8_STAGE_BYTES = F8_A_BYTES + F8_B_BYTES;
constexpr int F8_SMEM = F8_STAGES * F8_STAGE_BYTES + 1024;

struct Fp8Epilogue {
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* gate;
  int ldr, gate_stride, rows_per_batch, act;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const float* __restrict__ sa, int lds_a, const float* __restrict__ sw, int lds_w,
                __nv_bfloat16* __restrict__ C, int ldc, int M, int N, int K, Fp8Epilogue epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[F8_STAGES], empty_bar[F8_STAGES];
  __shared__ __align__(8) uint64_t pfull_bar[F8_SLOTS], pempty_bar[F8_SLOTS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_m = (M + F8_BM - 1) / F8_BM, num_n = (N + F8_BN - 1) / F8_BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + F8_BK - 1) / F8_BK;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < F8_STAGES; ++i) { mbar_init(smem_u32(&full_bar[i]), 1); mbar_init(smem_u32(&empty_bar[i]), 1); }
    for (int i = 0; i < F8_SLOTS; ++i) { mbar_init(smem_u32(&pfull_bar[i]), 1); mbar_init(smem_u32(&pempty_bar[i]), 8); }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const int mb = t % num_m, nb = t / num_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t s = smem_base + stage * F8_STAGE_BYTES;
          mbar_expect_tx(fb, F8_STAGE_BYTES);
          tma_load_2d(s, &tmA, fb, kb * F8_BK, mb * F8_BM);
          tma_load_2d(s + F8_A_BYTES, &tmB, fb, kb * F8_BK, nb * F8_BN);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(F8_BM, F8_BN, 0, 0, 0, 0);   // e4m3 x e4m3 -> f32
      int stage = 0; uint32_t phase = 0;
      int slot = 0; uint32_t sphase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&pempty_bar[slot]), sphase ^ 1, &s_abort, status, ERR_WAIT_TMEM_EMPTY);
          mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort, status, ERR_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t s = smem_base + stage * F8_STAGE_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(s);
          const uint64_t b_desc = umma_desc_kmajor_sw128(s + F8_A_BYTES);
          const uint32_t d = tmem_base + slot * F8_BN;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k) mma_f8_ss(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k != 0);
          tc_commit(smem_u32(&empty_bar[stage]));
          tc_commit(smem_u32(&pfull_bar[slot]));
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
          if (++slot == F8_SLOTS) { slot = 0; sphase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;             // columns [64*half, 64*half + 64)
    int slot = 0; uint32_t sphase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int mb = t % num_m, nb = t / num_m;
      const int row = mb * F8_BM + q * 32 + lane;
      const bool row_ok = row < M;
      float acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      const float* sa_row = sa + (size_t)(row_ok ? row : 0) * lds_a;
      const float* sw_row = sw + (size_t)nb * lds_w;
      float s_next = sa_row[0] * sw_row[0];
      for (int kb = 0; kb < num_kb; ++kb) {
        const float sc = s_next;
        if (kb + 1 < num_kb) s_next = sa_row[kb + 1] * sw_row[kb + 1];
        mbar_wait(smem_u32(&pfull_bar[slot]), sphase, &s_abort, status, ERR_WAIT_TMEM_FULL);
        tc_fence_after_sync();
        const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + slot * F8_BN + half * 64;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(ta, v0);
        tmem_ld_32x32(ta + 32, v1);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&pempty_bar[slot]));
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[i] = fmaf(sc, __uint_as_float(v0[i]), acc[i]);
          acc[32 + i] = fmaf(sc, __uint_as_float(v1[i]), acc[32 + i]);
        }
        if (++slot == F8_SLOTS) { slot = 0; sphase ^= 1; }
      }
      if (row_ok) {
        const int col_base = nb * F8_BN + half * 64;
        const __nv_bfloat16* gate_row = epi.gate ? epi.gate + (size_t)(row / epi.rows_per_batch) * epi.gate_stride : nullptr;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int col = col_base + j * 8;
          if (col >= N) break;
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = acc[j * 8 + e];
          if (epi.bias) {
            const uint4 b = *reinterpret_cast<const uint4*>(epi.bias + col);
            const float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
            x[0] += b0.x; x[1] += b0.y; x[2] += b1.x; x[3] += b1.y; x[4] += b2.x; x[5] += b2.y; x[6] += b3.x; x[7] += b3.y;
          }
          if (epi.act == 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = gelu_tanh(x[e]);
          } else if (epi.act == 2) {
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] = silu(x[e]);
          }
          if (gate_row) {
            const uint4 g = *reinterpret_cast<const uint4*>(gate_row + col);
            const float2 g0 = unpack_bf16(g.x), g1 = unpack_bf16(g.y), g2 = unpack_bf16(g.z), g3 = unpack_bf16(g.w);
            x[0] *= g0.x; x[1] *= g0.y; x[2] *= g1.x; x[3] *= g1.y; x[4] *= g2.x; x[5] *= g2.y; x[6] *= g3.x; x[7] *= g3.y;
          }
          if (epi.residual) {
            const uint4 r = *reinterpret_cast<const uint4*>(epi.residual + (size_t)row * epi.ldr + col);
            const float2 r0 = unpack_bf16(r.x), r1 = unpack_bf16(r.y), r2 = unpack_bf16(r.z), r3 = unpack_bf16(r.w);
            x[0] += r0.x; x[1] += r0.y; x[2] += r1.x; x[3] += r1.y; x[4] += r2.x; x[5] += r2.y; x[6] += r3.x; x[7] += r3.y;
          }
          uint4 o;
          o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]); o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
          *reinterpret_cast<uint4*>(C + (size_t)row * ldc + col) = o;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// One warp per row: dynamic per-(row, 128-block) scales, bf16 -> e4m3.  K % 128 == 0.
__global__ void __launch_bounds__(256)
quant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long ldx, uint8_t* __restrict__ q, long ldq,
                      float* __restrict__ scales, int lds, int rows, int K) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nblk = K / 128;
  for (int b = 0; b < nblk; ++b) {
    const uint2 u = *reinterpret_cast<const uint2*>(x + (size_t)row * ldx + b * 128 + lane * 4);
    const float2 a = unpack_bf16(u.x), c = unpack_bf16(u.y);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-8f) * (1.0f / 448.0f);
    const float inv = 1.0f / scale;
    const __nv_fp8x2_storage_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(c.x * inv, c.y * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(q + (size_t)row * ldq + b * 128 + lane * 4) = (uint32_t)p0 | ((uint32_t)p1 << 16);
    if (lane == 0) scales[(size_t)row * lds + b] = scale;
  }
}

}  // namespace omni

using namespace omni;

extern "C" int omni_quant_fp8_rows(const void* x, long ldx, void* q, long ldq, float* scales, int lds, int rows,
                                   int K, void* stream) {
  if (rows <= 0) return RC_OK;
  if (K % 128 || (ldx & 3) || (ldq & 3)) return RC_BAD_ARG;
  quant_fp8_rows_kernel<<<(rows + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq,
                                                                          scales, lds, rows, K);
  return (int)cudaGetLastError();
}

extern "C" int omni_gemm_fp8(const void* A, long lda, const float* sa, int lds_a, const void* W, long ldw,
                             const float* sw, int lds_w, void* C, int ldc, int M, int N, int K, const void* bias,
                             const void* residual, int ldr, const void* gate, int gate_stride, int rows_per_batch,
                             int act, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return RC_OK;
  if (K % 128 || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7) || (ldr & 7) || (gate_stride & 7)) return RC_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint64_t)lda, F8_BM, F8_BK);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, F8_BN, F8_BK);
  if (rc) return rc;
  static unsigned long long prepared = 0;
  if (int e = ensure_dynamic_smem((const void*)gemm_fp8_kernel, F8_SMEM, prepared)) return e;
  Fp8Epilogue epi;
  epi.bias = (const __nv_bfloat16*)bias; epi.residual = (const __nv_bfloat16*)residual; epi.gate = (const __nv_bfloat16*)gate;
  epi.ldr = ldr; epi.gate_stride = gate_stride; epi.rows_per_batch = rows_per_batch > 0 ? rows_per_batch : 1; epi.act = act;
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int ctas = sm_count();
  gemm_fp8_kernel<<<tiles < ctas ? tiles : ctas, F8_THREADS, F8_SMEM, (cudaStream_t)stream>>>(
      tmA, tmB, sa, lds_a, sw, lds_w, (__nv_bfloat16*)C, ldc, M, N, K, epi, status);
  return (int)cudaGetLastError();
}
