// K1: persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] (bf16) = epilogue( A[M,K] (bf16, row-major) * W[N,K]^T (bf16, row-major) )
//
// i.e. the nn.Linear contraction with both operands K-major.  Two kernels share one epilogue:
//
// gemm_bf16_kernel<BN>       one CTA per SM walks a strided list of 128 x BN output tiles
//                            (BN = 128 / 192 / 256).  Also runs the grouped (MoE expert) GEMM, where
//                            every 128-row tile names its expert, and the implicit-GEMM convolution,
//                            where the A tile of a (tap, channel block) is a shifted 4-D TMA box.
// gemm_bf16_pair_kernel<TN>  two CTAs of a cluster (cta_group::2) compute one 256 x TN tile; each
//                            stages its own 128 rows of A and half of the W tile, the even CTA issues
//                            the M=256 MMAs.  Used whenever the problem fills a wave of such tiles;
//                            one launch can carry two problems of the same (N, K).
//
// Roles inside a CTA (both kernels):
//   warp 0    TMA producer: cp.async.bulk.tensor loads of the A / W k-blocks (128-byte
//             swizzle) into a multi-stage shared-memory ring, completion on mbarriers
//   warp 1    MMA issuer: one elected thread issues tcgen05.mma (K=16 per instruction) with
//             the fp32 accumulator in tensor memory; tcgen05.commit hands ring slots back
//             to the producer and finished accumulators to the epilogue
//   warps 2-9 epilogue: two warps per TMEM lane quadrant, each draining half of the tile's
//             columns: tcgen05.ld of the accumulator (one row per thread, 32 columns per
//             instruction), fused bias / GELU-tanh / SiLU / gate*x + residual, bf16 stores to
//             local memory or, for the fused collectives, straight into peers' buffers
//             (column groups: Ulysses head scatter; row blocks: tensor-parallel reduce-scatter)
// Two accumulators live in TMEM so the epilogue of tile i overlaps the main loop of
// tile i+1.  All mbarrier waits are bounded (see ptx_sm100.cuh); a timeout is reported
// through *status and the kernel still terminates and frees its TMEM.  No TMA load in this
// file is a multicast.
//
// Replaces the cuBLAS calls behind the reference's vLLM linear layers
// (vllm_omni/diffusion/models/qwen_image/qwen_image_transformer.py:427-560).
#include "host_util.h"
#include "ptx_sm100.cuh"
#include "peer_signal.cuh"

namespace omni {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue

enum Act : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SILU = 2 };

struct GemmEpilogue {
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, ldr] or nullptr (may alias C)
  const __nv_bfloat16* gate;      // row (r / rows_per_batch) of a [B, gate_stride] matrix, or nullptr
  int ldr;
  int gate_stride;
  int rows_per_batch;
  int act;
  // output row r lands at C + (r / c_rows_per_batch) * c_batch_stride + (r % c_rows_per_batch) * ldc,
  // which lets two GEMMs write the text and image rows of one joint [B, S_txt + S_img, N] buffer
  int c_rows_per_batch;  // 0 = plain row-major output
  long c_batch_stride;
  // Fused all-to-all (Ulysses head scatter): with scatter_P > 1 the output columns are cut into
  // groups of scatter_G columns (a multiple of 32); group g belongs to rank g % P and lands in
  // that rank's buffer peer_out[g % P] at column (g / P) * G + (col % G).  peer_out[] are peer
  // (NVLink-mapped) or local pointers that already include this rank's row offset.
  int scatter_P;
  int scatter_G;
  // Fused reduce-scatter feed (tensor parallel): with scatter_rows > 0 output row r belongs to rank
  // r / scatter_rows and is stored, as row r % scatter_rows, through peer_out[that rank] (each
  // pointer already addresses the slot reserved for THIS rank's partial sums on the owner).
  int scatter_rows;
  __nv_bfloat16* peer_out[16];
};

// Implicit-GEMM convolution (stride 1, "same" padding, NHWC bf16): the M dimension is the output
// pixels, walked in patches of CONV_BH x CONV_BW = 128 pixels; K runs over taps x input-channel
// blocks of 64.  The A tile of one (tap, channel block) is ONE 4-D TMA box
// {64 channels, CONV_BW, CONV_BH, 1 image} of the input, shifted by the tap's offset; pixels
// outside the image are filled with zeros by TMA, which is the padding.  taps == 0: plain GEMM.
//
// One-dimensional mode (one_d, vocoder stacks, channels-last [B, T, C]): the M dimension is the
// output time steps in runs of 128; tap j of a kernel of `taps` taps reads the input `j * dil - pad`
// steps away, so the A tile of one (tap, channel block) is the box {64 channels, 128 steps} shifted by
// that offset, and both paddings (causal left, "same", the ragged end) are TMA's zero fill.  A
// transposed convolution of stride r is the same kernel on weights stacked by output phase: its
// [B, Tq, r * Cout] result read as [B, Tq * r, Cout].
constexpr int CONV_BW = 16, CONV_BH = 8;
struct ConvGeom {
  int taps;        // 0 (GEMM); 2-D: 1 (1x1) or 9 (3x3); 1-D: kernel size
  int H, W;        // output (= input) height and width; 1-D: H = 1, W = output steps
  int tiles_x, tiles_y;
  int cin_blocks;  // ceil(Cin / 64); the weight matrix is [Cout, taps * cin_blocks * 64]
  int one_d, dil, pad;
};

// Grouped (MoE) mode without row padding: the rows of all experts sit back to back in A and C; M-tile
// t starts at row0[t] and owns rows[t] (<= 128) rows of expert tile_expert[t].  The TMA box always
// brings 128 rows (the surplus belongs to the next expert or is zero fill past the end; its products
// are never stored), so the activations are read and the results written once per REAL row instead
// of once per 128-row padded segment.  row0 == nullptr: rows of tile t start at t * 128.
struct GroupTiles {
  const int* row0;
  const int* rows;
  int num_m;        // number of M tiles when row0 is set
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 192 ? 4 : 6);
  static constexpr int ACC_STRIDE = (BN > 128) ? 256 : 128;
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;
  // ring + the epilogue warps' staging blocks for peer stores + alignment slack
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * 32 * 128 + 1024;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
  // groups of 8 row-blocks sweep the column blocks together so that the CTAs that run
  // at the same time share A and W tiles in L2
  constexpr int GROUP_M = 8;
  const int group_size = GROUP_M * num_n;
  const int g = t / group_size;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int in_g = t - g * group_size;
  mb = first_m + in_g % gm;
  nb = in_g / gm;
}

// Where output element (row, col0) lands: plain row-major, batched rows, or a peer's buffer for
// the fused collectives (column groups: Ulysses head scatter; row blocks: reduce-scatter feed).
__device__ __forceinline__ __nv_bfloat16* epilogue_dest(int row, int col0, __nv_bfloat16* __restrict__ C, int ldc,
                                                        const GemmEpilogue& epi) {
  __nv_bfloat16* cbase = C;
  int dcol = col0;
  if (epi.scatter_P > 1) {
    const int g = col0 / epi.scatter_G;
    cbase = epi.peer_out[g % epi.scatter_P];
    dcol = (g / epi.scatter_P) * epi.scatter_G + (col0 - g * epi.scatter_G);
  }
  if (epi.scatter_rows > 0) {
    const int owner = row / epi.scatter_rows;
    return epi.peer_out[owner] + (size_t)(row - owner * epi.scatter_rows) * ldc + dcol;
  }
  if (epi.c_rows_per_batch > 0) {
    const int cb = row / epi.c_rows_per_batch;
    return cbase + (size_t)cb * epi.c_batch_stride + (size_t)(row - cb * epi.c_rows_per_batch) * ldc + dcol;
  }
  return cbase + (size_t)row * ldc + dcol;
}

// Fused epilogue math for 32 accumulator columns of one output row: bias, activation, gate,
// residual, bf16 conversion.  o[j] holds columns [col0 + 8j, col0 + 8j + 8); groups at or past N
// are left untouched.
__device__ __forceinline__ void epilogue_math32(const uint32_t (&v)[32], int row, int col0, int N,
                                                const GemmEpilogue& epi, const __nv_bfloat16* gate_row,
                                                uint4* __restrict__ o) {
  const __nv_bfloat16* res = epi.residual ? epi.residual + (size_t)row * epi.ldr + col0 : nullptr;
#pragma unroll
  for (int j = 0; j < 4; ++j) {  // 8 columns per 16-byte group
    if (col0 + j * 8 < N) {
      float x[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(v[j * 8 + e]);
      if (epi.bias) {
        uint4 b = *reinterpret_cast<const uint4*>(epi.bias + col0 + j * 8);
        float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
        x[0] += b0.x; x[1] += b0.y; x[2] += b1.x; x[3] += b1.y;
        x[4] += b2.x; x[5] += b2.y; x[6] += b3.x; x[7] += b3.y;
      }
      if (epi.act == ACT_GELU_TANH) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = gelu_tanh(x[e]);
      } else if (epi.act == ACT_SILU) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = silu(x[e]);
      }
      if (gate_row) {
        uint4 g = *reinterpret_cast<const uint4*>(gate_row + col0 + j * 8);
        float2 g0 = unpack_bf16(g.x), g1 = unpack_bf16(g.y), g2 = unpack_bf16(g.z), g3 = unpack_bf16(g.w);
        x[0] *= g0.x; x[1] *= g0.y; x[2] *= g1.x; x[3] *= g1.y;
        x[4] *= g2.x; x[5] *= g2.y; x[6] *= g3.x; x[7] *= g3.y;
      }
      if (res) {
        uint4 r = *reinterpret_cast<const uint4*>(res + j * 8);
        float2 r0 = unpack_bf16(r.x), r1 = unpack_bf16(r.y), r2 = unpack_bf16(r.z), r3 = unpack_bf16(r.w);
        x[0] += r0.x; x[1] += r0.y; x[2] += r1.x; x[3] += r1.y;
        x[4] += r2.x; x[5] += r2.y; x[6] += r3.x; x[7] += r3.y;
      }
      o[j].x = pack_bf16(x[0], x[1]);
      o[j].y = pack_bf16(x[2], x[3]);
      o[j].z = pack_bf16(x[4], x[5]);
      o[j].w = pack_bf16(x[6], x[7]);
    }
  }
}

// Direct store of one row's 32 columns from the thread that owns the row (local outputs: L2
// merges the 16-byte pieces of a line).
__device__ __forceinline__ void epilogue_store32(const uint32_t (&v)[32], int row, int col0, int N,
                                                 __nv_bfloat16* __restrict__ C, int ldc, const GemmEpilogue& epi,
                                                 const __nv_bfloat16* gate_row) {
  uint4 o[4];
  epilogue_math32(v, row, col0, N, epi, gate_row, o);
  __nv_bfloat16* out = epilogue_dest(row, col0, C, ldc, epi);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (col0 + j * 8 < N) *reinterpret_cast<uint4*>(out + j * 8) = o[j];
}

// Peer stores (fused collectives) go through a per-warp staging block in shared memory so that
// the warp writes whole 128-byte row segments: a store from the row-owning thread would put 32
// separate 16-byte writes on NVLink per instruction, which is request-bound far below link speed.
//   write phase: lane = row, `ngroups` (4 or 8) 16-byte groups, group index XOR-swizzled by the row
//   read  phase: 8 lanes per row, 4 rows per instruction -> 4 x 128 contiguous bytes per store
constexpr int EPI_STAGE_BYTES = 32 * 128;          // per epilogue warp: 32 rows x 64 bf16 columns
constexpr int EPI_STAGE_TOTAL = 8 * EPI_STAGE_BYTES;

__device__ __forceinline__ void epilogue_store_staged(uint32_t stg, const uint4* __restrict__ o, int ngroups, int lane,
                                                      int row0, int M, int col0, int N, __nv_bfloat16* __restrict__ C,
                                                      int ldc, const GemmEpilogue& epi) {
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (k < ngroups) st_shared_v4(stg + lane * 128 + ((k ^ (lane & 7)) << 4), o[k]);
  __syncwarp();
  const int k = lane & 7;
  const int col = col0 + k * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const int row = row0 + r;
    if (k < ngroups && row < M && col < N) {
      const uint4 val = ld_shared_v4(stg + r * 128 + ((k ^ (r & 7)) << 4));
      *reinterpret_cast<uint4*>(epilogue_dest(row, col, C, ldc, epi)) = val;
    }
  }
  __syncwarp();
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 __nv_bfloat16* __restrict__ C, int ldc, int M, int N, int K, GemmEpilogue epi,
                 const int* __restrict__ tile_expert, GroupTiles gt, ConvGeom conv, PeerSignal sig, PeerWait wt, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int num_m = gt.row0 ? gt.num_m : (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      peer_wait_arrivals(wt, &s_abort, status);   // A may hold rows that peers write (fused exchange)
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, num_m, num_n, mb, nb);
        // grouped (MoE) mode: every 128-row tile belongs to one expert; -1 = padding tile
        const int ex = tile_expert ? tile_expert[mb] : 0;
        if (ex < 0) continue;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(fb, Cfg::STAGE_BYTES);
          if (conv.taps) {
            const int per_img = conv.tiles_x * conv.tiles_y;
            const int img = mb / per_img, rem = mb - img * per_img;
            const int y0 = (rem / conv.tiles_x) * CONV_BH, x0 = (rem % conv.tiles_x) * CONV_BW;
            const int tap = kb / conv.cin_blocks, cb = kb - tap * conv.cin_blocks;
            if (conv.one_d) {
              tma_load_4d(sa, &tmA, fb, cb * BK, rem * BM + tap * conv.dil - conv.pad, 0, img);
            } else {
              const int dy = conv.taps == 9 ? tap / 3 - 1 : 0, dx = conv.taps == 9 ? tap % 3 - 1 : 0;
              tma_load_4d(sa, &tmA, fb, cb * BK, x0 + dx, y0 + dy, img);
            }
          } else {
            tma_load_2d(sa, &tmA, fb, kb * BK, gt.row0 ? gt.row0[mb] : mb * BM);
          }
          tma_load_3d(sa + Cfg::A_BYTES, &tmB, fb, kb * BK, nb * BN, ex);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        if (tile_expert) {
          int mb, nb;
          tile_coords(t, num_m, num_n, mb, nb);
          if (tile_expert[mb] < 0) continue;
        }
        mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, &s_abort, status, ERR_WAIT_TMEM_EMPTY);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort, status, ERR_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(sa);
          const uint64_t b_desc = umma_desc_kmajor_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in >>4 units
            mma_f16_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        tc_commit(smem_u32(&tfull_bar[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;         // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    constexpr int CH_PER_WARP = BN / 64;
    const bool peer_stores = (epi.scatter_P > 1 || epi.scatter_rows > 0) && conv.taps == 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb;
      tile_coords(t, num_m, num_n, mb, nb);
      if (tile_expert && tile_expert[mb] < 0) continue;
      mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, &s_abort, status, ERR_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      int row = mb * BM + q * 32 + lane;
      bool row_ok = row < M;
      if (gt.row0) {
        row = gt.row0[mb] + q * 32 + lane;
        row_ok = q * 32 + lane < gt.rows[mb] && row < M;
      }
      if (conv.taps) {
        // row of the tile -> pixel of the patch -> row of the [N*H*W, Cout] output
        const int per_img = conv.tiles_x * conv.tiles_y;
        const int img = mb / per_img, rem = mb - img * per_img;
        const int r = q * 32 + lane;
        int y = (rem / conv.tiles_x) * CONV_BH + r / CONV_BW, x = (rem % conv.tiles_x) * CONV_BW + r % CONV_BW;
        if (conv.one_d) { y = 0; x = rem * BM + r; }
        row_ok = y < conv.H && x < conv.W;
        row = (img * conv.H + y) * conv.W + x;
      }
      const __nv_bfloat16* gate_row = nullptr;
      if (epi.gate && row_ok) gate_row = epi.gate + (size_t)(row / epi.rows_per_batch) * epi.gate_stride;
      if (peer_stores) {
        // fused collectives: 64 columns at a time through the staging block
        const uint32_t stg = smem_base + STAGES * Cfg::STAGE_BYTES + (warp - 2) * EPI_STAGE_BYTES;
#pragma unroll 1
        for (int c = half * CH_PER_WARP; c < (half + 1) * CH_PER_WARP; c += 2) {
          const int col0 = nb * BN + c * 32;
          if (col0 >= N) break;
          const int nsub = min(2, (half + 1) * CH_PER_WARP - c);
          uint4 o[8];
          for (int sidx = 0; sidx < nsub; ++sidx) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * Cfg::ACC_STRIDE + (c + sidx) * 32, v);
            tmem_wait_ld();
            if (row_ok) epilogue_math32(v, row, col0 + sidx * 32, N, epi, gate_row, o + sidx * 4);
          }
          epilogue_store_staged(stg, o, nsub * 4, lane, mb * BM + q * 32, M, col0, N, C, ldc, epi);
        }
      } else {
#pragma unroll 1
        for (int c = half * CH_PER_WARP; c < (half + 1) * CH_PER_WARP; ++c) {
          const int col0 = nb * BN + c * 32;
          if (col0 >= N) break;
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * Cfg::ACC_STRIDE + c * 32, v);
          tmem_wait_ld();
          if (row_ok) epilogue_store32(v, row, col0, N, C, ldc, epi, gate_row);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    // every peer store of this CTA was issued before the barrier above
    peer_signal_cta_done(sig, gridDim.x);
    peer_wait_cta_exit(wt, gridDim.x);
  }
  if (s_abort) {
    // give copies and MMAs that may still be in flight time to land before TMEM and
    // shared memory are handed back
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): two CTAs of a cluster compute one 256 x 256 output tile.
// Each CTA stages its own 128 rows of A and HALF of the W tile (128 of the 256 output columns'
// weights) per k-block, so a k-block costs 32 KB of L2 -> shared-memory traffic per SM instead
// of 48 KB, and the ring holds 6 stages instead of 4.  The even CTA issues one M=256, N=256
// tcgen05.mma per 16 K-elements that reads A and W from both CTAs' shared memory; each CTA's
// TMEM receives the 128 accumulator rows it owns and its own epilogue warps drain them.
//   full_bar   (even CTA)   bytes of BOTH CTAs' loads land on it (the odd CTA's TMA names it)
//   empty_bar  (each CTA)   released by two tcgen05.commit of the even CTA, one per CTA
//   tfull_bar  (each CTA)   accumulator ready, same two-commit scheme
//   tempty_bar (even CTA)   16 arrivals: 8 epilogue warps of each CTA
// No load in this kernel is a multicast; every CTA fetches exactly the bytes it alone needs.
// The tile width TN is 256, 192 or 128 (picked to minimise waves x width, like the one-CTA kernel).
template <int TN>
struct PairCfg {
  static constexpr int A_BYTES = BM * BK * 2;            // 16 KiB: this CTA's 128 rows of A
  static constexpr int B_BYTES = (TN / 2) * BK * 2;      // this CTA's half of the W tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // a multiple of 1 KiB for every TN
  static constexpr int STAGES = (TN == 256) ? 6 : (TN == 192 ? 6 : 7);
  // ring + the epilogue warps' staging blocks for peer stores + alignment slack
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 8 * 32 * 128 + 1024;
};

// One launch can carry TWO problems that share N and K (the image and the text stream of a
// dual-stream DiT block: same layer shape, different activations, weights, outputs and epilogue
// operands).  The tile list is problem 0's tiles followed by problem 1's, so the short text
// problem fills the partial last wave of the image problem instead of paying for a launch and a
// mostly idle grid of its own.
struct PairProblem {
  CUtensorMap tmA, tmB;
  __nv_bfloat16* C;
  int ldc;
  int M;
  GemmEpilogue epi;
};
struct PairArgs {
  PairProblem p[2];
  int n_problems;   // 1 or 2
  int N, K;
  PeerSignal sig;   // arrivals this launch reports to the group once its peer stores are out
  PeerWait wt;      // arrivals this launch needs before it reads its A operands
};

template <int TN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ PairArgs args, int* status) {
  constexpr int P_TILE_N = TN;
  const int N = args.N, K = args.K;
  constexpr int P_STAGES = PairCfg<TN>::STAGES;
  constexpr int P_STAGE_BYTES = PairCfg<TN>::STAGE_BYTES;
  constexpr int P_A_BYTES = PairCfg<TN>::A_BYTES;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[P_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[P_STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0: issues the MMAs, 1: its partner
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int num_n = (N + P_TILE_N - 1) / P_TILE_N;
  const int num_m0 = (args.p[0].M + 2 * BM - 1) / (2 * BM);
  const int num_m1 = args.n_problems > 1 ? (args.p[1].M + 2 * BM - 1) / (2 * BM) : 0;
  const int tiles0 = num_m0 * num_n;
  const int num_tiles = tiles0 + num_m1 * num_n;
  const int num_kb = (K + BK - 1) / BK;
  // tile index -> (problem, row block, column block)
  auto locate = [&](int t, int& prob, int& mb, int& nb) {
    prob = t >= tiles0 ? 1 : 0;
    tile_coords(prob ? t - tiles0 : t, prob ? num_m1 : num_m0, num_n, mb, nb);
  };

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < P_STAGES; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 16);
    }
    fence_mbar_init();
    for (int i = 0; i < args.n_problems; ++i) {
      tma_prefetch_desc(&args.p[i].tmA);
      tma_prefetch_desc(&args.p[i].tmB);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_base_s), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before either touches the other's
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      peer_wait_arrivals(args.wt, &s_abort, status);   // A may hold rows that peers write (fused exchange)
      for (int t = pair; t < num_tiles; t += num_pairs) {
        int prob, mb, nb;
        locate(t, prob, mb, nb);
        const CUtensorMap* tmA = &args.p[prob].tmA;
        const CUtensorMap* tmB = &args.p[prob].tmB;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
          if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * P_STAGE_BYTES);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[stage]), 0);
          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          tma_load_2d_pair(sa, tmA, fb, kb * BK, mb * 2 * BM + (int)rank * BM);
          tma_load_2d_pair(sa + P_A_BYTES, tmB, fb, kb * BK, nb * P_TILE_N + (int)rank * (P_TILE_N / 2));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (even CTA)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc(2 * BM, P_TILE_N, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = pair; t < num_tiles; t += num_pairs) {
        mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, &s_abort, status, ERR_WAIT_TMEM_EMPTY);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort, status, ERR_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(sa);
          const uint64_t b_desc = umma_desc_kmajor_sw128(sa + P_A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) mma_f16_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 0));
          tc_commit_pair(mapa_shared(smem_u32(&empty_bar[stage]), 1));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        tc_commit_pair(mapa_shared(smem_u32(&tfull_bar[acc]), 0));
        tc_commit_pair(mapa_shared(smem_u32(&tfull_bar[acc]), 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int prob, mb, nb;
      locate(t, prob, mb, nb);
      const GemmEpilogue& epi = args.p[prob].epi;
      __nv_bfloat16* C = args.p[prob].C;
      const int ldc = args.p[prob].ldc;
      mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, &s_abort, status, ERR_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      const int row = mb * 2 * BM + (int)rank * BM + q * 32 + lane;
      const bool row_ok = row < args.p[prob].M;
      const __nv_bfloat16* gate_row = nullptr;
      if (epi.gate && row_ok) gate_row = epi.gate + (size_t)(row / epi.rows_per_batch) * epi.gate_stride;
      if (epi.scatter_P > 1 || epi.scatter_rows > 0) {
        // fused collectives: 64 columns at a time through the staging block
        const uint32_t stg = smem_base + P_STAGES * P_STAGE_BYTES + (warp - 2) * EPI_STAGE_BYTES;
        const int M = args.p[prob].M;
#pragma unroll 1
        for (int c = half * (P_TILE_N / 64); c < (half + 1) * (P_TILE_N / 64); c += 2) {
          const int col0 = nb * P_TILE_N + c * 32;
          if (col0 >= N) break;
          const int nsub = min(2, (half + 1) * (P_TILE_N / 64) - c);
          uint4 o[8];
          for (int sidx = 0; sidx < nsub; ++sidx) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * 256 + (c + sidx) * 32, v);
            tmem_wait_ld();
            if (row_ok) epilogue_math32(v, row, col0 + sidx * 32, N, epi, gate_row, o + sidx * 4);
          }
          epilogue_store_staged(stg, o, nsub * 4, lane, mb * 2 * BM + (int)rank * BM + q * 32, M, col0, N, C, ldc, epi);
        }
      } else {
#pragma unroll 1
        for (int c = half * (P_TILE_N / 64); c < (half + 1) * (P_TILE_N / 64); ++c) {
          const int col0 = nb * P_TILE_N + c * 32;
          if (col0 >= N) break;
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * 256 + c * 32, v);
          tmem_wait_ld();
          if (row_ok) epilogue_store32(v, row, col0, N, C, ldc, epi, gate_row);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    peer_signal_cta_done(args.sig, gridDim.x);
    peer_wait_cta_exit(args.wt, gridDim.x);
  }
  if (s_abort) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  cluster_sync_all();   // neither CTA frees TMEM or exits while its partner may still signal it
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}


// ------------------------------------------------------------------------------------------
// One-CTA tiles (128 x BN) over the tile list of up to TWO problems that share N and K: the same
// scheduling idea as the CTA-pair kernel for problems too small to fill a wave of 256-row tiles
// (a sequence-parallel rank's rows, a text stream of a few dozen rows).  With 128-row tiles and
// 148 schedulable units instead of 74 the launcher can usually find a tile width whose tile count
// fits whole waves, and the short problem's tiles run beside the long one's instead of in a launch
// of their own that would last a full K loop for a handful of tiles.
template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_multi_kernel(const __grid_constant__ PairArgs args, int* status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  const int N = args.N, K = args.K;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tfull_bar[2];
  __shared__ __align__(8) uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const int num_n = (N + BN - 1) / BN;
  const int num_m0 = (args.p[0].M + BM - 1) / BM;
  const int num_m1 = args.n_problems > 1 ? (args.p[1].M + BM - 1) / BM : 0;
  const int tiles0 = num_m0 * num_n;
  const int num_tiles = tiles0 + num_m1 * num_n;
  const int num_kb = (K + BK - 1) / BK;
  auto locate = [&](int t, int& prob, int& mb, int& nb) {
    prob = t >= tiles0 ? 1 : 0;
    tile_coords(prob ? t - tiles0 : t, prob ? num_m1 : num_m0, num_n, mb, nb);
  };

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(smem_u32(&full_bar[i]), 1);
      mbar_init(smem_u32(&empty_bar[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tfull_bar[i]), 1);
      mbar_init(smem_u32(&tempty_bar[i]), 8);
    }
    fence_mbar_init();
    for (int i = 0; i < args.n_problems; ++i) {
      tma_prefetch_desc(&args.p[i].tmA);
      tma_prefetch_desc(&args.p[i].tmB);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      peer_wait_arrivals(args.wt, &s_abort, status);   // A may hold rows that peers write (fused exchange)
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int prob, mb, nb;
        locate(t, prob, mb, nb);
        const CUtensorMap* tmA = &args.p[prob].tmA;
        const CUtensorMap* tmB = &args.p[prob].tmB;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, &s_abort, status, ERR_WAIT_EMPTY);
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          mbar_expect_tx(fb, Cfg::STAGE_BYTES);
          tma_load_2d(sa, tmA, fb, kb * BK, mb * BM);
          tma_load_2d(sa + Cfg::A_BYTES, tmB, fb, kb * BK, nb * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, &s_abort, status, ERR_WAIT_TMEM_EMPTY);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort, status, ERR_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(sa);
          const uint64_t b_desc = umma_desc_kmajor_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) mma_f16_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          tc_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        tc_commit(smem_u32(&tfull_bar[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int CH_PER_WARP = BN / 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int prob, mb, nb;
      locate(t, prob, mb, nb);
      const GemmEpilogue& epi = args.p[prob].epi;
      __nv_bfloat16* C = args.p[prob].C;
      const int ldc = args.p[prob].ldc;
      const int M = args.p[prob].M;
      mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, &s_abort, status, ERR_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      const int row = mb * BM + q * 32 + lane;
      const bool row_ok = row < M;
      const __nv_bfloat16* gate_row = nullptr;
      if (epi.gate && row_ok) gate_row = epi.gate + (size_t)(row / epi.rows_per_batch) * epi.gate_stride;
      if (epi.scatter_P > 1 || epi.scatter_rows > 0) {
        const uint32_t stg = smem_base + STAGES * Cfg::STAGE_BYTES + (warp - 2) * EPI_STAGE_BYTES;
#pragma unroll 1
        for (int c = half * CH_PER_WARP; c < (half + 1) * CH_PER_WARP; c += 2) {
          const int col0 = nb * BN + c * 32;
          if (col0 >= N) break;
          const int nsub = min(2, (half + 1) * CH_PER_WARP - c);
          uint4 o[8];
          for (int sidx = 0; sidx < nsub; ++sidx) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * Cfg::ACC_STRIDE + (c + sidx) * 32, v);
            tmem_wait_ld();
            if (row_ok) epilogue_math32(v, row, col0 + sidx * 32, N, epi, gate_row, o + sidx * 4);
          }
          epilogue_store_staged(stg, o, nsub * 4, lane, mb * BM + q * 32, M, col0, N, C, ldc, epi);
        }
      } else {
#pragma unroll 1
        for (int c = half * CH_PER_WARP; c < (half + 1) * CH_PER_WARP; ++c) {
          const int col0 = nb * BN + c * 32;
          if (col0 >= N) break;
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * Cfg::ACC_STRIDE + c * 32, v);
          tmem_wait_ld();
          if (row_ok) epilogue_store32(v, row, col0, N, C, ldc, epi, gate_row);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    peer_signal_cta_done(args.sig, gridDim.x);
    peer_wait_cta_exit(args.wt, gridDim.x);
  }
  if (s_abort) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

static int g_pair_mode = 1;   // 0: never unless forced, 1: automatic for large problems

// w_box_rows: rows of W one TMA box brings (half a tile for the CTA-pair kernel, a whole tile for the
// one-CTA kernel)
static int fill_pair_problem(PairProblem& pp, const void* A, int lda, const void* W, int ldw, __nv_bfloat16* C,
                             int ldc, int M, int N, int K, const GemmEpilogue& epi, int w_box_rows) {
  int rc = make_tmap_2d(&pp.tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, BK);
  if (rc) return rc;
  rc = make_tmap_2d(&pp.tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2, w_box_rows, BK);
  if (rc) return rc;
  pp.C = C; pp.ldc = ldc; pp.M = M; pp.epi = epi;
  return RC_OK;
}

template <int TN>
static int launch_gemm_pair(const PairArgs& args, int* status, int max_pairs, cudaStream_t stream) {
  using Cfg = PairCfg<TN>;
  static unsigned long long prepared = 0;
  if (int e = ensure_dynamic_smem((const void*)gemm_bf16_pair_kernel<TN>, Cfg::SMEM_BYTES, prepared)) return e;
  const int num_n = (args.N + TN - 1) / TN;
  int num_tiles = 0;
  for (int i = 0; i < args.n_problems; ++i) num_tiles += ((args.p[i].M + 2 * BM - 1) / (2 * BM)) * num_n;
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  gemm_bf16_pair_kernel<TN><<<2 * pairs, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(args, status);
  return (int)cudaGetLastError();
}

static int launch_pair_tn(int tn, const PairArgs& args, int* status, int pairs, cudaStream_t s) {
  switch (tn) {
    case 256: return launch_gemm_pair<256>(args, status, pairs, s);
    case 192: return launch_gemm_pair<192>(args, status, pairs, s);
    default: return launch_gemm_pair<128>(args, status, pairs, s);
  }
}

// how many CTA pairs can be resident at once (one CTA per SM, two SMs of one TPC per pair)
static int max_resident_pairs() {
  static int cached = 0;
  if (cached) return cached;
  int n = 0;
  if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           PairCfg<256>::SMEM_BYTES) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = PairCfg<256>::SMEM_BYTES;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel<256>, &cfg) != cudaSuccess) n = 0;
  }
  (void)cudaGetLastError();
  if (n <= 0 || n > sm_count() / 2) n = sm_count() / 2;
  cached = n;
  return n;
}

static int pick_pair_tn(int M, int N, int pairs) {
  const int cand[3] = {256, 192, 128};
  int best = 256;
  long best_cost = -1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  for (int i = 0; i < 3; ++i) {
    const int tn = cand[i];
    const long tiles = (long)num_m * ((N + tn - 1) / tn);
    const long waves = (tiles + pairs - 1) / pairs;
    const long cost = waves * tn * (tn == 128 ? 108 : (tn == 192 ? 102 : 100));
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = tn; }
  }
  return best;
}

template <int BN>
static int launch_gemm(const CUtensorMap& tmA, const void* W, __nv_bfloat16* C, int ldc, int M,
                       int N, int K, int ldw, const GemmEpilogue& epi, int* status, int max_ctas,
                       cudaStream_t stream, int num_experts = 1, const int* tile_expert = nullptr,
                       const ConvGeom* conv = nullptr, const OmniSync* sync = nullptr, const GroupTiles* gtiles = nullptr) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmB;
  // weights as [E, N, K]; a plain linear layer is E = 1
  int rc = make_tmap_3d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)K, (uint64_t)N,
                        (uint64_t)num_experts, (uint64_t)ldw * 2, (uint64_t)N * ldw * 2, BK, BN);
  if (rc) return rc;
  static unsigned long long prepared = 0;
  if (int e = ensure_dynamic_smem((const void*)gemm_bf16_kernel<BN>, Cfg::SMEM_BYTES, prepared)) return e;
  GroupTiles gt = {nullptr, nullptr, 0};
  if (gtiles) gt = *gtiles;
  const int num_tiles = (gt.row0 ? gt.num_m : (M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = num_tiles < max_ctas ? num_tiles : max_ctas;
  ConvGeom geom = {};
  if (conv) geom = *conv;
  PeerSignal sig;
  PeerWait wt;
  unpack_sync(sync, sig, wt);
  gemm_bf16_kernel<BN><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, C, ldc, M, N, K, epi, tile_expert, gt, geom, sig, wt, status);
  return (int)cudaGetLastError();
}


template <int BN>
static int launch_gemm_multi(const PairArgs& args, int* status, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static unsigned long long prepared = 0;
  if (int e = ensure_dynamic_smem((const void*)gemm_bf16_multi_kernel<BN>, Cfg::SMEM_BYTES, prepared)) return e;
  const int num_n = (args.N + BN - 1) / BN;
  int num_tiles = 0;
  for (int i = 0; i < args.n_problems; ++i) num_tiles += ((args.p[i].M + BM - 1) / BM) * num_n;
  const int grid = num_tiles < max_ctas ? num_tiles : max_ctas;
  gemm_bf16_multi_kernel<BN><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(args, status);
  return (int)cudaGetLastError();
}

static int launch_multi_bn(int bn, const PairArgs& args, int* status, int ctas, cudaStream_t s) {
  switch (bn) {
    case 256: return launch_gemm_multi<256>(args, status, ctas, s);
    case 192: return launch_gemm_multi<192>(args, status, ctas, s);
    default: return launch_gemm_multi<128>(args, status, ctas, s);
  }
}

// Which kernel and tile width finish a list of (one or two) problems soonest.  A wave of tiles costs
// time in proportion to the tile width (K and the 128 rows per SM are the same for every choice);
// the CTA-pair kernel runs 74 tiles of 256 rows per wave and streams about 14 % faster per SM, the
// one-CTA kernel 148 tiles of 128 rows; narrow tiles re-read A more often.
struct TilePlan { bool pair; int bn; };
static TilePlan plan_tiles(const int* Ms, int n_problems, int N, int ctas, int pairs, bool allow_pair) {
  const int cand[3] = {256, 192, 128};
  TilePlan best = {false, 256};
  double best_cost = -1.0;
  for (int kind = 0; kind < 2; ++kind) {
    if (kind == 1 && (!allow_pair || pairs <= 0)) continue;
    for (int i = 0; i < 3; ++i) {
      const int bn = cand[i];
      const int rows = kind ? 2 * BM : BM;
      long tiles = 0;
      for (int p = 0; p < n_problems; ++p) tiles += (long)((Ms[p] + rows - 1) / rows) * ((N + bn - 1) / bn);
      const int units = kind ? pairs : ctas;
      const long waves = (tiles + units - 1) / units;
      const double width_penalty = bn == 128 ? 1.08 : (bn == 192 ? 1.03 : 1.0);
      const double cost = (double)waves * bn * width_penalty * (kind ? 0.88 : 1.0);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; best.pair = kind == 1; best.bn = bn; }
    }
  }
  return best;
}

static int pick_bn(int M, int N, int ctas) {
  // minimise waves x tile width (time per tile is proportional to BN); wide tiles win ties
  const int cand[3] = {256, 192, 128};
  int best = 256;
  long best_cost = -1;
  const int num_m = (M + BM - 1) / BM;
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    const long tiles = (long)num_m * ((N + bn - 1) / bn);
    const long waves = (tiles + ctas - 1) / ctas;
    // narrow tiles re-read A more often: charge them a small penalty
    const long cost = waves * bn * (bn == 128 ? 110 : (bn == 192 ? 103 : 100));
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

}  // namespace omni

// C ABI.  All pointers are device pointers; `status` is a device int32 that receives the
// first timeout code (0 = none).  Strides are in elements.  force_bn = 0 lets the launcher
// choose the tile width.
// `sync` (may be null): arrivals this launch waits for before reading A, and / or reports to the
// group after its peer stores (see peer_signal.cuh).
extern "C" int omni_gemm_bf16_sync(const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                                   int M, int N, int K, const void* bias, const void* residual, int ldr,
                                   const void* gate, int gate_stride, int rows_per_batch, int act,
                                   int c_rows_per_batch, long c_batch_stride, int scatter_P, int scatter_G,
                                   int scatter_rows, void* const* peer_out, int force_bn, const omni::OmniSync* sync,
                                   int* status, void* stream) {
  using namespace omni;
  if (M <= 0 || N <= 0 || K <= 0) return sync ? RC_BAD_ARG : RC_OK;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7) || (ldr & 7) || (gate_stride & 7))
    return RC_BAD_ARG;
  if (gate && rows_per_batch <= 0) return RC_BAD_ARG;
  CUtensorMap tmA;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K,
                        (uint64_t)lda * 2, BM, BK);
  if (rc) return rc;
  GemmEpilogue epi;
  epi.bias = static_cast<const __nv_bfloat16*>(bias);
  epi.residual = static_cast<const __nv_bfloat16*>(residual);
  epi.gate = static_cast<const __nv_bfloat16*>(gate);
  epi.ldr = ldr;
  epi.gate_stride = gate_stride;
  epi.rows_per_batch = rows_per_batch > 0 ? rows_per_batch : 1;
  epi.act = act;
  epi.c_rows_per_batch = c_rows_per_batch;
  epi.c_batch_stride = c_batch_stride;
  if (c_rows_per_batch > 0 && (c_batch_stride & 7)) return RC_BAD_ARG;
  epi.scatter_P = 0;
  epi.scatter_G = 0;
  epi.scatter_rows = 0;
  for (int i = 0; i < 16; ++i) epi.peer_out[i] = nullptr;
  if (scatter_rows > 0) {
    // row owners: ceil(M / scatter_rows) ranks, at most 16
    const int owners = (M + scatter_rows - 1) / scatter_rows;
    if (owners > 16 || peer_out == nullptr || scatter_P != owners) return RC_BAD_ARG;
    epi.scatter_rows = scatter_rows;
    for (int i = 0; i < owners; ++i) epi.peer_out[i] = static_cast<__nv_bfloat16*>(peer_out[i]);
  } else if (scatter_P > 1) {
    if (scatter_P > 16 || scatter_G <= 0 || (scatter_G & 31) || peer_out == nullptr || (N % scatter_G)) return RC_BAD_ARG;
    epi.scatter_P = scatter_P;
    epi.scatter_G = scatter_G;
    for (int i = 0; i < scatter_P; ++i) epi.peer_out[i] = static_cast<__nv_bfloat16*>(peer_out[i]);
  }
  const int ctas = sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
  // force_bn = 576 / 448 / 384 selects the CTA-pair kernel with a 256 / 192 / 128 wide tile on two
  // SMs, 512 the pair kernel with the launcher's choice of width; in automatic mode the pair kernel takes every
  // problem with at least one full wave of 256 x 256 tiles
  TilePlan plan = {false, 0};
  if (force_bn == 0) plan = plan_tiles(&M, 1, N, ctas, g_pair_mode == 1 ? max_resident_pairs() : 0, g_pair_mode == 1);
  if (force_bn >= 384 || (force_bn == 0 && plan.pair)) {
    const int pairs = max_resident_pairs();
    const int tn = force_bn == 576 ? 256 : (force_bn == 448 ? 192 : (force_bn == 384 ? 128 :
                   (force_bn == 512 ? pick_pair_tn(M, N, pairs) : plan.bn)));
    PairArgs args = {};
    args.n_problems = 1; args.N = N; args.K = K;
    unpack_sync(sync, args.sig, args.wt);
    rc = fill_pair_problem(args.p[0], A, lda, W, ldw, c, ldc, M, N, K, epi, tn / 2);
    if (rc) return rc;
    return launch_pair_tn(tn, args, status, pairs, s);
  }
  const int bn = force_bn ? force_bn : plan.bn;
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, W, c, ldc, M, N, K, ldw, epi, status, ctas, s, 1, nullptr, nullptr, sync);
    case 192: return launch_gemm<192>(tmA, W, c, ldc, M, N, K, ldw, epi, status, ctas, s, 1, nullptr, nullptr, sync);
    case 128: return launch_gemm<128>(tmA, W, c, ldc, M, N, K, ldw, epi, status, ctas, s, 1, nullptr, nullptr, sync);
    default: return RC_BAD_ARG;
  }
}

extern "C" int omni_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                              int M, int N, int K, const void* bias, const void* residual, int ldr,
                              const void* gate, int gate_stride, int rows_per_batch, int act,
                              int c_rows_per_batch, long c_batch_stride, int scatter_P, int scatter_G,
                              int scatter_rows, void* const* peer_out, int force_bn, int* status, void* stream) {
  return omni_gemm_bf16_sync(A, lda, W, ldw, C, ldc, M, N, K, bias, residual, ldr, gate, gate_stride, rows_per_batch,
                             act, c_rows_per_batch, c_batch_stride, scatter_P, scatter_G, scatter_rows, peer_out,
                             force_bn, nullptr, status, stream);
}

// One-dimensional convolution, stride 1, channels-last bf16:
//   y[b, t, :] = act(sum_j x[b, t + j * dil - pad, :] W_j^T + bias) (+ residual),  t in [0, T_out)
// x: [B, T_in, Cin] with step pitch ldx (elements, multiple of 8) and batch pitch x_bs; inputs outside [0, T_in)
// read as zero.  w: [Cout, k * cin_pad], tap-major, cin_pad = ceil(Cin / 64) * 64, zero in the padding
// columns.  y / residual: rows b * T_out + t with pitch ldy / ldr.
extern "C" int omni_conv1d_nlc_bf16(const void* x, long ldx, long x_bs, const void* w, void* y, int ldy, int B, int T_in,
                                    int T_out, int Cin, int Cout, int k, int dil, int pad, const void* bias,
                                    const void* residual, int ldr, int act, int* status, void* stream) {
  using namespace omni;
  if (B <= 0 || T_in <= 0 || T_out <= 0 || Cin <= 0 || Cout <= 0) return RC_OK;
  if (k < 1 || k > 64 || dil < 1 || (Cout & 7) || (ldx & 7) || (x_bs & 7) || (ldy & 7) || (ldr & 7)) return RC_BAD_ARG;
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return RC_NO_DRIVER;
  if (reinterpret_cast<uintptr_t>(x) & 15) return RC_BAD_ARG;
  ConvGeom g = {};
  g.taps = k;
  g.H = 1; g.W = T_out;
  g.tiles_x = (T_out + BM - 1) / BM;
  g.tiles_y = 1;
  g.cin_blocks = (Cin + BK - 1) / BK;
  g.one_d = 1; g.dil = dil; g.pad = pad;
  CUtensorMap tmA;
  {
    cuuint64_t gdim[4] = {(cuuint64_t)Cin, (cuuint64_t)T_in, 1, (cuuint64_t)B};
    cuuint64_t gstr[3] = {(cuuint64_t)ldx * 2, (cuuint64_t)ldx * 2 * T_in, (cuuint64_t)x_bs * 2};
    cuuint32_t box[4] = {BK, BM, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return RC_TMAP;
  }
  GemmEpilogue epi = {};
  epi.bias = static_cast<const __nv_bfloat16*>(bias);
  epi.residual = static_cast<const __nv_bfloat16*>(residual);
  epi.ldr = ldr;
  epi.rows_per_batch = 1;
  epi.act = act;
  const int K = g.taps * g.cin_blocks * BK;
  const int M = B * g.tiles_x * BM;
  const int ctas = sm_count();
  const int bn = pick_bn(M, Cout, ctas);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(y);
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
    case 192: return launch_gemm<192>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
    default: return launch_gemm<128>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
  }
}

// Two linear layers of the same shape (N, K) in one launch of the CTA-pair kernel: the image and
// text streams of a dual-stream DiT block.  Each descriptor carries its own activations, weights,
// output mapping and epilogue operands.  Falls back to two launches when the pair kernel does not
// apply (too few tiles for one wave).
struct OmniGemmDesc {
  const void* A; const void* W; void* C;
  const void* bias; const void* residual; const void* gate;
  long c_batch_stride;
  int lda, ldw, ldc, M, ldr, gate_stride, rows_per_batch, act, c_rows_per_batch;
  int scatter_P, scatter_G;      // > 1: column groups of scatter_G go to peer_out[g % scatter_P] (see GemmEpilogue)
  void* peer_out[16];
};

static int desc_epilogue(const OmniGemmDesc& d, omni::GemmEpilogue& epi) {
  if ((d.lda & 7) || (d.ldw & 7) || (d.ldc & 7) || (d.ldr & 7) || (d.gate_stride & 7)) return omni::RC_BAD_ARG;
  if (d.gate && d.rows_per_batch <= 0) return omni::RC_BAD_ARG;
  if (d.c_rows_per_batch > 0 && (d.c_batch_stride & 7)) return omni::RC_BAD_ARG;
  epi = omni::GemmEpilogue{};
  epi.bias = static_cast<const __nv_bfloat16*>(d.bias);
  epi.residual = static_cast<const __nv_bfloat16*>(d.residual);
  epi.gate = static_cast<const __nv_bfloat16*>(d.gate);
  epi.ldr = d.ldr;
  epi.gate_stride = d.gate_stride;
  epi.rows_per_batch = d.rows_per_batch > 0 ? d.rows_per_batch : 1;
  epi.act = d.act;
  epi.c_rows_per_batch = d.c_rows_per_batch;
  epi.c_batch_stride = d.c_batch_stride;
  if (d.scatter_P > 1) {
    if (d.scatter_P > 16 || d.scatter_G <= 0 || (d.scatter_G & 31)) return omni::RC_BAD_ARG;
    epi.scatter_P = d.scatter_P;
    epi.scatter_G = d.scatter_G;
    for (int i = 0; i < d.scatter_P; ++i) epi.peer_out[i] = static_cast<__nv_bfloat16*>(d.peer_out[i]);
  }
  return omni::RC_OK;
}

// One launch for both problems: the CTA-pair kernel (256-row tiles) or the one-CTA kernel (128-row
// tiles), whichever tile plan finishes sooner.  With `sync` the launch waits and reports once.
extern "C" int omni_gemm_bf16_dual_sync(const OmniGemmDesc* d0, const OmniGemmDesc* d1, int N, int K, int force_pair,
                                        const omni::OmniSync* sync, int* status, void* stream) {
  using namespace omni;
  if (!d0 || !d1 || N <= 0 || K <= 0 || (N & 7) || (K & 7)) return RC_BAD_ARG;
  const OmniGemmDesc* ds[2] = {d0, d1};
  const int ctas = sm_count();
  if (d0->M <= 0 || d1->M <= 0) {
    // one of the two is empty: a plain launch of the other carries the whole synchronisation
    const OmniGemmDesc& d = d0->M > 0 ? *d0 : *d1;
    if (d.M <= 0) return sync ? RC_BAD_ARG : RC_OK;
    if (d.scatter_P > 1 && (N % d.scatter_G)) return RC_BAD_ARG;
    return omni_gemm_bf16_sync(d.A, d.lda, d.W, d.ldw, d.C, d.ldc, d.M, N, K, d.bias, d.residual, d.ldr, d.gate,
                               d.gate_stride, d.rows_per_batch, d.act, d.c_rows_per_batch, d.c_batch_stride,
                               d.scatter_P > 1 ? d.scatter_P : 0, d.scatter_P > 1 ? d.scatter_G : 0, 0,
                               d.scatter_P > 1 ? d.peer_out : nullptr, 0, sync, status, stream);
  }
  const int pairs = max_resident_pairs();
  const int Ms[2] = {d0->M, d1->M};
  TilePlan plan = plan_tiles(Ms, 2, N, ctas, pairs, g_pair_mode == 1 || force_pair);
  if (force_pair) { plan.pair = true; plan.bn = pick_pair_tn(d0->M + d1->M, N, pairs); }
  PairArgs args = {};
  args.n_problems = 2; args.N = N; args.K = K;
  unpack_sync(sync, args.sig, args.wt);
  for (int i = 0; i < 2; ++i) {
    GemmEpilogue epi;
    int rc = desc_epilogue(*ds[i], epi);
    if (rc) return rc;
    if (epi.scatter_P > 1 && (N % epi.scatter_G)) return RC_BAD_ARG;
    rc = fill_pair_problem(args.p[i], ds[i]->A, ds[i]->lda, ds[i]->W, ds[i]->ldw, static_cast<__nv_bfloat16*>(ds[i]->C),
                           ds[i]->ldc, ds[i]->M, N, K, epi, plan.pair ? plan.bn / 2 : plan.bn);
    if (rc) return rc;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return plan.pair ? launch_pair_tn(plan.bn, args, status, pairs, st) : launch_multi_bn(plan.bn, args, status, ctas, st);
}

extern "C" int omni_gemm_bf16_dual(const OmniGemmDesc* d0, const OmniGemmDesc* d1, int N, int K, int force_pair,
                                   int* status, void* stream) {
  return omni_gemm_bf16_dual_sync(d0, d1, N, K, force_pair, nullptr, status, stream);
}

// 0: the CTA-pair kernel runs only when forced (force_bn = 512); 1: automatic for large problems.
extern "C" void omni_gemm_set_pair_mode(int mode) { omni::g_pair_mode = mode; }

// Grouped (MoE expert) GEMM: A is the expert-major, 128-row-padded activation buffer [M, K];
// W is [E, N, K] contiguous; tile_expert[m_tile] names the expert of every 128-row tile (-1 =
// padding, skipped).  C[M, N] = act(A * W[e]^T).
extern "C" int omni_gemm_bf16_grouped(const void* A, int lda, const void* W, int num_experts, void* C, int ldc,
                                      int M, int N, int K, const int* tile_expert, int act, int force_bn,
                                      int* status, void* stream) {
  using namespace omni;
  if (M <= 0 || N <= 0 || K <= 0) return RC_OK;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldc & 7) || (M % BM) || tile_expert == nullptr) return RC_BAD_ARG;
  CUtensorMap tmA;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K,
                        (uint64_t)lda * 2, BM, BK);
  if (rc) return rc;
  GemmEpilogue epi = {};
  epi.rows_per_batch = 1;
  epi.act = act;
  const int ctas = sm_count();
  const int bn = force_bn ? force_bn : pick_bn(M, N, ctas);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert);
    case 192: return launch_gemm<192>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert);
    case 128: return launch_gemm<128>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert);
    default: return RC_BAD_ARG;
  }
}


// Grouped GEMM over experts whose rows sit back to back (no padding): M rows in A and C in total, M-tile t
// covers rows [tile_row0[t], tile_row0[t] + tile_rows[t]) of expert tile_expert[t] (-1 = unused tile).
extern "C" int omni_gemm_bf16_grouped_compact(const void* A, int lda, const void* W, int num_experts, void* C, int ldc,
                                              int M, int N, int K, const int* tile_expert, const int* tile_row0,
                                              const int* tile_rows, int num_tiles, int act, int force_bn, int* status,
                                              void* stream) {
  using namespace omni;
  if (M <= 0 || N <= 0 || K <= 0 || num_tiles <= 0) return RC_OK;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldc & 7) || !tile_expert || !tile_row0 || !tile_rows) return RC_BAD_ARG;
  CUtensorMap tmA;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K,
                        (uint64_t)lda * 2, BM, BK);
  if (rc) return rc;
  GemmEpilogue epi = {};
  epi.rows_per_batch = 1;
  epi.act = act;
  GroupTiles gt = {tile_row0, tile_rows, num_tiles};
  const int ctas = sm_count();
  const int bn = force_bn ? force_bn : pick_bn(num_tiles * BM, N, ctas);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert, nullptr, nullptr, &gt);
    case 192: return launch_gemm<192>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert, nullptr, nullptr, &gt);
    case 128: return launch_gemm<128>(tmA, W, c, ldc, M, N, K, K, epi, status, ctas, s, num_experts, tile_expert, nullptr, nullptr, &gt);
    default: return RC_BAD_ARG;
  }
}


// Convolution, stride 1, zero "same" padding, NHWC bf16:  y[n,h,w,:] = act(sum_taps x[n,h+dy,w+dx,:] W_tap^T + bias)
// (+ residual).  x: [Nimg, H, W, Cin] with pixel pitch ldx (elements, >= Cin, multiple of 8);
// w: [Cout, taps * cin_pad] with cin_pad = ceil(Cin / 64) * 64, tap-major (tap = ky * 3 + kx for 3x3),
// zero in the padding columns; y / residual: [Nimg*H*W, ldy / ldr].  ksize is 1 or 3.
extern "C" int omni_conv2d_nhwc_bf16(const void* x, long ldx, const void* w, void* y, int ldy, int Nimg, int H, int W,
                                     int Cin, int Cout, int ksize, const void* bias, const void* residual, int ldr,
                                     int act, int* status, void* stream) {
  using namespace omni;
  if (Nimg <= 0 || H <= 0 || W <= 0 || Cin <= 0 || Cout <= 0) return RC_OK;
  if ((ksize != 1 && ksize != 3) || (Cout & 7) || (ldx & 7) || (ldy & 7) || (ldr & 7)) return RC_BAD_ARG;
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return RC_NO_DRIVER;
  if (reinterpret_cast<uintptr_t>(x) & 15) return RC_BAD_ARG;
  ConvGeom g = {};
  g.taps = ksize * ksize;
  g.H = H; g.W = W;
  g.tiles_x = (W + CONV_BW - 1) / CONV_BW;
  g.tiles_y = (H + CONV_BH - 1) / CONV_BH;
  g.cin_blocks = (Cin + BK - 1) / BK;
  CUtensorMap tmA;
  {
    cuuint64_t gdim[4] = {(cuuint64_t)Cin, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)Nimg};
    cuuint64_t gstr[3] = {(cuuint64_t)ldx * 2, (cuuint64_t)ldx * 2 * W, (cuuint64_t)ldx * 2 * W * H};
    cuuint32_t box[4] = {BK, CONV_BW, CONV_BH, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return RC_TMAP;
  }
  GemmEpilogue epi = {};
  epi.bias = static_cast<const __nv_bfloat16*>(bias);
  epi.residual = static_cast<const __nv_bfloat16*>(residual);
  epi.ldr = ldr;
  epi.rows_per_batch = 1;
  epi.act = act;
  const int K = g.taps * g.cin_blocks * BK;
  const int M = Nimg * g.tiles_x * g.tiles_y * BM;       // rows as the tile scheduler counts them
  const int ctas = sm_count();
  const int bn = pick_bn(M, Cout, ctas);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* c = static_cast<__nv_bfloat16*>(y);
  switch (bn) {
    case 256: return launch_gemm<256>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
    case 192: return launch_gemm<192>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
    default: return launch_gemm<128>(tmA, w, c, ldy, M, Cout, K, K, epi, status, ctas, s, 1, nullptr, &g);
  }
}
