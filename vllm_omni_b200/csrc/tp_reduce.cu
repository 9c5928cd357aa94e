// K2: the reduce + all-gather half of the tensor-parallel row-parallel linear layer.
//
// The GEMM before it (gemm_sm100.cu, scatter_rows epilogue) has already pushed every rank's
// partial product over NVLink into the slot reserved for it on the rank that OWNS each block of
// rows, so after one barrier the P partial sums of my rows sit in MY memory:
//
//   slots [P, rows_per_owner, N]   slot s = partial sums of my rows computed by rank s (bf16)
//
// This kernel adds them in fp32, applies bias, the per-batch gate and the residual, converts to
// bf16 and stores the finished rows into the result buffer of EVERY rank (plain peer stores), so
// that after the second barrier all ranks hold the full [M, N] activation again.  All loads are
// local; only stores cross NVLink.
//
// The reference reaches the same result with vLLM's RowParallelLinear: cuBLAS GEMM, NCCL
// all-reduce of the whole [M, N] tensor, then eager gate / residual kernels
// (vllm_omni/diffusion/distributed/parallel_state.py:769, qwen_image_transformer.py:427-560).
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

struct TpPeers {
  __nv_bfloat16* result[16];   // [M, ldres] on every rank (peer-mapped or local)
};

__global__ void __launch_bounds__(256)
tp_reduce_gather_kernel(const __nv_bfloat16* __restrict__ slots, int P, int rows_per_owner, int N, int row0,
                        int n_rows, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ gate,
                        int gate_stride, int rows_per_batch, const __nv_bfloat16* __restrict__ residual, long ldr,
                        TpPeers peers, long ldres) {
  const int chunks = N >> 3;
  const long total = (long)n_rows * chunks;
  const size_t slot_elems = (size_t)rows_per_owner * N;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int lr = (int)(i / chunks);          // row inside my block
    const int c = (int)(i % chunks) * 8;
    const int row = row0 + lr;                 // row of the full activation
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < P; ++s) {
      const uint4 u = *reinterpret_cast<const uint4*>(slots + s * slot_elems + (size_t)lr * N + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (bias) {
      const uint4 u = *reinterpret_cast<const uint4*>(bias + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (gate) {
      const uint4 u = *reinterpret_cast<const uint4*>(gate + (size_t)(row / rows_per_batch) * gate_stride + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] *= a.x; acc[1] *= a.y; acc[2] *= b.x; acc[3] *= b.y;
      acc[4] *= cc.x; acc[5] *= cc.y; acc[6] *= d.x; acc[7] *= d.y;
    }
    if (residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + (size_t)row * ldr + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    for (int d = 0; d < P; ++d) *reinterpret_cast<uint4*>(peers.result[d] + (size_t)row * ldres + c) = o;
  }
}

}  // namespace omni

using namespace omni;

// slots: this rank's [P, rows_per_owner, N] slot block; rows [row0, row0 + n_rows) of the full
// activation are mine; result_ptrs[d]: rank d's [M, ldres] result buffer.
extern "C" int omni_tp_reduce_gather(const void* slots, int P, int rows_per_owner, int N, int row0, int n_rows,
                                     const void* bias, const void* gate, int gate_stride, int rows_per_batch,
                                     const void* residual, long ldr, void* const* result_ptrs, long ldres,
                                     void* stream) {
  if (n_rows <= 0) return RC_OK;
  if (P < 1 || P > 16 || (N & 7) || (ldr & 7) || (ldres & 7) || (gate_stride & 7) || n_rows > rows_per_owner ||
      result_ptrs == nullptr)
    return RC_BAD_ARG;
  if (gate && rows_per_batch <= 0) return RC_BAD_ARG;
  TpPeers peers;
  for (int i = 0; i < 16; ++i) peers.result[i] = i < P ? static_cast<__nv_bfloat16*>(result_ptrs[i]) : nullptr;
  const long total = (long)n_rows * (N >> 3);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  tp_reduce_gather_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(slots), P, rows_per_owner, N, row0, n_rows, static_cast<const __nv_bfloat16*>(bias),
      static_cast<const __nv_bfloat16*>(gate), gate_stride, rows_per_batch > 0 ? rows_per_batch : 1,
      static_cast<const __nv_bfloat16*>(residual), ldr, peers, ldres);
  return (int)cudaGetLastError();
}
