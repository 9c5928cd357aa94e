// Bandwidth-bound fused kernels of the DiT / AR blocks (K6, K7, K8, K9, K14).
// Each of them reads its inputs once with 16-byte vector loads, does all arithmetic in
// fp32 registers and writes bf16 once, so the roofline is bytes / HBM bandwidth.
//
//  omni_norm_modulate   LayerNorm / RMSNorm (+weight, +bias) fused with the AdaLN
//                       modulation y = norm(x) * (1 + scale[b]) + shift[b]
//                       (reference: vllm_omni/diffusion/layers/adalayernorm.py)
//  omni_qk_norm_rope    per-head RMSNorm of q and k fused with rotary embedding, in place on
//                       a packed [B, S, 3, H, D] qkv buffer; interleaved (complex-pair) or
//                       half-rotation layout; separate norm weights for rows >= s_alt (the text
//                       rows that follow the image rows in the joint sequence)
//                       (reference: qwen_image_transformer.py:561-661, layers/rope.py:94-154)
//  omni_cfg_euler_step  guidance mix neg + s (pos - neg), optional norm rescale, flow-match
//                       Euler update x += dt * v, bf16 copy of the new latents
//                       (reference: vllm_omni/diffusion/distributed/cfg_parallel.py:99-137)
//  omni_silu_mul        SwiGLU gate: silu(x[:, :N]) * x[:, N:]
//  omni_rel_l1_partial / omni_rel_l1_finish
//                       TeaCache residual metric sum|a-b| / sum|b| with the polynomial
//                       rescale, accumulation and skip decision kept on the device
//                       (reference: vllm_omni/diffusion/cache/teacache/hook.py:185-232)
#include "host_util.h"
#include "ptx_sm100.cuh"
#include "peer_signal.cuh"

namespace omni {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
  uint4 u;
  u.x = pack_bf16(x[0], x[1]); u.y = pack_bf16(x[2], x[3]);
  u.z = pack_bf16(x[4], x[5]); u.w = pack_bf16(x[6], x[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------- norm + modulate
// One CTA (256 threads) per row; each thread keeps up to MAXV 8-element chunks in
// registers, so the row is read exactly once.  D % 8 == 0, D <= 256 * 8 * MAXV.
constexpr int NM_THREADS = 256;
constexpr int NM_MAXV = 4;

__global__ void __launch_bounds__(NM_THREADS)
norm_modulate_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int rows,
                     int D, int ldx, int ldy, const __nv_bfloat16* __restrict__ weight,
                     const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ shift,
                     const __nv_bfloat16* __restrict__ scale, int mod_stride, int rows_per_batch,
                     int rms, float eps) {
  __shared__ float red[2][NM_THREADS / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  float v[NM_MAXV][8];
  float s = 0.f, ss = 0.f;
  const int nchunk = D >> 3;
#pragma unroll
  for (int i = 0; i < NM_MAXV; ++i) {
    const int c = threadIdx.x + i * NM_THREADS;
    if (c < nchunk) {
      load8(xr + c * 8, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) { s += v[i][e]; ss += v[i][e] * v[i][e]; }
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = ss; }
  __syncthreads();
  s = 0.f; ss = 0.f;
#pragma unroll
  for (int w = 0; w < NM_THREADS / 32; ++w) { s += red[0][w]; ss += red[1][w]; }
  const float inv_d = 1.0f / (float)D;
  float mean = rms ? 0.f : s * inv_d;
  float var = rms ? ss * inv_d : fmaxf(ss * inv_d - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  const int b = row / rows_per_batch;
  const __nv_bfloat16* sh = shift ? shift + (size_t)b * mod_stride : nullptr;
  const __nv_bfloat16* sc = scale ? scale + (size_t)b * mod_stride : nullptr;
  __nv_bfloat16* yr = y + (size_t)row * ldy;
#pragma unroll
  for (int i = 0; i < NM_MAXV; ++i) {
    const int c = threadIdx.x + i * NM_THREADS;
    if (c < nchunk) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd;
      if (weight) { float w[8]; load8(weight + c * 8, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= w[e]; }
      if (bias) { float w[8]; load8(bias + c * 8, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += w[e]; }
      if (sc) { float w[8]; load8(sc + c * 8, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= (1.0f + w[e]); }
      if (sh) { float w[8]; load8(sh + c * 8, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += w[e]; }
      store8(yr + c * 8, o);
    }
  }
}

// Warp-per-row variant: the row stays packed (bf16) in VPL 16-byte registers per lane, all
// loads of a row are in flight at once, no shared memory and no block barrier.
template <int VPL>
__global__ void __launch_bounds__(256)
norm_modulate_warp_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int rows,
                          int D, int ldx, int ldy, const __nv_bfloat16* __restrict__ weight,
                          const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ shift,
                          const __nv_bfloat16* __restrict__ scale, int mod_stride, int rows_per_batch,
                          int rms, float eps) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nchunk = D >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint4 v[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + i * 32;
    v[i] = c < nchunk ? xr[c] : make_uint4(0u, 0u, 0u, 0u);
  }
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      s += f.x + f.y;
      ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const float inv_d = 1.0f / (float)D;
  const float mean = rms ? 0.f : s * inv_d;
  const float var = rms ? ss * inv_d : fmaxf(ss * inv_d - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  const int b = row / rows_per_batch;
  const __nv_bfloat16* sh = shift ? shift + (size_t)b * mod_stride : nullptr;
  const __nv_bfloat16* sc = scale ? scale + (size_t)b * mod_stride : nullptr;
  __nv_bfloat16* yr = y + (size_t)row * ldy;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + i * 32;
    if (c < nchunk) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(w[j]);
        o[2 * j] = (f.x - mean) * rstd;
        o[2 * j + 1] = (f.y - mean) * rstd;
      }
      if (weight) { float t[8]; load8(weight + c * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= t[e]; }
      if (bias) { float t[8]; load8(bias + c * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += t[e]; }
      if (sc) { float t[8]; load8(sc + c * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(o[e], t[e], o[e]); }
      if (sh) { float t[8]; load8(sh + c * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += t[e]; }
      store8(yr + c * 8, o);
    }
  }
}

// Fast q/k norm + rope for D = 128: one warp per (batch, position) row walks all q and k heads
// of that row; half a warp owns one head (8 contiguous elements per lane, one 16-byte access),
// four heads-pairs are in flight per iteration.
__global__ void __launch_bounds__(256)
qk_norm_rope128_kernel(__nv_bfloat16* __restrict__ qkv, long rows, int S, int H, int Hkv, int ld,
                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                       const __nv_bfloat16* __restrict__ wq_alt, const __nv_bfloat16* __restrict__ wk_alt,
                       int s_alt, const float* __restrict__ cosb, const float* __restrict__ sinb,
                       int interleaved, float eps, const int* __restrict__ positions, PeerWait wt, int* status) {
  constexpr int D = 128;
  if (wt.counter) {
    // fused exchange: the rows come from the peers' QKV GEMM epilogues; wait for their arrivals
    // here instead of in a barrier kernel of its own
    if (threadIdx.x == 0) {
      peer_wait_arrivals(wt, nullptr, status);
      peer_wait_cta_exit(wt, gridDim.x);      // only this thread reads the epoch word
    }
    __syncthreads();
  }
  const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int l16 = lane & 15;
  const int hsel = lane >> 4;
  const int s = (int)(row % S);
  const int pos = positions ? positions[row] : s;
  const bool alt = s >= s_alt;
  const __nv_bfloat16* wqq = (alt && wq_alt) ? wq_alt : wq;
  const __nv_bfloat16* wkk = (alt && wk_alt) ? wk_alt : wk;
  float wqf[8], wkf[8];
  if (wqq) { load8(wqq + l16 * 8, wqf); load8(wkk + l16 * 8, wkf); }
  // rotation coefficients of this lane's elements
  float cs[8], sn[8];
  if (cosb) {
    const float* cr = cosb + (size_t)pos * (D / 2);
    const float* sr = sinb + (size_t)pos * (D / 2);
    if (interleaved) {   // elements 8*l16 .. +7 = pairs 4*l16 .. +3
      const float4 c4 = *reinterpret_cast<const float4*>(cr + 4 * l16);
      const float4 s4 = *reinterpret_cast<const float4*>(sr + 4 * l16);
      cs[0] = cs[1] = c4.x; cs[2] = cs[3] = c4.y; cs[4] = cs[5] = c4.z; cs[6] = cs[7] = c4.w;
      sn[0] = -s4.x; sn[1] = s4.x; sn[2] = -s4.y; sn[3] = s4.y; sn[4] = -s4.z; sn[5] = s4.z; sn[6] = -s4.w; sn[7] = s4.w;
    } else {             // element i pairs with i +- 64; frequency index i mod 64
      const int f0 = (l16 & 7) * 8;
      const float sign = l16 < 8 ? -1.f : 1.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) { cs[e] = cr[f0 + e]; sn[e] = sign * sr[f0 + e]; }
    }
  }
  __nv_bfloat16* base = qkv + (size_t)row * ld;
  const int heads = H + Hkv;
  constexpr int U = 4;
  for (int h0 = 0; h0 < heads; h0 += 2 * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int h = h0 + 2 * u + hsel;
      v[u] = h < heads ? *reinterpret_cast<const uint4*>(base + (size_t)h * D + l16 * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int h = h0 + 2 * u + hsel;
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      float xv[8];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16(w[j]);
        xv[2 * j] = f.x; xv[2 * j + 1] = f.y;
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
      if (wqq) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = rsqrtf(ss * (1.0f / D) + eps);
        const bool is_k = h >= H;
#pragma unroll
        for (int e = 0; e < 8; ++e) xv[e] = xv[e] * r * (is_k ? wkf[e] : wqf[e]);
      }
      if (cosb) {
        if (interleaved) {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float a = xv[e], bb = xv[e + 1];
            xv[e] = fmaf(a, cs[e], bb * sn[e]);          // a*c - b*s
            xv[e + 1] = fmaf(bb, cs[e + 1], a * sn[e + 1]);  // b*c + a*s
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float partner = __shfl_xor_sync(0xffffffffu, xv[e], 8);
            xv[e] = fmaf(xv[e], cs[e], partner * sn[e]);
          }
        }
      }
      if (h < heads) store8(base + (size_t)h * D + l16 * 8, xv);
    }
  }
}

// ------------------------------------------------------------------ qk norm + rope
// qkv: [B, S, 3, H, D] (row pitch ld elements between consecutive s), D in {64, 128}.
// One warp per (row, head); lane owns D/32 consecutive elements (2 or 4), i.e. whole
// (even, odd) pairs for the interleaved layout.  For the half-rotation layout lane l
// owns elements {l*D/64 .. } of both halves.  cos/sin: [S, D/2] fp32.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(__nv_bfloat16* __restrict__ qkv, int B, int S, int H, int Hkv, int ld,
                    const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                    const __nv_bfloat16* __restrict__ wq_alt, const __nv_bfloat16* __restrict__ wk_alt,
                    int s_alt, const float* __restrict__ cosb, const float* __restrict__ sinb,
                    int interleaved, float eps, const int* __restrict__ positions) {
  constexpr int E = D / 32;  // elements per lane
  const int warps_per_block = blockDim.x >> 5;
  const long gw = (long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = H + Hkv;
  const long total = (long)B * S * heads;
  if (gw >= total) return;
  const int hh = (int)(gw % heads);
  const long rs = gw / heads;
  const int s = (int)(rs % S);
  const int b = (int)(rs / S);
  const bool is_k = hh >= H;
  const int h = is_k ? hh - H : hh;
  __nv_bfloat16* p = qkv + ((size_t)b * S + s) * ld + (is_k ? (size_t)H * D : 0) + (size_t)h * D;
  const __nv_bfloat16* w = is_k ? (s >= s_alt && wk_alt ? wk_alt : wk) : (s >= s_alt && wq_alt ? wq_alt : wq);
  const int pos = positions ? positions[(size_t)b * S + s] : s;

  float x[E];
  int idx[E];
  if (interleaved) {
#pragma unroll
    for (int e = 0; e < E; ++e) idx[e] = lane * E + e;
  } else {
    // lane owns E/2 elements in each half so that rotation partners sit in one lane
#pragma unroll
    for (int e = 0; e < E / 2; ++e) { idx[e] = lane * (E / 2) + e; idx[e + E / 2] = D / 2 + lane * (E / 2) + e; }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) { x[e] = __bfloat162float(p[idx[e]]); ss += x[e] * x[e]; }
  if (w) {
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int e = 0; e < E; ++e) x[e] = x[e] * r * __bfloat162float(w[idx[e]]);
  }
  if (cosb) {
    const float* cr = cosb + (size_t)pos * (D / 2);
    const float* sr = sinb + (size_t)pos * (D / 2);
    if (interleaved) {
#pragma unroll
      for (int e = 0; e < E; e += 2) {
        const int pi = idx[e] >> 1;
        const float c = cr[pi], sn = sr[pi];
        const float a = x[e], bb = x[e + 1];
        x[e] = a * c - bb * sn;
        x[e + 1] = a * sn + bb * c;
      }
    } else {
#pragma unroll
      for (int e = 0; e < E / 2; ++e) {
        const int pi = idx[e];
        const float c = cr[pi], sn = sr[pi];
        const float a = x[e], bb = x[e + E / 2];
        x[e] = a * c - bb * sn;
        x[e + E / 2] = bb * c + a * sn;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < E; ++e) p[idx[e]] = __float2bfloat16(x[e]);
}

// ------------------------------------------------------------ CFG mix + Euler step
// pos/neg: [rows, C] bf16 velocity predictions; lat: [rows, C] fp32 latents (in place);
// lat_bf16: bf16 copy of the updated latents for the next transformer call.
// One warp per row.  neg == nullptr means no guidance (v = pos).
__global__ void __launch_bounds__(256)
cfg_euler_kernel(const __nv_bfloat16* __restrict__ pos, const __nv_bfloat16* __restrict__ neg,
                 float* __restrict__ lat, __nv_bfloat16* __restrict__ lat_bf16, long rows, int C,
                 float guidance, float dt, int renorm) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const size_t base = (size_t)row * C;
  float pn = 0.f, cn = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float p = __bfloat162float(pos[base + c]);
    float v = p;
    if (neg) {
      const float n = __bfloat162float(neg[base + c]);
      v = n + guidance * (p - n);
    }
    pn += p * p;
    cn += v * v;
  }
  float resc = 1.0f;
  if (renorm && neg) {
    pn = warp_sum(pn);
    cn = warp_sum(cn);
    resc = sqrtf(pn) / fmaxf(sqrtf(cn), 1e-12f);
  }
  for (int c = lane; c < C; c += 32) {
    const float p = __bfloat162float(pos[base + c]);
    float v = p;
    if (neg) {
      const float n = __bfloat162float(neg[base + c]);
      v = (n + guidance * (p - n)) * resc;
    }
    const float x = lat[base + c] + dt * v;
    lat[base + c] = x;
    if (lat_bf16) lat_bf16[base + c] = __float2bfloat16(x);
  }
}

// ------------------------------------------------------------------------ SwiGLU
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows, int N,
                int ldx, int ldy) {
  const long nchunk = (long)rows * (N >> 3);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nchunk; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (N >> 3);
    const int c = (int)(i % (N >> 3)) * 8;
    float g[8], u[8], o[8];
    load8(x + r * ldx + c, g);
    load8(x + r * ldx + N + c, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = silu(g[e]) * u[e];
    store8(y + r * ldy + c, o);
  }
}

// --------------------------------------------------------- TeaCache rel-L1 metric
// Stage 1: every CTA writes its partial (sum|a-b|, sum|b|) into scratch[2*blockIdx.x].
// Stage 2 (one CTA): reduces the partials, applies the polynomial rescale, accumulates
// and decides; state = {accumulated, last_rel_l1, skip_flag(as float), steps_skipped}.
constexpr int RL_THREADS = 256;

__global__ void __launch_bounds__(RL_THREADS)
rel_l1_partial_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, long n8,
                      float* __restrict__ scratch) {
  __shared__ float red[2][RL_THREADS / 32];
  float d = 0.f, m = 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    load8(a + i * 8, x);
    load8(b + i * 8, y);
#pragma unroll
    for (int e = 0; e < 8; ++e) { d += fabsf(x[e] - y[e]); m += fabsf(y[e]); }
  }
  d = warp_sum(d);
  m = warp_sum(m);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = d; red[1][threadIdx.x >> 5] = m; }
  __syncthreads();
  if (threadIdx.x == 0) {
    d = 0.f; m = 0.f;
    for (int w = 0; w < RL_THREADS / 32; ++w) { d += red[0][w]; m += red[1][w]; }
    scratch[2 * blockIdx.x] = d;
    scratch[2 * blockIdx.x + 1] = m;
  }
}

__global__ void __launch_bounds__(RL_THREADS)
rel_l1_finish_kernel(const float* __restrict__ scratch, int nparts, float* __restrict__ state,
                     const float* __restrict__ coef, int ncoef, float thresh, int force_compute,
                     float* __restrict__ sums_out) {
  __shared__ float red[2][RL_THREADS / 32];
  float d = 0.f, m = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) { d += scratch[2 * i]; m += scratch[2 * i + 1]; }
  d = warp_sum(d);
  m = warp_sum(m);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = d; red[1][threadIdx.x >> 5] = m; }
  __syncthreads();
  if (threadIdx.x == 0) {
    d = 0.f; m = 0.f;
    for (int w = 0; w < RL_THREADS / 32; ++w) { d += red[0][w]; m += red[1][w]; }
    if (sums_out) { sums_out[0] = d; sums_out[1] = m; }
    if (state) {
      // mean|a-b| / (mean|b| + 1e-8) with equal element counts reduces to the ratio of sums
      const float rel = d / (m + 1e-8f);
      float r = rel;
      if (ncoef > 0) {  // numpy.poly1d order: highest power first
        r = coef[0];
        for (int i = 1; i < ncoef; ++i) r = r * rel + coef[i];
      }
      // the reference accumulates |rescale(rel)| (teacache/hook.py:225): a polynomial that dips below
      // zero at small rel must not pull the accumulator down
      float acc = state[0] + fabsf(r);
      float skip = 0.f;
      if (!force_compute && acc < thresh) skip = 1.f; else acc = 0.f;
      state[0] = acc;
      state[1] = rel;
      state[2] = skip;
      state[3] += skip;
    }
  }
}

}  // namespace omni

using namespace omni;

extern "C" int omni_norm_modulate(const void* x, void* y, int rows, int D, int ldx, int ldy,
                                  const void* weight, const void* bias, const void* shift,
                                  const void* scale, int mod_stride, int rows_per_batch, int rms,
                                  float eps, void* stream) {
  if (rows <= 0) return RC_OK;
  if ((D & 7) || D > NM_THREADS * 8 * NM_MAXV || (ldx & 7) || (ldy & 7) || (mod_stride & 7)) return RC_BAD_ARG;
  if (rows_per_batch <= 0) rows_per_batch = rows;
  auto xx = (const __nv_bfloat16*)x; auto yy = (__nv_bfloat16*)y;
  auto w = (const __nv_bfloat16*)weight; auto bb = (const __nv_bfloat16*)bias;
  auto sh = (const __nv_bfloat16*)shift; auto sc = (const __nv_bfloat16*)scale;
  cudaStream_t st = (cudaStream_t)stream;
  const int vpl = ((D >> 3) + 31) / 32;
  const unsigned wgrid = (unsigned)((rows + 7) / 8);
#define OMNI_NM_WARP(V) norm_modulate_warp_kernel<V><<<wgrid, 256, 0, st>>>(xx, yy, rows, D, ldx, ldy, w, bb, sh, sc, mod_stride, rows_per_batch, rms, eps)
  if (vpl <= 2) OMNI_NM_WARP(2);
  else if (vpl <= 4) OMNI_NM_WARP(4);
  else if (vpl <= 8) OMNI_NM_WARP(8);
  else if (vpl <= 12) OMNI_NM_WARP(12);
  else if (vpl <= 16) OMNI_NM_WARP(16);
  else if (vpl <= 20) OMNI_NM_WARP(20);
  else
    norm_modulate_kernel<<<rows, NM_THREADS, 0, st>>>(xx, yy, rows, D, ldx, ldy, w, bb, sh, sc, mod_stride,
                                                      rows_per_batch, rms, eps);
#undef OMNI_NM_WARP
  return (int)cudaGetLastError();
}

// `sync` (may be null, head_dim 128 only): arrivals from the peers' QKV epilogues that the kernel
// waits for before it touches the buffer (see peer_signal.cuh); `status` receives a timeout code.
extern "C" int omni_qk_norm_rope_sync(void* qkv, int B, int S, int H, int Hkv, int D, int ld, const void* wq,
                                      const void* wk, const void* wq_alt, const void* wk_alt, int s_alt,
                                      const float* cosb, const float* sinb, int interleaved, float eps,
                                      const int* positions, const OmniSync* sync, int* status, void* stream) {
  const long total = (long)B * S * (H + Hkv);
  if (total <= 0) return sync ? RC_BAD_ARG : RC_OK;
  PeerSignal unused;
  PeerWait wt;
  unpack_sync(sync, unused, wt);
  if (wt.counter && !(D == 128 && (ld & 7) == 0 && (wq != nullptr) == (wk != nullptr))) return RC_BAD_ARG;
  const int wpb = 8;
  const unsigned grid = (unsigned)((total + wpb - 1) / wpb);
  auto q = (__nv_bfloat16*)qkv;
  auto a = (const __nv_bfloat16*)wq; auto b = (const __nv_bfloat16*)wk;
  auto c = (const __nv_bfloat16*)wq_alt; auto d = (const __nv_bfloat16*)wk_alt;
  const bool have_w = wq != nullptr;
  if (D == 128 && (ld & 7) == 0 && (wq != nullptr) == (wk != nullptr)) {
    const long rows = (long)B * S;
    (void)have_w;
    qk_norm_rope128_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
        q, rows, S, H, Hkv, ld, a, b, c, d, s_alt, cosb, sinb, interleaved, eps, positions, wt, status);
  } else if (D == 128)
    qk_norm_rope_kernel<128><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(q, B, S, H, Hkv, ld, a, b, c, d, s_alt, cosb, sinb, interleaved, eps, positions);
  else if (D == 64)
    qk_norm_rope_kernel<64><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(q, B, S, H, Hkv, ld, a, b, c, d, s_alt, cosb, sinb, interleaved, eps, positions);
  else
    return RC_BAD_ARG;
  return (int)cudaGetLastError();
}

extern "C" int omni_qk_norm_rope(void* qkv, int B, int S, int H, int Hkv, int D, int ld, const void* wq,
                                 const void* wk, const void* wq_alt, const void* wk_alt, int s_alt,
                                 const float* cosb, const float* sinb, int interleaved, float eps,
                                 const int* positions, void* stream) {
  return omni_qk_norm_rope_sync(qkv, B, S, H, Hkv, D, ld, wq, wk, wq_alt, wk_alt, s_alt, cosb, sinb, interleaved, eps,
                                positions, nullptr, nullptr, stream);
}

extern "C" int omni_cfg_euler_step(const void* pos, const void* neg, float* lat, void* lat_bf16, long rows,
                                   int C, float guidance, float dt, int renorm, void* stream) {
  if (rows <= 0) return RC_OK;
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
  cfg_euler_kernel<<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)pos, (const __nv_bfloat16*)neg, lat, (__nv_bfloat16*)lat_bf16, rows, C, guidance, dt, renorm);
  return (int)cudaGetLastError();
}

extern "C" int omni_silu_mul(const void* x, void* y, long rows, int N, int ldx, int ldy, void* stream) {
  if (rows <= 0) return RC_OK;
  if ((N & 7) || (ldx & 7) || (ldy & 7)) return RC_BAD_ARG;
  const long nchunk = rows * (N >> 3);
  long blocks = (nchunk + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, N, ldx, ldy);
  return (int)cudaGetLastError();
}

// Number of partial pairs omni_rel_l1 writes for n elements (scratch needs 2x floats).
extern "C" int omni_rel_l1_parts(long n) {
  long blocks = ((n >> 3) + RL_THREADS - 1) / RL_THREADS;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// scratch: >= 2 * omni_rel_l1_parts(n) floats of device memory owned by the caller.
extern "C" int omni_rel_l1(const void* a, const void* b, long n, float* scratch, float* state,
                           const float* coef, int ncoef, float thresh, int force_compute,
                           float* sums_out, void* stream) {
  if (n <= 0 || (n & 7) || a == nullptr || b == nullptr || scratch == nullptr) return RC_BAD_ARG;
  if (ncoef < 0 || (state != nullptr && ncoef > 0 && coef == nullptr)) return RC_BAD_ARG;
  const int parts = omni_rel_l1_parts(n);
  rel_l1_partial_kernel<<<parts, RL_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, n >> 3, scratch);
  rel_l1_finish_kernel<<<1, RL_THREADS, 0, (cudaStream_t)stream>>>(scratch, parts, state, coef, ncoef, thresh, force_compute, sums_out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------
// Allocation-free variant of omni_rel_l1 (declared in omni_noalloc.h).
//
// The two-stage reduction needs 2 floats of scratch per stage-1 CTA.  The general entry
// point takes that scratch from the caller; this one keeps it in a file-scope device array
// so that a caller which owns no allocator can still use the kernel.
constexpr int RL_NOALLOC_MAX_PARTS = 148 * 4;                 // same cap as omni_rel_l1_parts()
constexpr long RL_NOALLOC_MAX_ELEMS = 1L << 28;               // 268,435,456 elements per operand
static __device__ __align__(256) float g_rel_l1_scratch[2 * RL_NOALLOC_MAX_PARTS];  // 4,736 bytes

namespace {
constexpr int RL_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[RL_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" long omni_rel_l1_noalloc_max_elems(void) { return RL_NOALLOC_MAX_ELEMS; }

extern "C" const char* omni_rel_l1_noalloc_strerror(int rc) {
  switch (rc) {
    case 0: return "ok";
    case RC_BAD_ARG: return "bad argument: n must be a positive multiple of 8, the pointers non-null, ncoef >= 0 and coef non-null when state and ncoef are given";
    case RC_TOO_LARGE: return "n exceeds omni_rel_l1_noalloc_max_elems() (2^28 elements per operand)";
    default: return rc > 0 ? "CUDA runtime error (the value is the cudaError_t)" : "unknown error";
  }
}

extern "C" int omni_rel_l1_noalloc(const void* a, const void* b, long n, float* sums_out, float* state,
                                   const float* coef, int ncoef, float thresh, int force_compute,
                                   void* stream) {
  if (a == nullptr || b == nullptr || n <= 0 || (n & 7)) return RC_BAD_ARG;
  if (sums_out == nullptr && state == nullptr) return RC_BAD_ARG;
  if (ncoef < 0 || (state != nullptr && ncoef > 0 && coef == nullptr)) return RC_BAD_ARG;
  if (n > RL_NOALLOC_MAX_ELEMS) return RC_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= RL_MAX_DEVICES) return RC_BAD_ARG;
  float* scratch = nullptr;
  {
    // First call on this device: resolve the device address of the static array.  The array's
    // name is only a host-side handle here; a kernel must be given the address the runtime
    // reports for the current device.
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_rel_l1_scratch);
      if (e != cudaSuccess) return (int)e;
      g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  const int parts = omni_rel_l1_parts(n);  // <= RL_NOALLOC_MAX_PARTS by construction
  // Stage 1 overwrites scratch[0 .. 2*parts) completely and stage 2 reads exactly that range,
  // so nothing left over from an earlier call is ever read and nothing needs clearing.
  rel_l1_partial_kernel<<<parts, RL_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, n >> 3, scratch);
  e = cudaGetLastError();                 // report a failed first launch, not only the second
  if (e != cudaSuccess) return (int)e;
  rel_l1_finish_kernel<<<1, RL_THREADS, 0, (cudaStream_t)stream>>>(scratch, parts, state, coef, ncoef, thresh,
                                                                   force_compute, sums_out);
  return (int)cudaGetLastError();
}
