// K12 (element-wise part): the VAE decoder's non-convolution kernels on channels-last (NHWC) bf16
// activations.  The convolutions themselves run as implicit GEMMs on the tcgen05 kernel
// (gemm_sm100.cu, omni_conv2d_nhwc_bf16).
//
//   omni_rmsnorm_silu_nhwc   y = silu( x / sqrt(mean_c x^2) * gamma )      per pixel, fused
//   omni_upsample2x_nhwc     nearest-neighbour 2x up-sampling
//   omni_nchw_to_nhwc        fp32/bf16 [N,C,H,W] -> bf16 [N,H,W,Cpad] (zero padded channels)
//   omni_nhwc_to_image       bf16 [N,H,W,ld] -> uint8 [N,H,W,3] ((x * 0.5 + 0.5) clamped, * 255, rounded)
//                            or fp32 [N,3,H,W] in [-1, 1]
//
// The reference decodes through diffusers' AutoencoderKL* modules, i.e. cuDNN convolutions with
// separate eager norm / activation / interpolate / permute / clamp kernels
// (vllm_omni/diffusion/models/qwen_image/autoencoder_kl_qwenimage.py).
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

// one warp per pixel; C % 8 == 0, C <= 1024
__global__ void __launch_bounds__(256)
rmsnorm_silu_nhwc_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const __nv_bfloat16* __restrict__ gamma,
                         __nv_bfloat16* __restrict__ y, long ldy, long pixels, int C, int apply_silu) {
  const long p = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (p >= pixels) return;
  const int chunks = C >> 3;
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = lane + i * 32;
    if (c < chunks) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + p * ldx + c * 8);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = b.x; v[i][3] = b.y; v[i][4] = cc.x; v[i][5] = cc.y; v[i][6] = d.x; v[i][7] = d.y;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(fmaxf(ss / (float)C, 1e-24f));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = lane + i * 32;
    if (c < chunks) {
      const uint4 g = *reinterpret_cast<const uint4*>(gamma + c * 8);
      const float2 a = unpack_bf16(g.x), b = unpack_bf16(g.y), cc = unpack_bf16(g.z), d = unpack_bf16(g.w);
      const float gm[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float t = v[i][e] * inv * gm[e];
        o[e] = apply_silu ? silu(t) : t;
      }
      uint4 w;
      w.x = pack_bf16(o[0], o[1]); w.y = pack_bf16(o[2], o[3]); w.z = pack_bf16(o[4], o[5]); w.w = pack_bf16(o[6], o[7]);
      *reinterpret_cast<uint4*>(y + p * ldy + c * 8) = w;
    }
  }
}

__global__ void __launch_bounds__(256)
upsample2x_nhwc_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int N, int H, int W, int C) {
  const int chunks = C >> 3;
  const long total = (long)N * (2 * H) * (2 * W) * chunks;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    long p = i / chunks;
    const int ox = (int)(p % (2 * W)); p /= 2 * W;
    const int oy = (int)(p % (2 * H));
    const int n = (int)(p / (2 * H));
    const size_t src = (((size_t)n * H + (oy >> 1)) * W + (ox >> 1)) * C + c * 8;
    *reinterpret_cast<uint4*>(y + (i / chunks) * C + c * 8) = *reinterpret_cast<const uint4*>(x + src);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
nchw_to_nhwc_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ y, int N, int C, int H, int W, int Cpad) {
  const long total = (long)N * H * W * Cpad;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % Cpad);
    const long p = i / Cpad;                 // n * H * W + h * W + w
    const long hw = p % ((long)H * W);
    const long n = p / ((long)H * W);
    y[i] = c < C ? __float2bfloat16((float)x[(n * C + c) * (long)H * W + hw]) : __float2bfloat16(0.f);
  }
}

// mode 0: uint8 [N,H,W,3]; mode 1: fp32 [N,3,H,W] clamped to [-1, 1]
__global__ void __launch_bounds__(256)
nhwc_to_image_kernel(const __nv_bfloat16* __restrict__ x, long ldx, void* __restrict__ out, long pixels, long HW, int mode) {
  for (long p = (long)blockIdx.x * blockDim.x + threadIdx.x; p < pixels; p += (long)gridDim.x * blockDim.x) {
    float v[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) v[c] = fminf(fmaxf(__bfloat162float(x[p * ldx + c]), -1.f), 1.f);
    if (mode == 0) {
      uint8_t* o = static_cast<uint8_t*>(out) + p * 3;
#pragma unroll
      for (int c = 0; c < 3; ++c) o[c] = (uint8_t)__float2int_rn((v[c] * 0.5f + 0.5f) * 255.f);
    } else {
      float* o = static_cast<float*>(out);
      const long n = p / HW, hw = p % HW;
#pragma unroll
      for (int c = 0; c < 3; ++c) o[(n * 3 + c) * HW + hw] = v[c];
    }
  }
}

static unsigned grid_for(long total) {
  long b = (total + 255) / 256;
  if (b > 148L * 16) b = 148L * 16;
  return (unsigned)(b < 1 ? 1 : b);
}

// Snake activation of the vocoders, channels-last: y = x + inv_b[c] * sin^2(x * a[c]) with per-channel
// a = exp(alpha) and inv_b = 1 / (exp(beta) + 1e-9) computed by the caller (fp32, [C]).  One thread per
// 8 channels (16-byte load and store); C is a multiple of 8, rows have pitch ldx / ldy elements.
__global__ void __launch_bounds__(256)
snake_nlc_kernel(const __nv_bfloat16* __restrict__ x, long ldx, const float* __restrict__ a, const float* __restrict__ inv_b,
                 __nv_bfloat16* __restrict__ y, long ldy, long rows, int C8) {
  const long total = rows * C8;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / C8;
    const int c = (int)(i - r * C8) * 8;
    const uint4 v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      const float s0 = sinf(f.x * a[c + 2 * j]), s1 = sinf(f.y * a[c + 2 * j + 1]);
      q[j] = __floats2bfloat162_rn(fmaf(inv_b[c + 2 * j] * s0, s0, f.x), fmaf(inv_b[c + 2 * j + 1] * s1, s1, f.y));
    }
    *reinterpret_cast<uint4*>(y + r * ldy + c) = o;
  }
}

// Depthwise convolution over time, channels-last (the ConvNeXt blocks of the vocoders):
// y[b, t, c] = bias[c] + sum_j x[b, t + j * dil - pad, c] * w[j, c]; one thread per 8 channels of one step.
__global__ void __launch_bounds__(256)
dwconv1d_nlc_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                    __nv_bfloat16* __restrict__ y, int B, int T, int C8, int k, int dil, int pad) {
  const long total = (long)B * T * C8;
  const int C = C8 * 8;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8) * 8;
    const long bt = i / C8;
    const int t = (int)(bt % T);
    const long b = bt / T;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < k; ++j) {
      const int ti = t + j * dil - pad;
      if (ti < 0 || ti >= T) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(x + ((b * T + ti) * (long)C + c));
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float* wj = w + (long)j * C + c;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        acc[2 * e] = fmaf(f.x, wj[2 * e], acc[2 * e]);
        acc[2 * e + 1] = fmaf(f.y, wj[2 * e + 1], acc[2 * e + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) q[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(y + ((b * T + t) * (long)C + c)) = o;
  }
}

// Anti-aliased snake activation of BigVGAN, channels-last: 2x up-sampling by a 12-tap windowed-sinc
// filter (replicate padding), snake, 2x down-sampling by a 12-tap filter (replicate padding), in one pass:
//   u[s]   = 2 * sum_j x[clamp((s + 15 - j) / 2 - 5)] * fu[j]        over the j with (s + 15 - j) even, s in [0, 2T)
//   a[s]   = u[s] + inv_b[c] * sin^2(u[s] * alpha[c])
//   out[t] = sum_j a[clamp(2t + j - 5, 0, 2T - 1)] * fd[j]
// (the index arithmetic of conv_transpose1d(stride 2) on the input padded by 5, cropped by 15 on both sides,
// then conv1d(stride 2) on the result padded by (5, 6)).  One thread owns 8 channels of AA_RUN consecutive
// output steps, so that the up-sampled values are computed once per two outputs, not once per tap.
constexpr int AA_K = 12, AA_RUN = 4;
__global__ void __launch_bounds__(128)
aa_snake_nlc_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ alpha, const float* __restrict__ inv_b,
                    const float* __restrict__ fu, const float* __restrict__ fd, __nv_bfloat16* __restrict__ y, int B, int T,
                    int C8) {
  __shared__ float s_fu[AA_K], s_fd[AA_K];
  if (threadIdx.x < AA_K) { s_fu[threadIdx.x] = fu[threadIdx.x]; s_fd[threadIdx.x] = fd[threadIdx.x]; }
  __syncthreads();
  const int runs = (T + AA_RUN - 1) / AA_RUN;
  const long total = (long)B * runs * C8;
  const int C = C8 * 8;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8) * 8;
    const long br = i / C8;
    const int t0 = (int)(br % runs) * AA_RUN;
    const long b = br / runs;
    const __nv_bfloat16* xb = x + b * (long)T * C + c;
    float al[8], ib[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { al[e] = alpha[c + e]; ib[e] = inv_b[c + e]; }
    // up-sampled, activated values a[s] for s in [2 t0 - 5, 2 (t0 + AA_RUN - 1) + 6], clamped to [0, 2T - 1]
    constexpr int NS = 2 * AA_RUN + 10;
    float a[NS][8];
    int prev_s = -1;
#pragma unroll
    for (int k = 0; k < NS; ++k) {
      int s = 2 * t0 - 5 + k;
      s = s < 0 ? 0 : (s > 2 * T - 1 ? 2 * T - 1 : s);
      if (s == prev_s) {                              // clamped repeats at the ends of the signal
#pragma unroll
        for (int e = 0; e < 8; ++e) a[k][e] = a[k > 0 ? k - 1 : 0][e];
        continue;
      }
      prev_s = s;
      float u[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) u[e] = 0.f;
      const int sp = s + 15;
      for (int j = sp & 1; j < AA_K; j += 2) {        // taps with (sp - j) even
        int xi = (sp - j) / 2 - 5;
        xi = xi < 0 ? 0 : (xi > T - 1 ? T - 1 : xi);
        const uint4 v = *reinterpret_cast<const uint4*>(xb + (long)xi * C);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float w = 2.0f * s_fu[j];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(p[e]);
          u[2 * e] = fmaf(f.x, w, u[2 * e]);
          u[2 * e + 1] = fmaf(f.y, w, u[2 * e + 1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float sn = sinf(u[e] * al[e]);
        a[k][e] = fmaf(ib[e] * sn, sn, u[e]);
      }
    }
#pragma unroll
    for (int r = 0; r < AA_RUN; ++r) {
      const int t = t0 + r;
      if (t >= T) break;
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = 0.f;
#pragma unroll
      for (int j = 0; j < AA_K; ++j) {
        const float w = s_fd[j];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(a[2 * r + j][e], w, o[e]);
      }
      uint4 ov;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) q[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
      *reinterpret_cast<uint4*>(y + (b * (long)T + t) * C + c) = ov;
    }
  }
}

}  // namespace omni

using namespace omni;

extern "C" int omni_rmsnorm_silu_nhwc(const void* x, long ldx, const void* gamma, void* y, long ldy, long pixels, int C,
                                      int apply_silu, void* stream) {
  if (pixels <= 0) return RC_OK;
  if ((C & 7) || C > 1024 || (ldx & 7) || (ldy & 7)) return RC_BAD_ARG;
  rmsnorm_silu_nhwc_kernel<<<(unsigned)((pixels + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)y, ldy, pixels, C, apply_silu);
  return (int)cudaGetLastError();
}

extern "C" int omni_upsample2x_nhwc(const void* x, void* y, int N, int H, int W, int C, void* stream) {
  if (N <= 0 || H <= 0 || W <= 0) return RC_OK;
  if (C & 7) return RC_BAD_ARG;
  upsample2x_nhwc_kernel<<<grid_for((long)N * 4 * H * W * (C >> 3)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, H, W, C);
  return (int)cudaGetLastError();
}

extern "C" int omni_nchw_to_nhwc(const void* x, int is_fp32, void* y, int N, int C, int H, int W, int Cpad, void* stream) {
  if (N <= 0) return RC_OK;
  if (Cpad < C) return RC_BAD_ARG;
  const unsigned g = grid_for((long)N * H * W * Cpad);
  if (is_fp32)
    nchw_to_nhwc_kernel<float><<<g, 256, 0, (cudaStream_t)stream>>>((const float*)x, (__nv_bfloat16*)y, N, C, H, W, Cpad);
  else
    nchw_to_nhwc_kernel<__nv_bfloat16><<<g, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, C, H, W, Cpad);
  return (int)cudaGetLastError();
}

extern "C" int omni_nhwc_to_image(const void* x, long ldx, void* out, int N, int H, int W, int mode, void* stream) {
  if (N <= 0) return RC_OK;
  if (ldx < 3 || (mode != 0 && mode != 1)) return RC_BAD_ARG;
  const long pixels = (long)N * H * W;
  nhwc_to_image_kernel<<<grid_for(pixels), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, out, pixels,
                                                                         (long)H * W, mode);
  return (int)cudaGetLastError();
}

extern "C" int omni_snake_nlc(const void* x, long ldx, const float* a, const float* inv_b, void* y, long ldy, long rows, int C,
                              void* stream) {
  if (rows <= 0 || C <= 0) return omni::RC_OK;
  if ((C & 7) || (ldx & 7) || (ldy & 7)) return omni::RC_BAD_ARG;
  const long total = rows * (C / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  omni::snake_nlc_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, a, inv_b, (__nv_bfloat16*)y, ldy, rows, C / 8);
  return (int)cudaGetLastError();
}

// x, y: contiguous [B, T, C] bf16, C a multiple of 8; w: fp32 [k, C]; bias: fp32 [C] or null.
extern "C" int omni_dwconv1d_nlc(const void* x, const float* w, const float* bias, void* y, int B, int T, int C, int k,
                                 int dil, int pad, void* stream) {
  if (B <= 0 || T <= 0 || C <= 0) return omni::RC_OK;
  if ((C & 7) || k < 1 || dil < 1) return omni::RC_BAD_ARG;
  const long total = (long)B * T * (C / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  omni::dwconv1d_nlc_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, w, bias, (__nv_bfloat16*)y, B, T, C / 8, k, dil, pad);
  return (int)cudaGetLastError();
}

// x, y: contiguous [B, T, C] bf16, C a multiple of 8; alpha, inv_b: fp32 [C]; fu, fd: fp32 [12] (up / down filters).
extern "C" int omni_aa_snake_nlc(const void* x, const float* alpha, const float* inv_b, const float* fu, const float* fd, void* y,
                                 int B, int T, int C, void* stream) {
  if (B <= 0 || T <= 0 || C <= 0) return omni::RC_OK;
  if (C & 7) return omni::RC_BAD_ARG;
  const long total = (long)B * ((T + omni::AA_RUN - 1) / omni::AA_RUN) * (C / 8);
  long blocks = (total + 127) / 128;
  if (blocks > 148 * 32) blocks = 148 * 32;
  omni::aa_snake_nlc_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, alpha, inv_b, fu, fd, (__nv_bfloat16*)y, B, T, C / 8);
  return (int)cudaGetLastError();
}

namespace omni {

// Row softmax in place over bf16 scores: x[r, :] = softmax(scale * x[r, :]).  One CTA per row; the row
// is read twice (running maximum and sum in one pass, then the normalised write), the second time
// from L2.  N % 8 == 0, ld % 8 == 0.  Used by the VAE's single-head attention, whose head width (the
// channel count) is outside the flash kernel's head sizes: scores and P*V run as tcgen05 GEMMs.
__global__ void __launch_bounds__(256)
softmax_rows_kernel(__nv_bfloat16* __restrict__ x, long ld, int nvec, float scale_log2e) {
  __nv_bfloat16* row = x + (long)blockIdx.x * ld;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    const uint4 u = reinterpret_cast<const uint4*>(row)[i];
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    const float f[8] = {a.x * scale_log2e, a.y * scale_log2e, b.x * scale_log2e, b.y * scale_log2e,
                        c.x * scale_log2e, c.y * scale_log2e, d.x * scale_log2e, d.y * scale_log2e};
    float lm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) lm = fmaxf(lm, f[e]);
    if (lm > m) {
      s *= exp2f(m - lm);
      m = lm;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s += exp2f(f[e] - m);
  }
  // combine (m, s) over the warp, then over the 8 warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * exp2f(m - nm) + os * exp2f(om - nm);
    m = nm;
  }
  __shared__ float sm[8], ss[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  float M = sm[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) M = fmaxf(M, sm[w]);
  float S = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) S += (sm[w] == -INFINITY) ? 0.f : ss[w] * exp2f(sm[w] - M);
  const float inv = S > 0.f ? 1.f / S : 0.f;
  for (int i = threadIdx.x; i < nvec; i += 256) {
    uint4 u = reinterpret_cast<const uint4*>(row)[i];
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    u.x = pack_bf16(exp2f(a.x * scale_log2e - M) * inv, exp2f(a.y * scale_log2e - M) * inv);
    u.y = pack_bf16(exp2f(b.x * scale_log2e - M) * inv, exp2f(b.y * scale_log2e - M) * inv);
    u.z = pack_bf16(exp2f(c.x * scale_log2e - M) * inv, exp2f(c.y * scale_log2e - M) * inv);
    u.w = pack_bf16(exp2f(d.x * scale_log2e - M) * inv, exp2f(d.y * scale_log2e - M) * inv);
    reinterpret_cast<uint4*>(row)[i] = u;
  }
}

}  // namespace omni

// x: bf16 [rows, N] with row pitch ld (elements), rewritten in place.
extern "C" int omni_softmax_rows(void* x, long ld, long rows, int N, float scale, void* stream) {
  if (rows <= 0 || N <= 0) return omni::RC_OK;
  if ((N & 7) || (ld & 7) || ld < N || rows > 0x7fffffffL) return omni::RC_BAD_ARG;
  omni::softmax_rows_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, ld, N / 8,
                                                                             scale * 1.4426950408889634f);
  return (int)cudaGetLastError();
}

namespace omni {

// GroupNorm (+ SiLU) on channels-last activations, x: [N, P, C] bf16 (row pitch ld), G groups of C / G channels.
// Two kernels.  gn_stats: grid (GN_SPLITS, N); a CTA takes every GN_SPLITS-th run of pixels, each thread keeps the sums of
// ONE 8-channel vector position, the per-thread sums are combined per group in a fixed order, and the CTA writes
// (sum, sum of squares) per group to partial[n][g][split].  gn_apply: sums the GN_SPLITS partials of each group in
// order (so the result does not depend on scheduling), then normalises, scales, shifts and applies SiLU.
// Requirements: C % 8 == 0 and (C / 8) divides 256, so that a thread's vector position is the same for all its pixels.
constexpr int GN_SPLITS = 128;
constexpr int GN_MAX_GROUPS = 64;

__global__ void __launch_bounds__(256)
gn_stats_kernel(const __nv_bfloat16* __restrict__ x, long ld, long P, int C, int G, float* __restrict__ partial) {
  __shared__ float s_sum[256][8];
  __shared__ float s_sq[256][8];
  const int vecs = C >> 3;                      // vector positions per pixel
  const int ppb = 256 / vecs;                   // pixels per CTA pass
  const int v = threadIdx.x % vecs;
  const int po = threadIdx.x / vecs;
  const int n = blockIdx.y;
  const __nv_bfloat16* xs = x + (long)n * P * ld;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, q[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long p = (long)blockIdx.x * ppb + po; p < P; p += (long)GN_SPLITS * ppb) {
    const uint4 u = *reinterpret_cast<const uint4*>(xs + p * ld + v * 8);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      s[e] += f[e];
      q[e] += f[e] * f[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    s_sum[threadIdx.x][e] = s[e];
    s_sq[threadIdx.x][e] = q[e];
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    const int cpg = C / G;
    float ts = 0.f, tq = 0.f;
    for (int c = g * cpg; c < (g + 1) * cpg; ++c) {          // channels of the group, then the pixel lanes, in order
      const int vv = c >> 3, e = c & 7;
      for (int lane = 0; lane < ppb; ++lane) {
        ts += s_sum[lane * vecs + vv][e];
        tq += s_sq[lane * vecs + vv][e];
      }
    }
    float* out = partial + (((long)n * G + g) * GN_SPLITS + blockIdx.x) * 2;
    out[0] = ts;
    out[1] = tq;
  }
}

__global__ void __launch_bounds__(256)
gn_apply_kernel(const __nv_bfloat16* __restrict__ x, long ldx, __nv_bfloat16* __restrict__ y, long ldy, long P, int C, int G,
                const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ partial,
                float eps, int apply_silu) {
  __shared__ float s_mean[GN_MAX_GROUPS], s_rstd[GN_MAX_GROUPS];
  const int n = blockIdx.y;
  if (threadIdx.x < G) {
    const float* pp = partial + ((long)n * G + threadIdx.x) * GN_SPLITS * 2;
    float ts = 0.f, tq = 0.f;
    for (int i = 0; i < GN_SPLITS; ++i) {
      ts += pp[2 * i];
      tq += pp[2 * i + 1];
    }
    const float cnt = (float)P * (float)(C / G);
    const float mean = ts / cnt;
    const float var = fmaxf(tq / cnt - mean * mean, 0.f);
    s_mean[threadIdx.x] = mean;
    s_rstd[threadIdx.x] = rsqrtf(var + eps);
  }
  __syncthreads();
  const int vecs = C >> 3;
  const int cpg = C / G;
  const long total = P * vecs;
  const __nv_bfloat16* xs = x + (long)n * P * ldx;
  __nv_bfloat16* ys = y + (long)n * P * ldy;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long p = i / vecs;
    const int c0 = (int)(i % vecs) * 8;
    const uint4 u = *reinterpret_cast<const uint4*>(xs + p * ldx + c0);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int ch = c0 + e;
      const int g = ch / cpg;
      float vnorm = (f[e] - s_mean[g]) * s_rstd[g] * gamma[ch] + beta[ch];
      if (apply_silu) vnorm = vnorm / (1.f + __expf(-vnorm));
      f[e] = vnorm;
    }
    uint4 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]);
    o.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(ys + p * ldy + c0) = o;
  }
}

}  // namespace omni

// x, y: bf16 [N, P, C] with row pitches ldx / ldy (elements); gamma, beta: fp32 [C]; partial: fp32 scratch of
// N * G * 128 * 2 floats (every element is written before it is read).
extern "C" int omni_groupnorm_nhwc(const void* x, long ldx, void* y, long ldy, int N, long P, int C, int G, const float* gamma,
                                   const float* beta, float eps, int apply_silu, float* partial, void* stream) {
  if (N <= 0 || P <= 0) return omni::RC_OK;
  if (C <= 0 || (C & 7) || G <= 0 || G > omni::GN_MAX_GROUPS || (C % G) || (256 % (C >> 3)) || (C >> 3) > 256 || (ldx & 7) ||
      (ldy & 7) || partial == nullptr)
    return omni::RC_BAD_ARG;
  omni::gn_stats_kernel<<<dim3(omni::GN_SPLITS, N), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, P, C, G, partial);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  long blocks = (P * (C >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  omni::gn_apply_kernel<<<dim3((unsigned)blocks, N), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, (__nv_bfloat16*)y, ldy, P, C, G, gamma, beta, partial, eps, apply_silu);
  return (int)cudaGetLastError();
}
