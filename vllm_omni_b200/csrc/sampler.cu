// K16: token sampler.  One CTA per sequence over a vocabulary of up to ~1M entries, fp32 or
// bf16 logits, everything on the device (the reference masks talker tokens with a CPU round
// trip, vllm_omni/model_executor/models/qwen3_omni/qwen3_omni.py:1068-1104, and samples with
// vLLM's sampler).
//
// Per row, in order: suppressed-token mask (a list of ids), an allowed-range mask (tokens
// outside [lo, hi) are dropped unless listed in `keep`), repetition / presence / frequency
// penalties over the tokens generated so far, temperature, top-k, top-p, min-p, then a draw
// from the remaining distribution with a counter-based RNG (seed, step), or argmax when the
// temperature is 0.  top-k and top-p thresholds are found by bisection on the logit value, so
// no sort of the vocabulary is needed; each bisection step is one pass over the row.
#include "host_util.h"
#include "ptx_sm100.cuh"

namespace omni {

constexpr int SP_THREADS = 1024;

struct SampleRow {           // one per sequence
  float temperature, top_p, min_p;
  int top_k;
  float rep_penalty, presence_penalty, frequency_penalty;
  unsigned long long seed;   // per-request seed
  int step;                  // tokens generated so far (RNG counter)
  int hist_off, hist_len;    // slice of the history buffer (prompt + generated tokens)
  int gen_off;               // first generated token inside the slice (penalties that count only output)
  int sup_off, sup_len;      // slice of the suppressed-id buffer
  int range_lo, range_hi;    // allowed id range (hi <= 0: everything allowed)
};

__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = threadIdx.x < SP_THREADS / 32 ? sh[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    if (threadIdx.x == 0) sh[0] = r;
  }
  __syncthreads();
  r = sh[0];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = threadIdx.x < SP_THREADS / 32 ? sh[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (threadIdx.x == 0) sh[0] = r;
  }
  __syncthreads();
  r = sh[0];
  __syncthreads();
  return r;
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// work: float[V] per row (scaled logits after masks and penalties)
template <typename T>
__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const T* __restrict__ logits, long ld, int V, const SampleRow* __restrict__ rows,
              const int* __restrict__ history, const int* __restrict__ suppressed, float* __restrict__ work,
              int* __restrict__ cnt_work, int* __restrict__ out_ids, float* __restrict__ out_logprob) {
  __shared__ float sh[SP_THREADS / 32];
  __shared__ float s_scan[SP_THREADS];
  __shared__ int s_pick;
  const int r = blockIdx.x;
  const SampleRow p = rows[r];
  const T* lg = logits + (size_t)r * ld;
  float* w = work + (size_t)r * V;
  const bool greedy = p.temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / p.temperature;
  // 1. copy + range mask
  for (int i = threadIdx.x; i < V; i += SP_THREADS) {
    float x = (float)lg[i];
    if (p.range_hi > 0 && (i < p.range_lo || i >= p.range_hi)) x = -INFINITY;
    w[i] = x;
  }
  __syncthreads();
  // 2. suppressed ids
  for (int i = threadIdx.x; i < p.sup_len; i += SP_THREADS) {
    const int id = suppressed[p.sup_off + i];
    if (id >= 0 && id < V) w[id] = -INFINITY;
  }
  __syncthreads();
  // 3. penalties: count occurrences per token id in an int[V] scratch row (low 16 bits: all
  //    occurrences, high bits: occurrences among the generated tokens), then one pass over V.
  if (cnt_work && (p.rep_penalty != 1.f || p.presence_penalty != 0.f || p.frequency_penalty != 0.f)) {
    int* cnt = cnt_work + (size_t)r * V;
    for (int i = threadIdx.x; i < V; i += SP_THREADS) cnt[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < p.hist_len; i += SP_THREADS) {
      const int id = history[p.hist_off + i];
      if (id >= 0 && id < V) atomicAdd(&cnt[id], 1 + (i >= p.gen_off ? (1 << 16) : 0));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += SP_THREADS) {
      const int c = cnt[i];
      if (c == 0) continue;
      float x = w[i];
      if (p.rep_penalty != 1.f) x = x > 0.f ? x / p.rep_penalty : x * p.rep_penalty;
      const int c_out = c >> 16;
      if (c_out > 0) x -= p.presence_penalty + p.frequency_penalty * (float)c_out;
      w[i] = x;
    }
    __syncthreads();
  }
  // 4. temperature + max
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += SP_THREADS) {
    const float x = w[i] * inv_t;
    w[i] = x;
    mx = fmaxf(mx, x);
  }
  mx = block_reduce_max(mx, sh);
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += SP_THREADS) sum += __expf(w[i] - mx);
  sum = block_reduce_sum(sum, sh);
  const float log_z = mx + __logf(sum);
  if (greedy) {
    // argmax, lowest id wins ties
    int best = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SP_THREADS)
      if (w[i] == mx && i < best) best = i;
    __shared__ int s_best;
    if (threadIdx.x == 0) s_best = 0x7fffffff;
    __syncthreads();
    atomicMin(&s_best, best);
    __syncthreads();
    if (threadIdx.x == 0) {
      out_ids[r] = s_best;
      if (out_logprob) out_logprob[r] = mx - log_z;
    }
    return;
  }
  // 5. threshold: the largest cut (in logit units) allowed by top-k, top-p and min-p
  float cut = -INFINITY;
  if (p.min_p > 0.f) cut = fmaxf(cut, mx + __logf(p.min_p));
  if (p.top_k > 0 && p.top_k < V) {
    float lo = mx - 60.f, hi = mx;   // invariant: count(w >= lo) >= k (or everything), count(w > hi) < k
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += SP_THREADS) c += w[i] >= mid ? 1.f : 0.f;
      c = block_reduce_sum(c, sh);
      if (c >= (float)p.top_k) lo = mid; else hi = mid;
    }
    cut = fmaxf(cut, lo);
  }
  if (p.top_p < 1.f) {
    // top-p is measured on the distribution that survived min-p and top-k (vLLM applies top-k first
    // and top-p on the renormalised survivors), not on the full one
    float surv = sum;
    if (cut > -INFINITY) {
      surv = 0.f;
      for (int i = threadIdx.x; i < V; i += SP_THREADS) surv += w[i] >= cut ? __expf(w[i] - mx) : 0.f;
      surv = block_reduce_sum(surv, sh);
    }
    float lo = mx - 60.f, hi = mx;   // mass(w >= lo) >= top_p * surviving mass
    for (int it = 0; it < 26; ++it) {
      const float mid = 0.5f * (lo + hi);
      float c = 0.f;
      for (int i = threadIdx.x; i < V; i += SP_THREADS) c += (w[i] >= mid && w[i] >= cut) ? __expf(w[i] - mx) : 0.f;
      c = block_reduce_sum(c, sh);
      if (c >= p.top_p * surv) lo = mid; else hi = mid;
    }
    cut = fmaxf(cut, lo);
  }
  // 6. draw: contiguous chunk per thread so the scan order is the vocabulary order
  const int per = (V + SP_THREADS - 1) / SP_THREADS;
  const int b0 = threadIdx.x * per, b1 = min(V, b0 + per);
  float mass = 0.f;
  for (int i = b0; i < b1; ++i) mass += w[i] >= cut ? __expf(w[i] - mx) : 0.f;
  s_scan[threadIdx.x] = mass;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < SP_THREADS; ++i) total += s_scan[i];
    const unsigned long long h = splitmix64(p.seed ^ splitmix64((unsigned long long)p.step));
    const float u = ((h >> 40) + 0.5f) * (1.0f / 16777216.0f) * total;
    float acc = 0.f;
    int pick = SP_THREADS - 1;
    for (int i = 0; i < SP_THREADS; ++i) {
      if (acc + s_scan[i] > u && s_scan[i] > 0.f) { pick = i; break; }
      acc += s_scan[i];
    }
    s_pick = pick;
    sh[0] = u - acc;   // remaining mass to walk inside the chunk
  }
  __syncthreads();
  if (threadIdx.x == s_pick) {
    float rem = sh[0];
    int tok = -1, last_ok = -1;
    for (int i = b0; i < b1; ++i) {
      if (w[i] >= cut) {
        last_ok = i;
        const float e = __expf(w[i] - mx);
        if (rem < e) { tok = i; break; }
        rem -= e;
      }
    }
    if (tok < 0) tok = last_ok >= 0 ? last_ok : 0;
    out_ids[r] = tok;
    if (out_logprob) out_logprob[r] = w[tok] - log_z;
  }
}

}  // namespace omni

using namespace omni;

// rows: device array of SampleRow (56 bytes each, see ops/sampler.py for the packing).
extern "C" int omni_sample(const void* logits, int is_bf16, long ld, int V, int num_rows, const void* rows,
                           const int* history, const int* suppressed, float* work, int* cnt_work,
                           int* out_ids, float* out_logprob, void* stream) {
  if (num_rows <= 0) return RC_OK;
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<num_rows, SP_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)logits, ld, V, (const SampleRow*)rows, history, suppressed, work, cnt_work, out_ids, out_logprob);
  else
    sample_kernel<float><<<num_rows, SP_THREADS, 0, (cudaStream_t)stream>>>(
        (const float*)logits, ld, V, (const SampleRow*)rows, history, suppressed, work, cnt_work, out_ids, out_logprob);
  return (int)cudaGetLastError();
}

extern "C" int omni_sample_row_bytes(void) { return (int)sizeof(SampleRow); }
