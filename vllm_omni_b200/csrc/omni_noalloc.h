/* Allocation-free entry point of the TeaCache rel-L1 reduction.
 *
 * This entry point has no counterpart in the reference project; it exists for callers of
 * this library that are not able to allocate device memory at the point where they need
 * the metric.  Examples: a serving loop that has handed every spare byte of HBM to weights
 * and KV pages and runs with a sealed memory budget; a C or C++ host that links this library
 * without PyTorch and therefore has no caching allocator to ask; a latency-critical step
 * where a cudaMalloc/cudaFree pair would stall the device.
 *
 * What it computes is exactly what omni_rel_l1() computes:
 *   sums_out[0] = sum |a - b|,  sums_out[1] = sum |b|      (fp32, over n bf16 elements)
 * and, if `state` is given, the TeaCache bookkeeping in state[0..3] (accumulated rescaled
 * distance, last relative L1, skip flag, number of skipped steps) using the polynomial
 * `coef` (highest power first, `ncoef` entries, may be 0) and the threshold `thresh`.
 *
 * Memory: inputs (a, b, coef) and outputs (sums_out, state) are device pointers owned by the
 * caller.  The per-block partial sums live in a static device array inside the library:
 * 2 * 592 floats = 4,736 bytes.  Every GPU that loads the library holds that array until the
 * process exits.  The call makes no cudaMalloc, cudaFree or other allocating call.
 *
 * Limits: n must be a positive multiple of 8 and at most omni_rel_l1_noalloc_max_elems()
 * (2^28 = 268,435,456 elements per operand); a larger n is refused with a negative return
 * code (see omni_rel_l1_noalloc_strerror) and nothing is launched.
 *
 * First call on a device: the library looks up the device address of its static array with
 * cudaGetSymbolAddress while that device is current, and remembers it.  Make that first call
 * (per device) during set-up, before any stream capture is started.
 *
 * Sharing: all calls on one device use the same array.  The kernels overwrite the part of
 * it they read, so no clearing is needed between calls, but two calls that run on the GPU
 * at the same time (different streams, or different host threads on different streams)
 * would overwrite each other's partial sums: serialise them on one stream.
 *
 * Returns 0 on success, a negative library code for refused arguments, or a positive
 * cudaError_t value from the launch.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int omni_rel_l1_noalloc(const void* a, const void* b, long n, float* sums_out, float* state,
                        const float* coef, int ncoef, float thresh, int force_compute, void* stream);
long omni_rel_l1_noalloc_max_elems(void);
const char* omni_rel_l1_noalloc_strerror(int rc);

#ifdef __cplusplus
}
#endif
