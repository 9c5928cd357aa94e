// Host-side helpers shared by the kernel launchers: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda), device properties, and the
// C ABI error convention (0 = ok, negative = launcher rejected the arguments, positive =
// CUDA runtime error code).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace omni {

constexpr int RC_OK = 0;
constexpr int RC_BAD_ARG = -1;
constexpr int RC_NO_DRIVER = -2;
constexpr int RC_TMAP = -3;
constexpr int RC_TOO_LARGE = -4;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// Row-major 2-D tensor [rows, cols] of `elt_bytes` elements with a row pitch of
// `pitch_bytes`; box = {box_cols, box_rows}; 128-byte swizzle (box_cols * elt_bytes must
// be 128).  Out-of-range elements read as zero.
inline int make_tmap_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, int elt_bytes,
                        uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows,
                        uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return RC_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (pitch_bytes & 15)) return RC_BAD_ARG;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elt_bytes;
  return r == CUDA_SUCCESS ? RC_OK : RC_TMAP;
}

// 3-D tensor [d2, d1, d0] (d0 innermost, contiguous) with byte pitches p1 (between d1
// indices) and p2 (between d2 indices); box = {b0, b1, 1}.
inline int make_tmap_3d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t d0,
                        uint64_t d1, uint64_t d2, uint64_t p1, uint64_t p2, uint32_t b0,
                        uint32_t b1) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return RC_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (p1 & 15) || (p2 & 15)) return RC_BAD_ARG;
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstr[2] = {p1, p2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dt, 3, const_cast<void*>(ptr), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RC_OK : RC_TMAP;
}

// cudaFuncSetAttribute applies to the CURRENT device only, and one process may launch on several
// (stages of a pipeline running as threads, each on its own GPU).  `mask` remembers, one bit per
// device index, where the kernel has been prepared; returns 0 or the CUDA error.
inline int ensure_dynamic_smem(const void* fn, int bytes, unsigned long long& mask) {
  int dev = 0;
  cudaGetDevice(&dev);
  const unsigned long long bit = 1ull << (dev & 63);
  if (mask & bit) return 0;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  mask |= bit;
  return 0;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace omni
