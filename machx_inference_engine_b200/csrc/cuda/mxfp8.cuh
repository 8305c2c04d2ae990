// MXFP8 (e4m3 elements, one e8m0 scale per 32) rounding helpers and the scale-factor atom layout shared by the block-scaled expert
// GEMM, its quantisers and the decode kernels that produce its input.
#pragma once
#include "common.cuh"
#include <cuda_fp8.h>

namespace mx {

constexpr int SF_ATOM = 512;     // bytes of one scale-factor atom: 128 rows x 4 k-blocks
constexpr int MXF_KBLOCK = 128;  // elements of K per scale-factor atom column group (= one pipeline stage of the expert GEMM)

// scale-factor atom: row r (0..127), k-block q (0..3) -> byte (r % 32) * 16 + (r / 32) * 4 + q
__host__ __device__ constexpr int sf_atom_offset(int r, int q) { return (r & 31) * 16 + (r >> 5) * 4 + q; }

// e8m0 scale of a 32-element block with maximum magnitude amax: the smallest power of two that keeps the block inside e4m3's
// range (448).  Returns the biased exponent byte; *inv = 1 / scale.
__device__ __forceinline__ uint32_t mxfp8_scale(float amax, float* inv) {
  if (!(amax > 0.f)) { *inv = 1.f; return 127u; }
  int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 8;           // floor(log2 amax) - 8, biased
  ex = max(1, min(ex, 253));
  if (amax * __uint_as_float((uint32_t)(254 - ex) << 23) > 448.f) ex = min(ex + 1, 253);
  *inv = __uint_as_float((uint32_t)(254 - ex) << 23);
  return (uint32_t)ex;
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

}  // namespace mx
