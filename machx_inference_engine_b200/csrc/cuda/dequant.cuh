// In-register decoders for the runtime weight layouts (see WFormat in common.cuh).
//
// Two families:
//   * decode32_f32<FMT>  : 32 consecutive k-elements of one weight row -> 32 floats (GEMV path)
//   * decode32_bf16<FMT> : the same 32 elements -> 16 packed bf16x2 words (GEMM producer path)
// `kb` is the index of the 32-element block along K.  Rows are addressed by the caller through
// RowPtrs, which holds the per-row base pointers of every plane.
//
// Reference parity: these replace the whole-matrix dequant kernels of src/ops/dequant_kernels.cpp
// and the per-format inner loops of src/ops/gemv_q4k.cpp, gemv_q6k.cpp, gemv_q8dot.cpp,
// gemv_mxfp4.cpp; the weights are never materialised in fp16.
#pragma once
#include "common.cuh"

namespace mx {

struct RowPtrs {
  const uint8_t* p0;
  const uint8_t* p1;
  const uint8_t* p2;
  const uint8_t* p3;
};

// Per-row plane strides in bytes for a [N][K] matrix.
template <int FMT>
__device__ __forceinline__ RowPtrs row_ptrs(const WeightRef& w, long long row, int K) {
  RowPtrs r;
  const uint8_t* b0 = (const uint8_t*)w.p0;
  const uint8_t* b1 = (const uint8_t*)w.p1;
  const uint8_t* b2 = (const uint8_t*)w.p2;
  const uint8_t* b3 = (const uint8_t*)w.p3;
  if (FMT == WF_BF16) { r.p0 = b0 + row * K * 2; r.p1 = r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q8) { r.p0 = b0 + row * K; r.p1 = b1 + row * (K / 32) * 2; r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q4K) { r.p0 = b0 + row * (K / 256) * 144; r.p1 = r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q6K) { r.p0 = b0 + row * (K / 2); r.p1 = b1 + row * (K / 4); r.p2 = b2 + row * (K / 16); r.p3 = b3 + row * (K / 256) * 2; }
  else { r.p0 = b0 + row * (K / 2); r.p1 = b1 + row * (K / 32); r.p2 = r.p3 = nullptr; }
  return r;
}

// Byte offset between consecutive experts for each plane of a stacked [E][N][K] weight.
template <int FMT>
__device__ __forceinline__ WeightRef expert_weight(const WeightRef& w, long long e, long long N, int K) {
  WeightRef o = w;
  const long long nk = N * (long long)K;
  if (FMT == WF_BF16) o.p0 = (const uint8_t*)w.p0 + e * nk * 2;
  else if (FMT == WF_Q8) { o.p0 = (const uint8_t*)w.p0 + e * nk; o.p1 = (const uint8_t*)w.p1 + e * (nk / 32) * 2; }
  else if (FMT == WF_Q4K) o.p0 = (const uint8_t*)w.p0 + e * (nk / 256) * 144;
  else if (FMT == WF_Q6K) { o.p0 = (const uint8_t*)w.p0 + e * (nk / 2); o.p1 = (const uint8_t*)w.p1 + e * (nk / 4); o.p2 = (const uint8_t*)w.p2 + e * (nk / 16); o.p3 = (const uint8_t*)w.p3 + e * (nk / 256) * 2; }
  else { o.p0 = (const uint8_t*)w.p0 + e * (nk / 2); o.p1 = (const uint8_t*)w.p1 + e * (nk / 32); }
  return o;
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg8(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

// 6-bit (scale, min) pair of sub-block `sub` from the 12 scale bytes held in (s0,s1,s2) little-endian words
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int sub, int& sc, int& mn) {
  // bytes 0..3 = s0, 4..7 = s1, 8..11 = s2
  if (sub < 4) {
    sc = (s0 >> (8 * sub)) & 63;
    mn = (s1 >> (8 * sub)) & 63;
  } else {
    const int j = sub - 4;
    const uint32_t hi = (s2 >> (8 * j)) & 0xFF;
    sc = (hi & 0x0F) | (((s0 >> (8 * j + 6)) & 3) << 4);
    mn = (hi >> 4) | (((s1 >> (8 * j + 6)) & 3) << 4);
  }
}

// float(128 + byte i of `v`) built with one byte permute; exact for byte values < 128.
template <int I>
__device__ __forceinline__ float magic128(uint32_t v) {
  // result bytes: [3]=0x43, [2]=v.byte[I], [1]=0, [0]=0
  return __uint_as_float(__byte_perm(v, 0x00000043u, 0x4055 | (I << 8)));
}
// float(32768 + byte) : 0x47000000 has ulp 2^-8*... use bf16-style placement: value = 2^15 + byte*2^8?  (unused)

// ------------------------------------------------------------------ decode to 32 floats
template <int FMT>
__device__ __forceinline__ void decode32_f32(const RowPtrs& r, int kb, float (&w)[32]);

template <>
__device__ __forceinline__ void decode32_f32<WF_BF16>(const RowPtrs& r, int kb, float (&w)[32]) {
  const uint4* p = reinterpret_cast<const uint4*>(r.p0 + (size_t)kb * 64);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v = __ldg(p + i);
    w[8 * i + 0] = bf16_lo(v.x); w[8 * i + 1] = bf16_hi(v.x);
    w[8 * i + 2] = bf16_lo(v.y); w[8 * i + 3] = bf16_hi(v.y);
    w[8 * i + 4] = bf16_lo(v.z); w[8 * i + 5] = bf16_hi(v.z);
    w[8 * i + 6] = bf16_lo(v.w); w[8 * i + 7] = bf16_hi(v.w);
  }
}

template <>
__device__ __forceinline__ void decode32_f32<WF_Q8>(const RowPtrs& r, int kb, float (&w)[32]) {
  const float d = __half2float(__ldg(reinterpret_cast<const __half*>(r.p1) + kb));
  const uint4 a = ldg16(r.p0 + (size_t)kb * 32), b = ldg16(r.p0 + (size_t)kb * 32 + 16);
  const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[4 * i + 0] = d * (float)(int8_t)(q[i] & 0xFF);
    w[4 * i + 1] = d * (float)(int8_t)((q[i] >> 8) & 0xFF);
    w[4 * i + 2] = d * (float)(int8_t)((q[i] >> 16) & 0xFF);
    w[4 * i + 3] = d * (float)(int8_t)(q[i] >> 24);
  }
}

template <>
__device__ __forceinline__ void decode32_f32<WF_Q4K>(const RowPtrs& r, int kb, float (&w)[32]) {
  const uint8_t* blk = r.p0 + (size_t)(kb >> 3) * 144;
  const int sub = kb & 7;
  const uint4 hdr = ldg16(blk);   // d, dmin, scales[12]
  const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
  const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
  int sc, mn;
  q4k_scale_min(hdr.y, hdr.z, hdr.w, sub, sc, mn);
  const float ds = d * sc, c = -(128.f * ds + dmin * mn);
  const uint8_t* qs = blk + 16 + 32 * (sub >> 1);
  const uint4 a = ldg16(qs), b = ldg16(qs + 16);
  const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  const int sh = (sub & 1) * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t t = (q[i] >> sh) & 0x0F0F0F0Fu;
    w[4 * i + 0] = fmaf(magic128<0>(t), ds, c);
    w[4 * i + 1] = fmaf(magic128<1>(t), ds, c);
    w[4 * i + 2] = fmaf(magic128<2>(t), ds, c);
    w[4 * i + 3] = fmaf(magic128<3>(t), ds, c);
  }
}

// Q6K planes.  lo4: natural nibble order (byte i = e[2i] | e[2i+1]<<4).
// hi2: per 16 elements one 32-bit word; byte b holds e[2b] (bits 0-1), e[2b+1] (2-3), e[8+2b] (4-5), e[9+2b] (6-7).
template <>
__device__ __forceinline__ void decode32_f32<WF_Q6K>(const RowPtrs& r, int kb, float (&w)[32]) {
  const float d = __half2float(__ldg(reinterpret_cast<const __half*>(r.p3) + (kb >> 3)));
  const uint4 lo = ldg16(r.p0 + (size_t)kb * 16);
  const uint2 hi = ldg8(r.p1 + (size_t)kb * 8);
  const unsigned short scw = __ldg(reinterpret_cast<const unsigned short*>(r.p2) + kb);
  const float ds0 = d * (float)(int8_t)(scw & 0xFF), ds1 = d * (float)(int8_t)(scw >> 8);
  const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
  const uint32_t hw[2] = {hi.x, hi.y};
#pragma unroll
  for (int g = 0; g < 4; ++g) {          // 8 elements per lo word
    const uint32_t h = hw[g >> 1] >> ((g & 1) * 4);
    const uint32_t even = (lw[g] & 0x0F0F0F0Fu) | ((h & 0x03030303u) << 4);          // e0 e2 e4 e6
    const uint32_t odd = ((lw[g] >> 4) & 0x0F0F0F0Fu) | (((h >> 2) & 0x03030303u) << 4);  // e1 e3 e5 e7
    const float ds = g < 2 ? ds0 : ds1, c = -160.f * ds;
    w[8 * g + 0] = fmaf(magic128<0>(even), ds, c); w[8 * g + 1] = fmaf(magic128<0>(odd), ds, c);
    w[8 * g + 2] = fmaf(magic128<1>(even), ds, c); w[8 * g + 3] = fmaf(magic128<1>(odd), ds, c);
    w[8 * g + 4] = fmaf(magic128<2>(even), ds, c); w[8 * g + 5] = fmaf(magic128<2>(odd), ds, c);
    w[8 * g + 6] = fmaf(magic128<3>(even), ds, c); w[8 * g + 7] = fmaf(magic128<3>(odd), ds, c);
  }
}

// E2M1 magnitudes as bf16: {0, .5, 1, 1.5, 2, 3, 4, 6} -> high bytes / low bytes tables for PRMT lookups.
// four 4-bit codes (low 16 bits of `codes`) -> two bf16x2 words (elements 0,1 and 2,3), signed.
__device__ __forceinline__ void e2m1x4_to_bf16x2(uint32_t codes, uint32_t& p01, uint32_t& p23) {
  const uint32_t sel = codes & 0x7777u;
  const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);   // high bytes of the 4 magnitudes
  const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel);   // low bytes
  p01 = __byte_perm(lo, hi, 0x5140) | ((codes << 12) & 0x00008000u) | ((codes << 24) & 0x80000000u);
  p23 = __byte_perm(lo, hi, 0x7362) | ((codes << 4) & 0x00008000u) | ((codes << 16) & 0x80000000u);
}

template <>
__device__ __forceinline__ void decode32_f32<WF_MXFP4>(const RowPtrs& r, int kb, float (&w)[32]) {
  const float s = e8m0_f32(__ldg(r.p1 + kb));
  const uint4 v = ldg16(r.p0 + (size_t)kb * 16);
  const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t a, b, c, d2;
    e2m1x4_to_bf16x2(q[i], a, b);
    e2m1x4_to_bf16x2(q[i] >> 16, c, d2);
    w[8 * i + 0] = bf16_lo(a) * s; w[8 * i + 1] = bf16_hi(a) * s;
    w[8 * i + 2] = bf16_lo(b) * s; w[8 * i + 3] = bf16_hi(b) * s;
    w[8 * i + 4] = bf16_lo(c) * s; w[8 * i + 5] = bf16_hi(c) * s;
    w[8 * i + 6] = bf16_lo(d2) * s; w[8 * i + 7] = bf16_hi(d2) * s;
  }
}

// ------------------------------------------------------------------ decode to 16 bf16x2 words
template <int FMT>
__device__ __forceinline__ void decode32_bf16(const RowPtrs& r, int kb, uint32_t (&o)[16]) {
  if constexpr (FMT == WF_MXFP4) {
    // scale is a power of two: bf16 multiply is exact (up to under/overflow)
    const uint32_t e = __ldg(r.p1 + kb);
    const uint32_t sb = e == 0 ? 0x0040u : (e << 7);
    const uint32_t s2 = sb | (sb << 16);
    const __nv_bfloat162 sv = *reinterpret_cast<const __nv_bfloat162*>(&s2);
    const uint4 v = ldg16(r.p0 + (size_t)kb * 16);
    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t[4];
      e2m1x4_to_bf16x2(q[i], t[0], t[1]);
      e2m1x4_to_bf16x2(q[i] >> 16, t[2], t[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 p = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t[j]), sv);
        o[4 * i + j] = *reinterpret_cast<uint32_t*>(&p);
      }
    }
  } else if constexpr (FMT == WF_BF16) {
    const uint4* p = reinterpret_cast<const uint4*>(r.p0 + (size_t)kb * 64);
#pragma unroll
    for (int i = 0; i < 4; ++i) { uint4 v = __ldg(p + i); o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w; }
  } else {
    float w[32];
    decode32_f32<FMT>(r, kb, w);
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = pack_bf16(w[2 * i], w[2 * i + 1]);
  }
}

}  // namespace mx
