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

// Row strides of the auxiliary (scale) planes are padded to 16 bytes so that rows stay aligned
// for 4-byte asynchronous copies whatever K is.
__host__ __device__ __forceinline__ int mxfp4_e_stride(int K) { return ((K / 32 + 15) / 16) * 16; }   // bytes
__host__ __device__ __forceinline__ int q8_d_stride(int K) { return ((K / 32 + 7) / 8) * 8; }         // fp16 elements
__host__ __device__ __forceinline__ int q6k_d_stride(int K) { return ((K / 256 + 7) / 8) * 8; }       // fp16 elements

// Per-row plane strides in bytes for a [N][K] matrix.
template <int FMT>
__device__ __forceinline__ RowPtrs row_ptrs(const WeightRef& w, long long row, int K) {
  RowPtrs r;
  const uint8_t* b0 = (const uint8_t*)w.p0;
  const uint8_t* b1 = (const uint8_t*)w.p1;
  const uint8_t* b2 = (const uint8_t*)w.p2;
  const uint8_t* b3 = (const uint8_t*)w.p3;
  if (FMT == WF_BF16) { r.p0 = b0 + row * K * 2; r.p1 = r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q8) { r.p0 = b0 + row * K; r.p1 = b1 + row * q8_d_stride(K) * 2; r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q4K) { r.p0 = b0 + row * (K / 256) * 144; r.p1 = r.p2 = r.p3 = nullptr; }
  else if (FMT == WF_Q6K) { r.p0 = b0 + row * (K / 2); r.p1 = b1 + row * (K / 4); r.p2 = b2 + row * (K / 16); r.p3 = b3 + row * q6k_d_stride(K) * 2; }
  else { r.p0 = b0 + row * (K / 2); r.p1 = b1 + row * mxfp4_e_stride(K); r.p2 = r.p3 = nullptr; }
  return r;
}

// Byte offset between consecutive experts for each plane of a stacked [E][N][K] weight.
template <int FMT>
__device__ __forceinline__ WeightRef expert_weight(const WeightRef& w, long long e, long long N, int K) {
  WeightRef o = w;
  const long long nk = N * (long long)K;
  if (FMT == WF_BF16) o.p0 = (const uint8_t*)w.p0 + e * nk * 2;
  else if (FMT == WF_Q8) { o.p0 = (const uint8_t*)w.p0 + e * nk; o.p1 = (const uint8_t*)w.p1 + e * N * q8_d_stride(K) * 2; }
  else if (FMT == WF_Q4K) o.p0 = (const uint8_t*)w.p0 + e * (nk / 256) * 144;
  else if (FMT == WF_Q6K) { o.p0 = (const uint8_t*)w.p0 + e * (nk / 2); o.p1 = (const uint8_t*)w.p1 + e * (nk / 4); o.p2 = (const uint8_t*)w.p2 + e * (nk / 16); o.p3 = (const uint8_t*)w.p3 + e * N * q6k_d_stride(K) * 2; }
  else { o.p0 = (const uint8_t*)w.p0 + e * (nk / 2); o.p1 = (const uint8_t*)w.p1 + e * N * mxfp4_e_stride(K); }
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
// float(2^23 + byte i of `v`) built with one byte permute: exact for all 256 byte values (the int -> float conversion instruction
// issues at a quarter of the rate of the permute + add it replaces)
template <int I>
__device__ __forceinline__ float magic23(uint32_t v) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | I));     // bytes: [3] = 0x4B, [2] = [1] = 0, [0] = v.byte[I]
}

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
  constexpr float OFF = 8388736.f;                  // 2^23 + 128 (see magic23)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t u = q[i] ^ 0x80808080u;
    w[4 * i + 0] = d * (magic23<0>(u) - OFF);
    w[4 * i + 1] = d * (magic23<1>(u) - OFF);
    w[4 * i + 2] = d * (magic23<2>(u) - OFF);
    w[4 * i + 3] = d * (magic23<3>(u) - OFF);
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

// E2M1 magnitudes as bf16: {0, .5, 1, 1.5, 2, 3, 4, 6} = 0x0000 3F00 3F80 3FC0 4000 4040 4080 40C0.
// Eight 4-bit codes (natural order, code j in bits 4j..4j+3, sign in bit 3 of each nibble) are
// turned into four bf16x2 words with byte permutes only: the magnitude bytes come from two 8-entry
// byte tables indexed by the 3-bit magnitude, and the sign bits are produced by PRMT's
// sign-replicate mode (selector 8|b copies the top bit of byte b into a whole byte).
__device__ __forceinline__ void e2m1x8_to_bf16x2(uint32_t w, uint32_t (&o)[4]) {
  const uint32_t se = __byte_perm(w << 4, 0u, 0xBA98);      // byte b = 0xFF if code 2b   is negative
  const uint32_t so = __byte_perm(w, 0u, 0xBA98);           // byte b = 0xFF if code 2b+1 is negative
  const uint32_t sel = w & 0x77777777u;
  {
    const uint32_t sg = __byte_perm(se, so, 0x5140);                     // signs of codes 0,1,2,3
    const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel) | (sg & 0x80808080u);
    const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel);
    o[0] = __byte_perm(lo, hi, 0x5140);
    o[1] = __byte_perm(lo, hi, 0x7362);
  }
  {
    const uint32_t sel2 = sel >> 16;
    const uint32_t sg = __byte_perm(se, so, 0x7362);                     // signs of codes 4,5,6,7
    const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel2) | (sg & 0x80808080u);
    const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel2);
    o[2] = __byte_perm(lo, hi, 0x5140);
    o[3] = __byte_perm(lo, hi, 0x7362);
  }
}
// Eight E2M1 codes -> four f16x2 words with the sm_100a conversion instruction (low nibble -> low half).
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(unsigned short two_bytes) {   // converts the LOW byte
  uint32_t r;
  asm("{\n\t.reg .b8 lo8, hi8;\n\t"
      "mov.b16 {lo8, hi8}, %1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, lo8;\n\t}\n"
      : "=r"(r)
      : "h"(two_bytes));
  return r;
}
// The byte to convert is isolated first (one byte permute, upper byte zero): a non-zero neighbour in
// the 16-bit operand was observed to disturb the conversion of the upper nibble.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&o)[4]) {
  o[0] = e2m1x2_to_f16x2((unsigned short)__byte_perm(w, 0u, 0x4440));
  o[1] = e2m1x2_to_f16x2((unsigned short)__byte_perm(w, 0u, 0x4441));
  o[2] = e2m1x2_to_f16x2((unsigned short)__byte_perm(w, 0u, 0x4442));
  o[3] = e2m1x2_to_f16x2((unsigned short)__byte_perm(w, 0u, 0x4443));
}
// e8m0 exponent byte -> 2^(e-127) replicated in both halves of an f16x2 (flushes below 2^-24, clamps above 2^15)
__device__ __forceinline__ uint32_t e8m0_to_f16x2(uint32_t e) {
  const int x = (int)e - 112;                    // fp16 exponent field
  uint32_t b;
  if (x >= 1) b = (uint32_t)(x > 30 ? 30 : x) << 10;
  else b = x >= -9 ? (1u << (9 + x)) : 0u;       // subnormal fp16
  return b | (b << 16);
}
// four codes (low 16 bits) -> two bf16x2 words
__device__ __forceinline__ void e2m1x4_to_bf16x2(uint32_t codes, uint32_t& p01, uint32_t& p23) {
  uint32_t o[4];
  e2m1x8_to_bf16x2(codes & 0xFFFFu, o);
  p01 = o[0];
  p23 = o[1];
}

template <>
__device__ __forceinline__ void decode32_f32<WF_MXFP4>(const RowPtrs& r, int kb, float (&w)[32]) {
  const float s = e8m0_f32(__ldg(r.p1 + kb));
  const uint4 v = ldg16(r.p0 + (size_t)kb * 16);
  const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t t[4];
    e2m1x8_to_bf16x2(q[i], t);
    w[8 * i + 0] = bf16_lo(t[0]) * s; w[8 * i + 1] = bf16_hi(t[0]) * s;
    w[8 * i + 2] = bf16_lo(t[1]) * s; w[8 * i + 3] = bf16_hi(t[1]) * s;
    w[8 * i + 4] = bf16_lo(t[2]) * s; w[8 * i + 5] = bf16_hi(t[2]) * s;
    w[8 * i + 6] = bf16_lo(t[3]) * s; w[8 * i + 7] = bf16_hi(t[3]) * s;
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
      e2m1x8_to_bf16x2(q[i], t);
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

// ------------------------------------------------------------------ asynchronous raw staging (GEMM producers)
// A producer thread owns (row, half) of a 64-wide k tile.  raw_issue() starts cp.async copies of the
// packed bytes it needs for k-iteration `kiter` into its private shared-memory slot; raw_decode()
// later turns that slot into 16 bf16x2 words and tells which 16-byte chunks of the 128-byte B row
// they are.  Slots are private to the thread, so cp.async.wait_group is the only synchronisation.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Per producer thread and k-iteration: MAIN bytes (16-byte granules) and AUX bytes (scales) live in two
// separate shared arrays, each indexed by thread, so neighbouring threads touch neighbouring banks.
template <int FMT> struct RawSlot { static constexpr int MAIN = 16, AUX = 4; };
template <> struct RawSlot<WF_Q8> { static constexpr int MAIN = 32, AUX = 4; };
template <> struct RawSlot<WF_Q4K> { static constexpr int MAIN = 16, AUX = 16; };
template <> struct RawSlot<WF_Q6K> { static constexpr int MAIN = 16, AUX = 16; };

template <int FMT>
__device__ __forceinline__ void raw_issue(uint32_t slot, uint32_t aux, const RowPtrs& rp, int kiter, int half) {
  const int kb = 2 * kiter + half;
  if constexpr (FMT == WF_MXFP4) {
    cp_async16(slot, rp.p0 + (size_t)kb * 16);
    cp_async4(aux, rp.p1 + ((2 * kiter) & ~3));
  } else if constexpr (FMT == WF_Q8) {
    cp_async16(slot, rp.p0 + (size_t)kb * 32);
    cp_async16(slot + 16, rp.p0 + (size_t)kb * 32 + 16);
    cp_async4(aux, rp.p1 + 4 * kiter);
  } else if constexpr (FMT == WF_Q4K) {
    const uint8_t* blk = rp.p0 + (size_t)(kiter >> 2) * 144;
    cp_async16(slot, blk + 16 + 32 * (kiter & 3) + 16 * half);
    cp_async16(aux, blk);
  } else if constexpr (FMT == WF_Q6K) {
    cp_async16(slot, rp.p0 + (size_t)kb * 16);
    cp_async8(aux, rp.p1 + (size_t)kb * 8);
    cp_async4(aux + 8, rp.p2 + 4 * kiter);
    cp_async4(aux + 12, rp.p3 + ((2 * (kiter >> 2)) & ~3));
  }
}

// chunk(c) = index of the c-th produced 16-byte chunk inside the 8-chunk (64 element) B row
template <int FMT>
__device__ __forceinline__ int raw_chunk(int half, int c) {
  if constexpr (FMT == WF_Q4K) return (c < 2 ? 0 : 4) + 2 * half + (c & 1);
  return 4 * half + c;
}

template <int FMT>
__device__ __forceinline__ void raw_decode(const uint8_t* slot, const uint8_t* aux, int kiter, int half, uint32_t (&o)[16]) {
  if constexpr (FMT == WF_MXFP4) {
    // Byte-permute table decode to bf16 (ALU pipe), then one packed multiply by the power-of-two scale.
    // The hardware conversion (e2m1x8_to_f16x2) was measured slower here: it issues on the XU pipe,
    // which saturates at a quarter of the rate this loop needs.
    const uint32_t e = aux[(2 * kiter + half) & 3];
    const uint32_t sb = e == 0 ? 0x0040u : (e << 7);
    const uint32_t s2 = sb | (sb << 16);
    const __nv_bfloat162 sv = *reinterpret_cast<const __nv_bfloat162*>(&s2);
    const uint4 v = *reinterpret_cast<const uint4*>(slot);
    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t[4];
      e2m1x8_to_bf16x2(q[i], t);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 pr = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t[j]), sv);
        o[4 * i + j] = *reinterpret_cast<uint32_t*>(&pr);
      }
    }
  } else if constexpr (FMT == WF_Q8) {
    const float d = __half2float(*reinterpret_cast<const __half*>(aux + 2 * half));
    const uint4 a = *reinterpret_cast<const uint4*>(slot), b = *reinterpret_cast<const uint4*>(slot + 16);
    const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    constexpr float OFF = 8388736.f;                // 2^23 + 128: (2^23 + byte) - OFF is the signed value, exactly
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t u = q[i] ^ 0x80808080u;        // signed -> offset-128 unsigned bytes
      o[2 * i] = pack_bf16((magic23<0>(u) - OFF) * d, (magic23<1>(u) - OFF) * d);
      o[2 * i + 1] = pack_bf16((magic23<2>(u) - OFF) * d, (magic23<3>(u) - OFF) * d);
    }
  } else if constexpr (FMT == WF_Q4K) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(aux);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const int j = kiter & 3;
    int sc0, mn0, sc1, mn1;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j, sc0, mn0);
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * j + 1, sc1, mn1);
    const float ds0 = d * sc0, c0 = -(128.f * ds0 + dmin * mn0), ds1 = d * sc1, c1 = -(128.f * ds1 + dmin * mn1);
    const uint4 v = *reinterpret_cast<const uint4*>(slot);
    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = q[i] & 0x0F0F0F0Fu, hi = (q[i] >> 4) & 0x0F0F0F0Fu;
      o[2 * i] = pack_bf16(fmaf(magic128<0>(lo), ds0, c0), fmaf(magic128<1>(lo), ds0, c0));
      o[2 * i + 1] = pack_bf16(fmaf(magic128<2>(lo), ds0, c0), fmaf(magic128<3>(lo), ds0, c0));
      o[8 + 2 * i] = pack_bf16(fmaf(magic128<0>(hi), ds1, c1), fmaf(magic128<1>(hi), ds1, c1));
      o[8 + 2 * i + 1] = pack_bf16(fmaf(magic128<2>(hi), ds1, c1), fmaf(magic128<3>(hi), ds1, c1));
    }
  } else if constexpr (FMT == WF_Q6K) {
    const int dsel = (2 * (kiter >> 2)) & 3;
    const float d = __half2float(*reinterpret_cast<const __half*>(aux + 12 + dsel));
    const uint4 lo = *reinterpret_cast<const uint4*>(slot);
    const uint2 hi = *reinterpret_cast<const uint2*>(aux);
    const uint32_t scw = *reinterpret_cast<const unsigned short*>(aux + 8 + 2 * half);
    const float ds0 = d * (float)(int8_t)(scw & 0xFF), ds1 = d * (float)(int8_t)(scw >> 8);
    const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
    const uint32_t hw[2] = {hi.x, hi.y};
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t h = hw[g >> 1] >> ((g & 1) * 4);
      const uint32_t even = (lw[g] & 0x0F0F0F0Fu) | ((h & 0x03030303u) << 4);
      const uint32_t odd = ((lw[g] >> 4) & 0x0F0F0F0Fu) | (((h >> 2) & 0x03030303u) << 4);
      const float ds = g < 2 ? ds0 : ds1, c = -160.f * ds;
      o[4 * g + 0] = pack_bf16(fmaf(magic128<0>(even), ds, c), fmaf(magic128<0>(odd), ds, c));
      o[4 * g + 1] = pack_bf16(fmaf(magic128<1>(even), ds, c), fmaf(magic128<1>(odd), ds, c));
      o[4 * g + 2] = pack_bf16(fmaf(magic128<2>(even), ds, c), fmaf(magic128<2>(odd), ds, c));
      o[4 * g + 3] = pack_bf16(fmaf(magic128<3>(even), ds, c), fmaf(magic128<3>(odd), ds, c));
    }
  }
}

}  // namespace mx
