// Block-quantisation codecs (host side).
//
// Byte layouts are the ggml ones, so files written here load in any GGUF
// consumer and files produced elsewhere load here.  Reference parity:
// include/ie/quant_blocks.hpp:26-181 (layouts), include/ie/dequant_ref.hpp
// (decode formulas), src/loaders/quantize_q4k.cpp / quantize_q6k.cpp (encoders).
//
// The decoders are written as "element accessors": value(block, i) for one
// element i, and the bulk routines loop over them.  That form is what the CUDA
// repack kernels mirror, and it makes the odd ggml element orders explicit.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <cmath>

namespace mx {

// ggml type ids (GGUF tensor type field).
enum GgmlType : int32_t {
  T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
  T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_Q8_K = 15,
  T_I8 = 24, T_I16 = 25, T_I32 = 26, T_I64 = 27, T_F64 = 28, T_BF16 = 30, T_EXL3 = 37, T_MXFP4 = 39,
};

struct TypeTraits { int block_elems; int block_bytes; const char* name; };
// Returns {0,0,nullptr} for ids this engine does not decode.
TypeTraits type_traits(int32_t t);
// Bytes for n elements of type t (n must be a whole number of blocks); 0 if unknown.
size_t bytes_for(int32_t t, size_t n);

// ---- scalar conversions -------------------------------------------------
inline float fp16_to_fp32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {  // subnormal: renormalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + 112) << 23) | (man << 13);
  float f; std::memcpy(&f, &bits, 4); return f;
}
inline uint16_t fp32_to_fp16(float f) {
  uint32_t x; std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - exp;
    uint32_t r = man >> shift, rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)exp << 10) | (man >> 13), rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;  // carries into exp correctly
  return (uint16_t)(sign | r);
}
inline float bf16_to_fp32(uint16_t h) { uint32_t b = (uint32_t)h << 16; float f; std::memcpy(&f, &b, 4); return f; }
inline uint16_t fp32_to_bf16(float f) {
  uint32_t x; std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40);
  x += 0x7FFFu + ((x >> 16) & 1);
  return (uint16_t)(x >> 16);
}
// e8m0 exponent byte -> 2^(e-127).  e=0 is 2^-127 (a float subnormal), e=255 is NaN in OCP MX.
inline float e8m0_to_fp32(uint8_t e) {
  uint32_t bits = e == 0 ? 0x00400000u : ((uint32_t)e << 23);
  float f; std::memcpy(&f, &bits, 4); return f;
}
// E2M1 code (4 bits, sign in bit 3) -> value in {0,.5,1,1.5,2,3,4,6} with sign.
inline float e2m1_to_fp32(uint8_t c) {
  static const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float v = mag[c & 7]; return (c & 8) ? -v : v;
}

// ---- bulk API -------------------------------------------------------------
// dst receives n floats; src holds n elements of ggml type t. Returns 0 on success.
int dequantize(int32_t t, const void* src, float* dst, size_t n);
// src holds nrows*ncols floats (row-major); dst receives the packed rows.
// ncols must be a multiple of the type's block size. Uses up to nthreads workers.
int quantize(int32_t t, const float* src, void* dst, size_t nrows, size_t ncols, int nthreads);
// Q4_K / Q5_K sub-block fit: 0 = better of the two per sub-block (default), 1 = alternating least squares, 2 = ggml-style weighted grid search
void set_kquant_fit(int mode);

}  // namespace mx
