// Host codecs for the ggml block formats this engine reads and writes.
// See quant.h for the contract.  Decoders are per-element accessors (the CUDA
// repack kernels follow the same index maps); encoders are this project's own
// least-squares fits that emit valid ggml blocks.
#include "quant.h"

#include <algorithm>
#include <thread>
#include <vector>

namespace mx {

TypeTraits type_traits(int32_t t) {
  switch (t) {
    case T_F32:  return {1, 4, "F32"};
    case T_F16:  return {1, 2, "F16"};
    case T_BF16: return {1, 2, "BF16"};
    case T_I8:   return {1, 1, "I8"};
    case T_I16:  return {1, 2, "I16"};
    case T_I32:  return {1, 4, "I32"};
    case T_I64:  return {1, 8, "I64"};
    case T_F64:  return {1, 8, "F64"};
    case T_Q4_0: return {32, 18, "Q4_0"};
    case T_Q8_0: return {32, 34, "Q8_0"};
    case T_MXFP4:return {32, 17, "MXFP4"};
    case T_EXL3: return {1, 2, "EXL3"};        // trellis words (int16), dims {16 * bits, N / 16, K / 16}; decoded by exl3.cpp
    case T_Q4_K: return {256, 144, "Q4_K"};
    case T_Q5_K: return {256, 176, "Q5_K"};
    case T_Q6_K: return {256, 210, "Q6_K"};
    // Known ids whose payload we can size (so a file holding them can be listed) but not decode.
    case T_Q4_1: return {32, 20, "Q4_1"};
    case T_Q5_0: return {32, 22, "Q5_0"};
    case T_Q5_1: return {32, 24, "Q5_1"};
    case T_Q2_K: return {256, 84, "Q2_K"};
    case T_Q3_K: return {256, 110, "Q3_K"};
    case T_Q8_K: return {256, 292, "Q8_K"};
    default:     return {0, 0, nullptr};
  }
}

size_t bytes_for(int32_t t, size_t n) {
  TypeTraits tt = type_traits(t);
  if (!tt.block_elems || n % tt.block_elems) return 0;
  return n / tt.block_elems * (size_t)tt.block_bytes;
}

static inline uint16_t ld16(const uint8_t* p) { uint16_t v; std::memcpy(&v, p, 2); return v; }
static inline void st16(uint8_t* p, uint16_t v) { std::memcpy(p, &v, 2); }

// 6-bit (scale, min) pair `sub` (0..7) of a Q4_K/Q5_K 12-byte scale field.
static inline void k4_scale_min(const uint8_t* s, int sub, int& sc, int& mn) {
  if (sub < 4) { sc = s[sub] & 63; mn = s[sub + 4] & 63; }
  else {
    sc = (s[sub + 4] & 0x0F) | ((s[sub - 4] >> 6) << 4);
    mn = (s[sub + 4] >> 4)   | ((s[sub]     >> 6) << 4);
  }
}
static inline void k4_pack_scale_min(uint8_t* s, const int* sc, const int* mn) {
  std::memset(s, 0, 12);
  for (int j = 0; j < 8; ++j) {
    if (j < 4) { s[j] |= sc[j] & 63; s[j + 4] |= mn[j] & 63; }
    else {
      s[j + 4] = (uint8_t)((sc[j] & 0x0F) | ((mn[j] & 0x0F) << 4));
      s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
      s[j]     |= (uint8_t)((mn[j] >> 4) << 6);
    }
  }
}

// ---- element accessors ---------------------------------------------------------------
static inline float q8_0_at(const uint8_t* b, int i) { return fp16_to_fp32(ld16(b)) * (float)(int8_t)b[2 + i]; }
static inline float q4_0_at(const uint8_t* b, int i) {
  uint8_t byte = b[2 + (i & 15)];
  int q = (i < 16) ? (byte & 0x0F) : (byte >> 4);
  return fp16_to_fp32(ld16(b)) * (float)(q - 8);
}
static inline float mxfp4_at(const uint8_t* b, int i) {
  uint8_t byte = b[1 + (i & 15)];
  return e2m1_to_fp32((i < 16) ? (byte & 0x0F) : (byte >> 4)) * e8m0_to_fp32(b[0]);
}
static inline float q4_k_at(const uint8_t* b, int i) {
  int sc, mn; k4_scale_min(b + 4, i >> 5, sc, mn);
  uint8_t byte = b[16 + 32 * (i >> 6) + (i & 31)];
  int q = ((i >> 5) & 1) ? (byte >> 4) : (byte & 0x0F);
  return fp16_to_fp32(ld16(b)) * sc * q - fp16_to_fp32(ld16(b + 2)) * mn;
}
static inline float q5_k_at(const uint8_t* b, int i) {
  int sc, mn; k4_scale_min(b + 4, i >> 5, sc, mn);
  const uint8_t* qh = b + 16; const uint8_t* qs = b + 48;
  uint8_t byte = qs[32 * (i >> 6) + (i & 31)];
  int q = ((i >> 5) & 1) ? (byte >> 4) : (byte & 0x0F);
  q += ((qh[i & 31] >> (i >> 5)) & 1) << 4;
  return fp16_to_fp32(ld16(b)) * sc * q - fp16_to_fp32(ld16(b + 2)) * mn;
}
static inline float q6_k_at(const uint8_t* b, int i) {
  const uint8_t* ql = b; const uint8_t* qh = b + 128; const int8_t* sc = (const int8_t*)(b + 192);
  int half = i >> 7, r = i & 127, quarter = r >> 5, l = r & 31;
  uint8_t lo = ql[64 * half + l + ((quarter & 1) << 5)];
  int q = (quarter < 2 ? (lo & 0x0F) : (lo >> 4)) | (((qh[32 * half + l] >> (2 * quarter)) & 3) << 4);
  return fp16_to_fp32(ld16(b + 208)) * sc[8 * half + 2 * quarter + (l >> 4)] * (float)(q - 32);
}

int dequantize(int32_t t, const void* src_, float* dst, size_t n) {
  const uint8_t* src = (const uint8_t*)src_;
  TypeTraits tt = type_traits(t);
  if (!tt.block_elems || n % tt.block_elems) return -1;
  switch (t) {
    case T_F32: std::memcpy(dst, src, n * 4); return 0;
    case T_F16: for (size_t i = 0; i < n; ++i) dst[i] = fp16_to_fp32(ld16(src + 2 * i)); return 0;
    case T_BF16: for (size_t i = 0; i < n; ++i) dst[i] = bf16_to_fp32(ld16(src + 2 * i)); return 0;
    default: break;
  }
  float (*at)(const uint8_t*, int) = nullptr;
  switch (t) {
    case T_Q8_0: at = q8_0_at; break;   case T_Q4_0: at = q4_0_at; break;
    case T_MXFP4: at = mxfp4_at; break; case T_Q4_K: at = q4_k_at; break;
    case T_Q5_K: at = q5_k_at; break;   case T_Q6_K: at = q6_k_at; break;
    default: return -2;
  }
  const int be = tt.block_elems, bb = tt.block_bytes;
  for (size_t blk = 0; blk < n / be; ++blk)
    for (int i = 0; i < be; ++i) dst[blk * be + i] = at(src + blk * bb, i);
  return 0;
}

// ---- encoders -------------------------------------------------------------------------
static inline int nearest_int(float v) { return (int)std::lrintf(v); }

static void enc_q8_0(const float* x, uint8_t* b) {
  float amax = 0; for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  float d = amax / 127.f, id = d > 0 ? 1.f / d : 0.f;
  st16(b, fp32_to_fp16(d));
  for (int i = 0; i < 32; ++i) b[2 + i] = (uint8_t)(int8_t)std::clamp(nearest_int(x[i] * id), -127, 127);
}
static void enc_q4_0(const float* x, uint8_t* b) {
  float amax = 0, mx_ = 0;
  for (int i = 0; i < 32; ++i) if (std::fabs(x[i]) > amax) { amax = std::fabs(x[i]); mx_ = x[i]; }
  float d = mx_ / -8.f, id = d != 0 ? 1.f / d : 0.f;
  st16(b, fp32_to_fp16(d));
  for (int i = 0; i < 16; ++i) {
    int lo = std::clamp((int)(x[i] * id + 8.5f), 0, 15), hi = std::clamp((int)(x[i + 16] * id + 8.5f), 0, 15);
    b[2 + i] = (uint8_t)(lo | (hi << 4));
  }
}
static inline uint8_t e2m1_nearest(float v) {
  static const float mag[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float a = std::fabs(v); int best = 0; float bd = a;
  for (int k = 1; k < 8; ++k) { float dd = std::fabs(a - mag[k]); if (dd < bd) { bd = dd; best = k; } }
  return (uint8_t)(best | ((v < 0 && best) ? 8 : 0));
}
static void enc_mxfp4(const float* x, uint8_t* b) {
  float amax = 0; for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[i]));
  int e = 0;
  if (amax > 0) {
    // largest code is 6 = 1.5 * 2^2: choose the exponent so amax lands in [4,8) * 2^(e-127)
    e = (int)std::floor(std::log2(amax)) - 2 + 127;
    e = std::clamp(e, 0, 254);
  }
  float id = 1.f / e8m0_to_fp32((uint8_t)e);
  b[0] = (uint8_t)e;
  for (int i = 0; i < 16; ++i) b[1 + i] = (uint8_t)(e2m1_nearest(x[i] * id) | (e2m1_nearest(x[i + 16] * id) << 4));
}

// Fit x[i] ~ s*q[i] - m with q in [0,qmax], m >= 0.  A few rounds of (assign q, refit s and m).
static void fit_scale_min(const float* x, int n, int qmax, float& s, float& m) {
  float lo = x[0], hi = x[0];
  for (int i = 1; i < n; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); }
  lo = std::min(lo, 0.f);
  if (hi <= lo) { s = 0; m = -lo; return; }
  s = (hi - lo) / qmax; m = -lo;
  for (int it = 0; it < 4; ++it) {
    double sq = 0, sqq = 0, sx = 0, sqx = 0;
    for (int i = 0; i < n; ++i) {
      int q = std::clamp(nearest_int((x[i] + m) / s), 0, qmax);
      sq += q; sqq += (double)q * q; sx += x[i]; sqx += (double)q * x[i];
    }
    double det = n * sqq - sq * sq;
    if (det <= 0) break;
    double ns = (n * sqx - sq * sx) / det, nm = (sq * sqx - sqq * sx) / det;
    if (ns <= 0) break;
    if (nm < 0) { nm = 0; ns = sqq > 0 ? sqx / sqq : ns; if (ns <= 0) break; }
    s = (float)ns; m = (float)nm;
  }
}

// The same fit by the importance-weighted grid search ggml's K-quant encoders use (make_qkx2_quants: src/loaders/quantize_q4k.cpp:22-81
// in the reference): weights w_i = rms(x) + |x_i|, candidate inverse scales (rmin + rdelta * step + qmax) / (max - min), for each a
// weighted least-squares (scale, min) over the rounded codes, the candidate with the smallest weighted squared error wins.
static void fit_scale_min_search(const float* x, int n, int qmax, float rmin, float rdelta, int nstep, float& s, float& m) {
  float lo = x[0], hi = x[0];
  double sx2 = 0;
  for (int i = 0; i < n; ++i) { lo = std::min(lo, x[i]); hi = std::max(hi, x[i]); sx2 += (double)x[i] * x[i]; }
  lo = std::min(lo, 0.f);
  if (hi <= lo) { s = 0; m = -lo; return; }
  const float av = (float)std::sqrt(sx2 / n);
  float w[64];
  double sw = 0, swx = 0;
  for (int i = 0; i < n; ++i) { w[i] = av + std::fabs(x[i]); sw += w[i]; swx += (double)w[i] * x[i]; }
  auto err_of = [&](float sc, float mn, float inv) {
    double e = 0;
    for (int i = 0; i < n; ++i) {
      const int q = std::clamp(nearest_int(inv * (x[i] - mn)), 0, qmax);
      const double d = (double)sc * q + mn - x[i];
      e += w[i] * d * d;
    }
    return e;
  };
  float best_s = (hi - lo) / qmax, best_min = lo;
  double best = err_of(best_s, best_min, qmax / (hi - lo));
  for (int is = 0; is <= nstep; ++is) {
    const float inv = (rmin + rdelta * is + qmax) / (hi - lo);
    double sl = 0, sl2 = 0, sxl = 0;
    for (int i = 0; i < n; ++i) {
      const int q = std::clamp(nearest_int(inv * (x[i] - lo)), 0, qmax);
      sl += (double)w[i] * q; sl2 += (double)w[i] * q * q; sxl += (double)w[i] * q * x[i];
    }
    const double det = sw * sl2 - sl * sl;
    if (det <= 0) continue;
    double ts = (sw * sxl - swx * sl) / det, tm = (sl2 * swx - sl * sxl) / det;
    if (tm > 0) { tm = 0; ts = sl2 > 0 ? sxl / sl2 : ts; }
    if (ts <= 0) continue;
    const double e = err_of((float)ts, (float)tm, inv);
    if (e < best) { best = e; best_s = (float)ts; best_min = (float)tm; }
  }
  s = best_s; m = -best_min;
}

static double fit_error(const float* x, int n, int qmax, float s, float m) {
  double e = 0;
  for (int i = 0; i < n; ++i) {
    const int q = s > 0 ? std::clamp(nearest_int((x[i] + m) / s), 0, qmax) : 0;
    const double d = (double)s * q - m - x[i];
    e += d * d;
  }
  return e;
}

// 0: per sub-block the better (plain squared error) of the two fits; 1: the alternating least-squares fit only; 2: the grid search only
static int g_kquant_fit = 0;
void set_kquant_fit(int mode) { g_kquant_fit = mode; }

static void enc_q4k_q5k(const float* x, uint8_t* b, bool five) {
  const int qmax = five ? 31 : 15;
  float s[8], m[8], smax = 0, mmax = 0;
  for (int j = 0; j < 8; ++j) {
    const float* xs = x + 32 * j;
    float s1 = 0, m1 = 0, s2 = 0, m2 = 0;
    if (g_kquant_fit != 2) fit_scale_min(xs, 32, qmax, s1, m1);
    if (g_kquant_fit != 1) fit_scale_min_search(xs, 32, qmax, five ? -0.5f : -1.f, 0.1f, five ? 15 : 20, s2, m2);
    const bool second = g_kquant_fit == 2 || (g_kquant_fit == 0 && fit_error(xs, 32, qmax, s2, m2) < fit_error(xs, 32, qmax, s1, m1));
    s[j] = second ? s2 : s1; m[j] = second ? m2 : m1;
    smax = std::max(smax, s[j]); mmax = std::max(mmax, m[j]);
  }
  float d = smax / 63.f, dm = mmax / 63.f;
  uint16_t dh = fp32_to_fp16(d), dmh = fp32_to_fp16(dm);
  float df = fp16_to_fp32(dh), dmf = fp16_to_fp32(dmh);
  int sc[8], mn[8];
  for (int j = 0; j < 8; ++j) {
    sc[j] = df > 0 ? std::clamp(nearest_int(s[j] / df), 0, 63) : 0;
    mn[j] = dmf > 0 ? std::clamp(nearest_int(m[j] / dmf), 0, 63) : 0;
  }
  st16(b, dh); st16(b + 2, dmh);
  k4_pack_scale_min(b + 4, sc, mn);
  uint8_t* qh = five ? b + 16 : nullptr;
  uint8_t* qs = five ? b + 48 : b + 16;
  if (five) std::memset(qh, 0, 32);
  std::memset(qs, 0, 128);
  for (int i = 0; i < 256; ++i) {
    int sub = i >> 5; float es = df * sc[sub], em = dmf * mn[sub];
    int q = es > 0 ? std::clamp(nearest_int((x[i] + em) / es), 0, qmax) : 0;
    uint8_t& byte = qs[32 * (i >> 6) + (i & 31)];
    if ((i >> 5) & 1) byte |= (uint8_t)((q & 15) << 4); else byte |= (uint8_t)(q & 15);
    if (five && (q & 16)) qh[i & 31] |= (uint8_t)(1u << (i >> 5));
  }
}

// Symmetric fit x ~ s*q, q in [-32,31]; s may be negative so that the largest magnitude
// element can use the -32 code.
static float fit_symmetric(const float* x, int n) {
  float amax = 0, vmax = 0;
  for (int i = 0; i < n; ++i) if (std::fabs(x[i]) > amax) { amax = std::fabs(x[i]); vmax = x[i]; }
  if (amax == 0) return 0.f;
  float best_s = vmax / -32.f; double best_err = 1e300;
  for (int c = -4; c <= 4; ++c) {
    float s = vmax / (-32.f + 0.25f * c);
    double sqx = 0, sqq = 0;
    for (int i = 0; i < n; ++i) { int q = std::clamp(nearest_int(x[i] / s), -32, 31); sqx += (double)q * x[i]; sqq += (double)q * q; }
    if (sqq > 0) s = (float)(sqx / sqq);
    double err = 0;
    for (int i = 0; i < n; ++i) { int q = std::clamp(nearest_int(x[i] / s), -32, 31); double e = x[i] - s * q; err += e * e; }
    if (err < best_err) { best_err = err; best_s = s; }
  }
  return best_s;
}

static void enc_q6_k(const float* x, uint8_t* b) {
  float s[16], smax = 0, sabs = 0;
  for (int j = 0; j < 16; ++j) { s[j] = fit_symmetric(x + 16 * j, 16); if (std::fabs(s[j]) > sabs) { sabs = std::fabs(s[j]); smax = s[j]; } }
  std::memset(b, 0, 210);
  if (sabs == 0) return;
  float d = smax / -128.f;
  uint16_t dh = fp32_to_fp16(d); float df = fp16_to_fp32(dh);
  int8_t* sc = (int8_t*)(b + 192);
  st16(b + 208, dh);
  // sub-block j of 16 elements covers elements 16j..16j+15; its scale slot follows the decode map.
  for (int i = 0; i < 256; ++i) {
    int half = i >> 7, r = i & 127, quarter = r >> 5, l = r & 31;
    int slot = 8 * half + 2 * quarter + (l >> 4);
    if ((i & 15) == 0) sc[slot] = (int8_t)std::clamp(nearest_int(s[i >> 4] / df), -128, 127);
    float es = df * sc[slot];
    int q = (es != 0 ? std::clamp(nearest_int(x[i] / es), -32, 31) : 0) + 32;
    uint8_t& lo = b[64 * half + l + ((quarter & 1) << 5)];
    if (quarter < 2) lo |= (uint8_t)(q & 15); else lo |= (uint8_t)((q & 15) << 4);
    b[128 + 32 * half + l] |= (uint8_t)((q >> 4) << (2 * quarter));
  }
}

int quantize(int32_t t, const float* src, void* dst_, size_t nrows, size_t ncols, int nthreads) {
  uint8_t* dst = (uint8_t*)dst_;
  TypeTraits tt = type_traits(t);
  if (!tt.block_elems || ncols % tt.block_elems) return -1;
  const size_t total = nrows * ncols;
  if (t == T_F32) { std::memcpy(dst, src, total * 4); return 0; }
  if (t == T_F16) { for (size_t i = 0; i < total; ++i) st16(dst + 2 * i, fp32_to_fp16(src[i])); return 0; }
  if (t == T_BF16) { for (size_t i = 0; i < total; ++i) st16(dst + 2 * i, fp32_to_bf16(src[i])); return 0; }
  void (*enc)(const float*, uint8_t*) = nullptr;
  switch (t) {
    case T_Q8_0: enc = enc_q8_0; break; case T_Q4_0: enc = enc_q4_0; break; case T_MXFP4: enc = enc_mxfp4; break;
    case T_Q4_K: enc = [](const float* x, uint8_t* b) { enc_q4k_q5k(x, b, false); }; break;
    case T_Q5_K: enc = [](const float* x, uint8_t* b) { enc_q4k_q5k(x, b, true); }; break;
    case T_Q6_K: enc = enc_q6_k; break;
    default: return -2;
  }
  const size_t nblocks = total / tt.block_elems;
  const int be = tt.block_elems, bb = tt.block_bytes;
  int nt = std::max(1, std::min<int>(nthreads, (int)std::min<size_t>(nblocks / 256 + 1, 64)));
  auto work = [&](size_t lo, size_t hi) { for (size_t k = lo; k < hi; ++k) enc(src + k * be, dst + k * bb); };
  if (nt == 1) { work(0, nblocks); return 0; }
  std::vector<std::thread> th;
  for (int w = 0; w < nt; ++w) th.emplace_back(work, nblocks * w / nt, nblocks * (w + 1) / nt);
  for (auto& x : th) x.join();
  return 0;
}

}  // namespace mx
