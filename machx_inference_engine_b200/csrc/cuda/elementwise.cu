// Memory-bound glue kernels, each fusing what the reference ran as separate submits:
//   embed           : dequantising row gather into the fp32 residual stream
//   rmsnorm         : residual add (+bias) + RMSNorm (+ "1+w" form) -> bf16, one pass
//   qkv_post        : bias + per-head QK RMSNorm + NEOX RoPE (table driven: llama3 factors and
//                     YaRN are baked into the cos/sin tables) + Q|gate split + paged KV write
//   glu             : SwiGLU / clamped OAI SwiGLU / GeGLU over 16-column interleaved gate|up
//   gated_rmsnorm   : y = w * x / rms(x) * silu(z) per head (DeltaNet output norm)
//   misc            : sigmoid gate multiply, scaled add, casts
// Reference parity: src/ops/elementwise.cpp:29-786, src/ops/embedding.cpp:45-206,
// src/core/kv_cache.cpp:107-133, src/ops/deltanet.cpp:41-81.
#include "common.cuh"
#include "dequant.cuh"
#include "host_util.h"

namespace mx {

// ------------------------------------------------------------------ embed
template <int FMT>
__global__ void embed_kernel(WeightRef w, const int* __restrict__ ids, float* __restrict__ out, int H, int vocab, float scale) {
  pdl_prologue();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const RowPtrs rp = row_ptrs<FMT>(w, id, H);
  for (int kb = threadIdx.x; kb < H / 32; kb += blockDim.x) {
    float v[32];
    decode32_f32<FMT>(rp, kb, v);
    float4* o = reinterpret_cast<float4*>(out + (size_t)t * H + kb * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = make_float4(v[4 * i] * scale, v[4 * i + 1] * scale, v[4 * i + 2] * scale, v[4 * i + 3] * scale);
  }
}

// ------------------------------------------------------------------ rmsnorm
// x (fp32, [T,H]) += delta (bf16 or fp32, optional) + dbias (optional); out = norm(x) * w.
// delta_scale multiplies delta (Granite residual scale).  If out_f32 != null the normalised row
// is also written in fp32 (final norm feeding an fp32 consumer).
template <typename DT>
__global__ void __launch_bounds__(256) rmsnorm_kernel(float* __restrict__ x, const DT* __restrict__ delta, const float* __restrict__ dbias,
                                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ out, float eps, int H,
                                                      int one_plus_w, float delta_scale, int write_x) {
  pdl_prologue();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * H;
  __shared__ float red[8];
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(xr + i);
    if (delta) {
      float d0, d1, d2, d3;
      if constexpr (sizeof(DT) == 2) {
        const uint2 dv = *reinterpret_cast<const uint2*>(delta + (size_t)t * H + i);
        d0 = bf16_lo(dv.x); d1 = bf16_hi(dv.x); d2 = bf16_lo(dv.y); d3 = bf16_hi(dv.y);
      } else {
        const float4 dv = *reinterpret_cast<const float4*>(delta + (size_t)t * H + i);
        d0 = dv.x; d1 = dv.y; d2 = dv.z; d3 = dv.w;
      }
      if (dbias) { d0 += dbias[i]; d1 += dbias[i + 1]; d2 += dbias[i + 2]; d3 += dbias[i + 3]; }
      v.x += d0 * delta_scale; v.y += d1 * delta_scale; v.z += d2 * delta_scale; v.w += d3 * delta_scale;
      if (write_x) *reinterpret_cast<float4*>(xr + i) = v;
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / H + eps);
  }
  __syncthreads();
  const float inv = red[0];
  if (!out) return;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    // when the sum was not written back (write_x == 0 with delta) recompute it
    float4 v = *reinterpret_cast<const float4*>(xr + i);
    if (delta && !write_x) {
      float d0, d1, d2, d3;
      if constexpr (sizeof(DT) == 2) {
        const uint2 dv = *reinterpret_cast<const uint2*>(delta + (size_t)t * H + i);
        d0 = bf16_lo(dv.x); d1 = bf16_hi(dv.x); d2 = bf16_lo(dv.y); d3 = bf16_hi(dv.y);
      } else {
        const float4 dv = *reinterpret_cast<const float4*>(delta + (size_t)t * H + i);
        d0 = dv.x; d1 = dv.y; d2 = dv.z; d3 = dv.w;
      }
      if (dbias) { d0 += dbias[i]; d1 += dbias[i + 1]; d2 += dbias[i + 2]; d3 += dbias[i + 3]; }
      v.x += d0 * delta_scale; v.y += d1 * delta_scale; v.z += d2 * delta_scale; v.w += d3 * delta_scale;
    }
    float4 g = *reinterpret_cast<const float4*>(w + i);
    if (one_plus_w) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
    uint2 o;
    o.x = pack_bf16(v.x * inv * g.x, v.y * inv * g.y);
    o.y = pack_bf16(v.z * inv * g.z, v.w * inv * g.w);
    *reinterpret_cast<uint2*>(out + (size_t)t * H + i) = o;
  }
}

// Residual add + RMSNorm whose delta is the expert combine: delta[t] = sum_k cw[t,k] * yp[pair_to_packed[t*K+k]] (slot order,
// pairs with a negative position contribute nothing), so that the weighted sum of the expert outputs never exists as a tensor.
__global__ void __launch_bounds__(256) rmsnorm_combine_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ yp, const int* __restrict__ pair_to_packed,
                                                              const float* __restrict__ cw, int K, const float* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ out, float eps, int H, int one_plus_w, float delta_scale) {
  pdl_prologue();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * H;
  __shared__ float red[8];
  __shared__ int s_pos[32];
  __shared__ float s_w[32];
  if (threadIdx.x < K) {
    s_pos[threadIdx.x] = pair_to_packed[(size_t)t * K + threadIdx.x];
    s_w[threadIdx.x] = cw[(size_t)t * K + threadIdx.x];
  }
  __syncthreads();
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(xr + i);
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < K; ++k) {
      const int pos = s_pos[k];
      if (pos < 0) continue;
      const uint2 yv = *reinterpret_cast<const uint2*>(yp + (size_t)pos * H + i);
      const float ww = s_w[k];
      d.x = fmaf(ww, bf16_lo(yv.x), d.x); d.y = fmaf(ww, bf16_hi(yv.x), d.y);
      d.z = fmaf(ww, bf16_lo(yv.y), d.z); d.w = fmaf(ww, bf16_hi(yv.y), d.w);
    }
    v.x += d.x * delta_scale; v.y += d.y * delta_scale; v.z += d.z * delta_scale; v.w += d.w * delta_scale;
    *reinterpret_cast<float4*>(xr + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / H + eps);
  }
  __syncthreads();
  const float inv = red[0];
  if (!out) return;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    float4 g = *reinterpret_cast<const float4*>(w + i);
    if (one_plus_w) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
    *reinterpret_cast<uint2*>(out + (size_t)t * H + i) = make_uint2(pack_bf16(v.x * inv * g.x, v.y * inv * g.y), pack_bf16(v.z * inv * g.z, v.w * inv * g.w));
  }
}

// ------------------------------------------------------------------ qkv_post
struct QkvPostParams {
  const __nv_bfloat16* qkv;   // [T][q_cols + 2*n_kv*hd]
  const float* bias;          // [q_cols + 2*n_kv*hd] or null
  const float* q_norm_w;      // [hd] or null
  const float* k_norm_w;      // [hd] or null
  const int* positions;       // [T]
  const float* rope_cos;      // [max_pos][n_rot/2]
  const float* rope_sin;
  const long long* slot_map;  // [T] slot = block*block_size + offset, <0: do not store
  __nv_bfloat16* q_out;       // [T][n_q][hd]
  __nv_bfloat16* gate_out;    // [T][n_q][hd] when q_gate != 0
  __nv_bfloat16* k_cache;     // [blocks][n_kv][block_size][hd]
  __nv_bfloat16* v_cache;
  float* k_scale;             // non-null: the caches hold int8, one fp32 scale per (block, kv head, token) row
  float* v_scale;
  int T, n_q, n_kv, hd, n_rot, block_size;
  int q_gate;                 // 1: q columns hold per-head [q(hd) | gate(hd)]
  int norm_one_plus_w;
  int v_norm;                 // 1: V rows get a weightless RMS norm (Gemma-4)
  float eps;
  int max_pos;
};

__global__ void __launch_bounds__(128) qkv_post_kernel(const QkvPostParams p) {
  pdl_prologue();
  __shared__ float sh[4][512];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = p.n_q + 2 * p.n_kv;
  const int unit = blockIdx.x * 4 + warp;
  if (unit >= p.T * heads_total) return;
  const int t = unit / heads_total, h = unit % heads_total;
  const int hd = p.hd;
  const int q_stride = p.q_gate ? 2 * hd : hd;
  const int q_cols = p.n_q * q_stride;
  const int row_cols = q_cols + 2 * p.n_kv * hd;
  int kind, hh, col0;   // kind 0 q, 1 k, 2 v
  if (h < p.n_q) { kind = 0; hh = h; col0 = h * q_stride; }
  else if (h < p.n_q + p.n_kv) { kind = 1; hh = h - p.n_q; col0 = q_cols + hh * hd; }
  else { kind = 2; hh = h - p.n_q - p.n_kv; col0 = q_cols + p.n_kv * hd + hh * hd; }
  const __nv_bfloat16* src = p.qkv + (size_t)t * row_cols + col0;
  float* v = sh[warp];
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    float x = __bfloat162float(src[i]);
    if (p.bias) x += p.bias[col0 + i];
    v[i] = x;
    ss += x * x;
  }
  if (kind == 0 && p.q_gate) {
    for (int i = lane; i < hd; i += 32) {
      float g = __bfloat162float(src[hd + i]);
      if (p.bias) g += p.bias[col0 + hd + i];
      p.gate_out[((size_t)t * p.n_q + hh) * hd + i] = __float2bfloat16(g);
    }
  }
  const float* nw = kind == 0 ? p.q_norm_w : (kind == 1 ? p.k_norm_w : nullptr);
  if (nw) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / hd + p.eps);
    for (int i = lane; i < hd; i += 32) v[i] = v[i] * inv * (p.norm_one_plus_w ? 1.f + nw[i] : nw[i]);
  } else if (kind == 2 && p.v_norm) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / hd + p.eps);
    for (int i = lane; i < hd; i += 32) v[i] *= inv;
  }
  __syncwarp();
  if (kind != 2 && p.n_rot > 0) {
    const int half = p.n_rot / 2;
    int pos = p.positions[t];
    pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
    const float* cs = p.rope_cos + (size_t)pos * half;
    const float* sn = p.rope_sin + (size_t)pos * half;
    for (int i = lane; i < half; i += 32) {
      const float a = v[i], b = v[i + half], c = cs[i], s = sn[i];
      v[i] = a * c - b * s;
      v[i + half] = a * s + b * c;
    }
    __syncwarp();
  }
  __nv_bfloat16* dst;
  if (kind == 0) dst = p.q_out + ((size_t)t * p.n_q + hh) * hd;
  else {
    const long long slot = p.slot_map[t];
    if (slot < 0) return;
    const long long blk = slot / p.block_size, off = slot % p.block_size;
    __nv_bfloat16* cache = kind == 1 ? p.k_cache : p.v_cache;
    const long long row = (blk * p.n_kv + hh) * p.block_size + off;
    if (p.k_scale) {          // symmetric int8 per row: scale = max|x| / 127
      float amax = 0.f;
      for (int i = lane; i < hd; i += 32) amax = fmaxf(amax, fabsf(v[i]));
      amax = warp_max(amax);
      const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
      int8_t* d8 = reinterpret_cast<int8_t*>(cache) + row * hd;
      for (int i = lane; i < hd; i += 32) d8[i] = (int8_t)max(-127, min(127, __float2int_rn(v[i] * inv)));
      if (lane == 0) (kind == 1 ? p.k_scale : p.v_scale)[row] = sc;
      return;
    }
    dst = cache + row * hd;
  }
  for (int i = lane; i < hd; i += 32) dst[i] = __float2bfloat16(v[i]);
}

// Prefill form of the same epilogue: one CTA per token.  The token's position, cache slot and rope row are fetched once (the
// rope row into shared memory) and the warps walk the token's heads, a lane holding HD / 32 consecutive elements of a head (one
// vector load) and reaching its rotation partner with one shuffle.  The per-head math is that of qkv_post_kernel; the host picks
// this form for batches of many tokens when n_rot / 2 is a multiple of the lane's element count (every model so far).
template <int HD>
__global__ void __launch_bounds__(128) qkv_post_token_kernel(const QkvPostParams p) {
  constexpr int EPL = HD / 32;                 // elements per lane
  pdl_prologue();
  __shared__ float s_cos[256], s_sin[256];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = p.n_rot / 2;
  if (half > 0) {
    int pos = p.positions[t];
    pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      s_cos[i] = p.rope_cos[(size_t)pos * half + i];
      s_sin[i] = p.rope_sin[(size_t)pos * half + i];
    }
  }
  const long long slot = p.slot_map[t];
  __syncthreads();
  const int heads_total = p.n_q + 2 * p.n_kv;
  const int q_stride = p.q_gate ? 2 * HD : HD;
  const int q_cols = p.n_q * q_stride;
  const int row_cols = q_cols + 2 * p.n_kv * HD;
  const __nv_bfloat16* row = p.qkv + (size_t)t * row_cols;
  const int e0 = lane * EPL;                   // first element of this lane
  const int dl = half / EPL;                   // lane distance to the rotation partner
  for (int h = warp; h < heads_total; h += 4) {
    int kind, hh, col0;                        // kind 0 q, 1 k, 2 v
    if (h < p.n_q) { kind = 0; hh = h; col0 = h * q_stride; }
    else if (h < p.n_q + p.n_kv) { kind = 1; hh = h - p.n_q; col0 = q_cols + hh * HD; }
    else { kind = 2; hh = h - p.n_q - p.n_kv; col0 = q_cols + p.n_kv * HD + hh * HD; }
    if (kind != 0 && slot < 0) continue;       // this token's K/V rows are not stored
    float v[EPL];
    {
      uint32_t raw[EPL / 2];
      if constexpr (EPL == 2) raw[0] = *reinterpret_cast<const uint32_t*>(row + col0 + e0);
      else if constexpr (EPL == 4) { const uint2 r2 = *reinterpret_cast<const uint2*>(row + col0 + e0); raw[0] = r2.x; raw[1] = r2.y; }
      else {
#pragma unroll
        for (int c = 0; c < EPL / 8; ++c) {
          const uint4 r4 = *reinterpret_cast<const uint4*>(row + col0 + e0 + 8 * c);
          raw[4 * c] = r4.x; raw[4 * c + 1] = r4.y; raw[4 * c + 2] = r4.z; raw[4 * c + 3] = r4.w;
        }
      }
#pragma unroll
      for (int j = 0; j < EPL / 2; ++j) { v[2 * j] = bf16_lo(raw[j]); v[2 * j + 1] = bf16_hi(raw[j]); }
    }
    if (p.bias) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] += p.bias[col0 + e0 + j];
    }
    if (kind == 0 && p.q_gate) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        float g = __bfloat162float(row[col0 + HD + e0 + j]);
        if (p.bias) g += p.bias[col0 + HD + e0 + j];
        p.gate_out[((size_t)t * p.n_q + hh) * HD + e0 + j] = __float2bfloat16(g);
      }
    }
    const float* nw = kind == 0 ? p.q_norm_w : (kind == 1 ? p.k_norm_w : nullptr);
    if (nw || (kind == 2 && p.v_norm)) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
      const float inv = rsqrtf(warp_sum(ss) / HD + p.eps);
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] *= nw ? inv * (p.norm_one_plus_w ? 1.f + nw[e0 + j] : nw[e0 + j]) : inv;
    }
    if (kind != 2 && half > 0) {
      const bool lo = e0 < half, in = e0 < p.n_rot;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], dl);
        if (in) {
          const int f = (lo ? e0 : e0 - half) + j;
          v[j] = lo ? v[j] * s_cos[f] - other * s_sin[f] : other * s_sin[f] + v[j] * s_cos[f];
        }
      }
    }
    if (kind == 0) {
      __nv_bfloat16* dst = p.q_out + ((size_t)t * p.n_q + hh) * HD + e0;
#pragma unroll
      for (int j = 0; j < EPL; j += 2) *reinterpret_cast<uint32_t*>(dst + j) = pack_bf16(v[j], v[j + 1]);
      continue;
    }
    const long long blk = slot / p.block_size, off = slot % p.block_size;
    const long long crow = (blk * p.n_kv + hh) * p.block_size + off;
    __nv_bfloat16* cache = kind == 1 ? p.k_cache : p.v_cache;
    if (p.k_scale) {          // symmetric int8 per row: scale = max|x| / 127
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) amax = fmaxf(amax, fabsf(v[j]));
      amax = warp_max(amax);
      const float sc = amax > 0.f ? amax / 127.f : 1.f, inv = 1.f / sc;
      int8_t* d8 = reinterpret_cast<int8_t*>(cache) + crow * HD + e0;
#pragma unroll
      for (int j = 0; j < EPL; ++j) d8[j] = (int8_t)max(-127, min(127, __float2int_rn(v[j] * inv)));
      if (lane == 0) (kind == 1 ? p.k_scale : p.v_scale)[crow] = sc;
    } else {
      __nv_bfloat16* dst = cache + crow * HD + e0;
#pragma unroll
      for (int j = 0; j < EPL; j += 2) *reinterpret_cast<uint32_t*>(dst + j) = pack_bf16(v[j], v[j + 1]);
    }
  }
}

// ------------------------------------------------------------------ GLU over interleaved-16 columns
__device__ __forceinline__ float glu_act(int act, float g, float u, float alpha, float limit) {
  if (act == 1) return g / (1.f + __expf(-g)) * u;
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t) * u;
}
__global__ void glu_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long total_out, int F, int act,
                           float alpha, float limit) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_out) return;
  const long long t = i / F;
  const int f = (int)(i % F);
  const __nv_bfloat16* row = in + t * 2 * F;
  const int g = 32 * (f >> 4) + (f & 15);
  out[i] = __float2bfloat16(glu_act(act, __bfloat162float(row[g]), __bfloat162float(row[g + 16]), alpha, limit));
}

// y[i] = x[i] * sigmoid(g[i])   (gated attention output, shared-expert gate uses the scalar form below)
__global__ void sigmoid_mul_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ y, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16(__bfloat162float(x[i]) / (1.f + __expf(-__bfloat162float(g[i]))));
}
// out[t][:] (fp32) += scale_t * src[t][:], scale_t = sigmoid(gate_logit[t]) if gate_logit else 1
__global__ void scaled_add_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ src, const float* __restrict__ gate_logit, int H, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = gate_logit ? 1.f / (1.f + __expf(-gate_logit[i / H])) : 1.f;
  out[i] += s * __bfloat162float(src[i]);
}
__global__ void cast_f32_bf16_kernel(const float* __restrict__ a, __nv_bfloat16* __restrict__ b, long long n) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) b[i] = __float2bfloat16(a[i]);
}

// y[t,h,:] = w * x / rms(x) * silu(z)  over head_dim (one warp per (t,h))
__global__ void __launch_bounds__(128) gated_rmsnorm_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ z, const float* __restrict__ w,
                                                            __nv_bfloat16* __restrict__ y, int rows, int hd, float eps) {
  pdl_prologue();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* xr = x + (size_t)r * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) ss += xr[i] * xr[i];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / hd + eps);
  for (int i = lane; i < hd; i += 32) {
    const float zz = __bfloat162float(z[(size_t)r * hd + i]);
    y[(size_t)r * hd + i] = __float2bfloat16(xr[i] * inv * w[i] * (zz / (1.f + __expf(-zz))));
  }
}

// Decoder probe: every 32-bit word of `in` (eight E2M1 codes) is decoded twice, with the byte-permute
// table path (bf16) and with the hardware conversion path (fp16); out[w][0..7] and out[w][8..15].
__global__ void e2m1_probe_kernel(const uint32_t* __restrict__ in, float* __restrict__ out, int n) {
  pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t a[4], b[4];
  e2m1x8_to_bf16x2(in[i], a);
  e2m1x8_to_f16x2(in[i], b);
  for (int j = 0; j < 4; ++j) {
    out[(size_t)i * 16 + 2 * j] = bf16_lo(a[j]);
    out[(size_t)i * 16 + 2 * j + 1] = bf16_hi(a[j]);
    const __half2 h = *reinterpret_cast<const __half2*>(&b[j]);
    out[(size_t)i * 16 + 8 + 2 * j] = __low2float(h);
    out[(size_t)i * 16 + 8 + 2 * j + 1] = __high2float(h);
  }
}

}  // namespace mx

using namespace mx;

MX_HOST_API int mx_e2m1_probe(const void* in, float* out, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  launch_pdl(e2m1_probe_kernel, dim3((n + 127) / 128), dim3(128), 0, st, (const uint32_t*)in, out, n);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_embed(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const int* ids, float* out, int T,
                         int H, int vocab, float scale, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 32) return -102;
  WeightRef w{w0, w1, w2, w3};
  const int threads = 128;
  switch (wfmt) {
    case WF_BF16: launch_pdl(embed_kernel<WF_BF16>, dim3(T), dim3(threads), 0, st, w, ids, out, H, vocab, scale); break;
    case WF_Q8: launch_pdl(embed_kernel<WF_Q8>, dim3(T), dim3(threads), 0, st, w, ids, out, H, vocab, scale); break;
    case WF_Q4K: launch_pdl(embed_kernel<WF_Q4K>, dim3(T), dim3(threads), 0, st, w, ids, out, H, vocab, scale); break;
    case WF_Q6K: launch_pdl(embed_kernel<WF_Q6K>, dim3(T), dim3(threads), 0, st, w, ids, out, H, vocab, scale); break;
    case WF_MXFP4: launch_pdl(embed_kernel<WF_MXFP4>, dim3(T), dim3(threads), 0, st, w, ids, out, H, vocab, scale); break;
    default: return -100;
  }
  return (int)cudaGetLastError();
}

// delta_is_f32: 0 -> bf16 delta, 1 -> fp32 delta.  write_x: store x+delta back into x.
MX_HOST_API int mx_rmsnorm(float* x, const void* delta, int delta_is_f32, const float* dbias, const float* w, void* out_bf16, float eps,
                           int T, int H, int one_plus_w, float delta_scale, int write_x, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 4) return -107;
  if (delta_is_f32) launch_pdl(rmsnorm_kernel<float>, dim3(T), dim3(256), 0, st, x, (const float*)delta, dbias, w, (__nv_bfloat16*)out_bf16, eps, H, one_plus_w, delta_scale, write_x);
  else launch_pdl(rmsnorm_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, x, (const __nv_bfloat16*)delta, dbias, w, (__nv_bfloat16*)out_bf16, eps, H, one_plus_w, delta_scale, write_x);
  return (int)cudaGetLastError();
}

// x[t] += delta_scale * sum_k cw[t,k] * yp[pair_to_packed[t*K+k]];  out = rmsnorm(x) * w   (K <= 32)
MX_HOST_API int mx_rmsnorm_combine(float* x, const void* yp, const int* pair_to_packed, const float* cw, int K, const float* w, void* out_bf16,
                                   float eps, int T, int H, int one_plus_w, float delta_scale, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 4 || K > 32 || K < 1) return -107;
  launch_pdl(rmsnorm_combine_kernel, dim3(T), dim3(256), 0, st, x, (const __nv_bfloat16*)yp, pair_to_packed, cw, K, w, (__nv_bfloat16*)out_bf16, eps, H,
             one_plus_w, delta_scale);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_qkv_post_kv8(const void* qkv, const float* bias, const float* q_norm_w, const float* k_norm_w, const int* positions,
                                const float* rope_cos, const float* rope_sin, const long long* slot_map, void* q_out, void* gate_out,
                                void* k_cache, void* v_cache, float* k_scale, float* v_scale, int T, int n_q, int n_kv, int hd, int n_rot,
                                int block_size, int q_gate, int norm_one_plus_w, float eps, int max_pos, cudaStream_t st);

MX_HOST_API int mx_qkv_post(const void* qkv, const float* bias, const float* q_norm_w, const float* k_norm_w, const int* positions,
                            const float* rope_cos, const float* rope_sin, const long long* slot_map, void* q_out, void* gate_out,
                            void* k_cache, void* v_cache, int T, int n_q, int n_kv, int hd, int n_rot, int block_size, int q_gate,
                            int norm_one_plus_w, float eps, int max_pos, cudaStream_t st) {
  return mx_qkv_post_kv8(qkv, bias, q_norm_w, k_norm_w, positions, rope_cos, rope_sin, slot_map, q_out, gate_out, k_cache, v_cache, nullptr,
                         nullptr, T, n_q, n_kv, hd, n_rot, block_size, q_gate, norm_one_plus_w, eps, max_pos, st);
}

// k_scale / v_scale non-null: k_cache / v_cache are int8 [blocks][n_kv][block_size][hd] and the rows are quantised on the way in.
MX_HOST_API int mx_qkv_post_kv8(const void* qkv, const float* bias, const float* q_norm_w, const float* k_norm_w, const int* positions,
                                const float* rope_cos, const float* rope_sin, const long long* slot_map, void* q_out, void* gate_out,
                                void* k_cache, void* v_cache, float* k_scale, float* v_scale, int T, int n_q, int n_kv, int hd, int n_rot,
                                int block_size, int q_gate, int norm_one_plus_w, float eps, int max_pos, cudaStream_t st) {
  if (T <= 0) return 0;
  if (hd > 512) return -108;
  QkvPostParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.bias = bias; p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.positions = positions;
  p.rope_cos = rope_cos; p.rope_sin = rope_sin; p.slot_map = slot_map; p.q_out = (__nv_bfloat16*)q_out; p.gate_out = (__nv_bfloat16*)gate_out;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.k_scale = k_scale; p.v_scale = k_scale ? v_scale : nullptr;
  p.T = T; p.n_q = n_q; p.n_kv = n_kv; p.hd = hd; p.n_rot = n_rot; p.block_size = block_size; p.q_gate = q_gate & 1;
  p.v_norm = (q_gate >> 1) & 1;           // flag word: bit 0 = q columns carry a gate, bit 1 = weightless RMS norm on V
  p.norm_one_plus_w = norm_one_plus_w; p.eps = eps; p.max_pos = max_pos;
  const int half = n_rot / 2, epl = hd / 32;
  const int row_cols = n_q * (p.q_gate ? 2 * hd : hd) + 2 * n_kv * hd;
  // many tokens: the token-major form (vector loads need the row start and every head start on an element-count boundary)
  if (T >= 64 && (hd == 64 || hd == 128 || hd == 256 || hd == 512) && half <= 256 && half % epl == 0 && ((half / epl) & (half / epl - 1)) == 0 &&
      n_rot <= hd && row_cols % 8 == 0 && ((uintptr_t)qkv & 15) == 0) {
    switch (hd) {
      case 64: launch_pdl(qkv_post_token_kernel<64>, dim3(T), dim3(128), 0, st, p); break;
      case 128: launch_pdl(qkv_post_token_kernel<128>, dim3(T), dim3(128), 0, st, p); break;
      case 256: launch_pdl(qkv_post_token_kernel<256>, dim3(T), dim3(128), 0, st, p); break;
      default: launch_pdl(qkv_post_token_kernel<512>, dim3(T), dim3(128), 0, st, p); break;
    }
    return (int)cudaGetLastError();
  }
  const int units = T * (n_q + 2 * n_kv);
  launch_pdl(qkv_post_kernel, dim3((units + 3) / 4), dim3(128), 0, st, p);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_glu(const void* in, void* out, long long T, int F, int act, float alpha, float limit, cudaStream_t st) {
  const long long total = T * F;
  if (total <= 0) return 0;
  if (F % 16) return -104;
  launch_pdl(glu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, F, act, alpha, limit);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_sigmoid_mul(const void* x, const void* g, void* y, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  launch_pdl(sigmoid_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (__nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_scaled_add(float* out, const void* src, const float* gate_logit, int H, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  launch_pdl(scaled_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, out, (const __nv_bfloat16*)src, gate_logit, H, n);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_cast_f32_bf16(const float* a, void* b, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  launch_pdl(cast_f32_bf16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, a, (__nv_bfloat16*)b, n);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_gated_rmsnorm(const float* x, const void* z, const float* w, void* y, int rows, int hd, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  launch_pdl(gated_rmsnorm_kernel, dim3((rows + 3) / 4), dim3(128), 0, st, x, (const __nv_bfloat16*)z, w, (__nv_bfloat16*)y, rows, hd, eps);
  return (int)cudaGetLastError();
}
