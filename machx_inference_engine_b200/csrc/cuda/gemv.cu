// Decode-time GEMV family: y[m][n] = sum_k W[n][k] * x[m][k] (+bias), weights decoded in registers
// from the runtime layouts (bf16 / Q8 / Q4_K / Q6_K planes / MXFP4 planes), 16-byte loads only.
//
//   dense mode : up to 8 activation rows share every decoded weight (T<=8: decode and MTP verify)
//   expert mode: blockIdx.y selects a slot; slot -> expert id (device array) selects the weight slab
//                and slot / x_div selects the activation row (MoE decode: gate/up and down GEMVs)
//
// A warp owns ROWS consecutive output rows; lanes stride over 32-element k-blocks, so each
// weight byte is read exactly once and the activation chunk is reused across the warp's rows.
// Optional fused epilogue: bias, gated activation over 16-row interleaved gate/up pairs.
//
// Reference parity: src/ops/gemv_q4k.cpp:72, gemv_q8dot.cpp:276-680, gemv_q6k.cpp:76-670,
// gemv_mxfp4.cpp:94-323, gemv_fp16.cpp:64 and the batched-T verify kernels gemv_q8dot.cpp:391,499;
// MoE decode pair moe_fused.cpp:101-541.
#include "common.cuh"
#include "comm.cuh"
#include "dequant.cuh"
#include "host_util.h"

namespace mx {

constexpr int GEMV_WARPS = 4;
constexpr int GEMV_ROWS = 4;     // rows per warp
constexpr int GEMV_MAX_M = 8;

struct GemvParams {
  WeightRef w;
  const __nv_bfloat16* x;   // [M][K]
  void* y;                  // [M or slots][N_out]
  const float* bias;        // [N] or [E][N]
  const int* slot_expert;   // expert mode: [slots]
  const float* slot_scale;  // expert mode: optional per-slot multiplier on the output
  int x_div;                // expert mode: activation row = slot / x_div
  int e_lo, e_hi;           // expert mode: experts owned by this rank (weights hold [e_lo, e_hi)); other slots yield zeros
  int M, N, K;
  int out_f32;
  int act;                  // 0 none, 1 swiglu, 2 swiglu_oai, 3 geglu (16-row interleaved gate/up)
  float act_alpha, act_limit;
  PeerOut peer;             // world > 0: fp32 partials go to every rank's inbox instead of y (fused all-reduce)
};

__device__ __forceinline__ float gemv_act(int act, float g, float u, float alpha, float limit) {
  if (act == 1) return g / (1.f + __expf(-g)) * u;
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t) * u;
}

template <int FMT, int MM>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_kernel(const GemvParams p) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS;
  const int next_seq = p.peer.world ? *p.peer.seq + 1 : 0;
  if (n0 < p.N) {
  const int slot = blockIdx.y;
  WeightRef w = p.w;
  const __nv_bfloat16* x = p.x;
  const float* bias = p.bias;
  bool owned = true;
  if (p.slot_expert) {
    const int e = p.slot_expert[slot];
    owned = e >= p.e_lo && e < p.e_hi;
    const int el = owned ? e - p.e_lo : 0;
    w = expert_weight<FMT>(p.w, el, p.N, p.K);
    x += (size_t)(slot / p.x_div) * p.K;
    if (bias) bias += (size_t)el * p.N;
  }
  float acc[GEMV_ROWS][MM];
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;

  RowPtrs rp[GEMV_ROWS];
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r) rp[r] = row_ptrs<FMT>(w, min(n0 + r, p.N - 1), p.K);

  const int nkb = owned ? p.K / 32 : 0;       // slots routed to another rank's expert contribute zeros
  for (int kb = lane; kb < nkb; kb += 32) {
    float wv[32];
    if (MM == 1) {
      // keep x in registers, stream the rows
      float xv[32];
      const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)kb * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(xp + i);
        xv[8 * i + 0] = bf16_lo(v.x); xv[8 * i + 1] = bf16_hi(v.x); xv[8 * i + 2] = bf16_lo(v.y); xv[8 * i + 3] = bf16_hi(v.y);
        xv[8 * i + 4] = bf16_lo(v.z); xv[8 * i + 5] = bf16_hi(v.z); xv[8 * i + 6] = bf16_lo(v.w); xv[8 * i + 7] = bf16_hi(v.w);
      }
#pragma unroll
      for (int r = 0; r < GEMV_ROWS; ++r) {
        decode32_f32<FMT>(rp[r], kb, wv);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) s = fmaf(wv[i], xv[i], s);
        acc[r][0] += s;
      }
    } else {
#pragma unroll
      for (int r = 0; r < GEMV_ROWS; ++r) {
        decode32_f32<FMT>(rp[r], kb, wv);
#pragma unroll
        for (int m = 0; m < MM; ++m) {
          if (m < p.M) {
            const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * p.K + (size_t)kb * 32);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 v = __ldg(xp + i);
              s = fmaf(wv[8 * i + 0], bf16_lo(v.x), s); s = fmaf(wv[8 * i + 1], bf16_hi(v.x), s);
              s = fmaf(wv[8 * i + 2], bf16_lo(v.y), s); s = fmaf(wv[8 * i + 3], bf16_hi(v.y), s);
              s = fmaf(wv[8 * i + 4], bf16_lo(v.z), s); s = fmaf(wv[8 * i + 5], bf16_hi(v.z), s);
              s = fmaf(wv[8 * i + 6], bf16_lo(v.w), s); s = fmaf(wv[8 * i + 7], bf16_hi(v.w), s);
            }
            acc[r][m] += s;
          }
        }
      }
    }
  }
  if (FMT == WF_BF16 && (p.K & 31) && owned) {
    // ragged tail of a bf16 row (K % 32 != 0): one element per lane
    const int k = nkb * 32 + lane;
    if (k < p.K) {
#pragma unroll
      for (int r = 0; r < GEMV_ROWS; ++r) {
        const float wv1 = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rp[r].p0)[k]);
#pragma unroll
        for (int m = 0; m < MM; ++m)
          if (m < p.M) acc[r][m] = fmaf(wv1, __bfloat162float(x[(size_t)m * p.K + k]), acc[r][m]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[r][m] = warp_sum(acc[r][m]);

  if (lane == 0) {
  const float oscale = p.slot_scale ? p.slot_scale[slot] : 1.f;
  const int rows_out = p.slot_expert ? 1 : p.M;
#pragma unroll
  for (int m = 0; m < MM; ++m) {
    if (m >= rows_out) break;
    const size_t orow = p.slot_expert ? (size_t)slot : (size_t)m;
    if (p.act == 0) {
      for (int r = 0; r < GEMV_ROWS && n0 + r < p.N; ++r) {
        const float v = owned ? (acc[r][m] + (bias ? bias[n0 + r] : 0.f)) * oscale : 0.f;
        if (p.peer.world) {
          // fused all-reduce: the partial goes to slot [my_rank] of every rank's inbox
          for (int d = 0; d < p.peer.world; ++d) reinterpret_cast<float*>(peer_slot(p.peer, d, next_seq))[orow * p.N + n0 + r] = v;
        } else if (p.out_f32) ((float*)p.y)[orow * p.N + n0 + r] = v;
        else ((__nv_bfloat16*)p.y)[orow * p.N + n0 + r] = __float2bfloat16(v);
      }
    }
  }
  }
  }
  if (p.peer.world) peer_publish(p.peer, next_seq);
}

// Gated variant: a warp owns output features f0..f0+3 and reads the matching gate rows
// (16-row interleave: feature f lives at row 32*(f/16) + f%16, its up row 16 further).
template <int FMT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_gated_kernel(const GemvParams p) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int F = p.N / 2;
  const int f0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS;
  if (f0 >= F) return;
  const int slot = blockIdx.y;
  WeightRef w = p.w;
  const __nv_bfloat16* x = p.x + (size_t)(p.slot_expert ? slot / p.x_div : slot) * p.K;
  const float* bias = p.bias;
  bool owned = true;
  if (p.slot_expert) {
    const int e = p.slot_expert[slot];
    owned = e >= p.e_lo && e < p.e_hi;
    const int el = owned ? e - p.e_lo : 0;
    w = expert_weight<FMT>(p.w, el, p.N, p.K);
    if (bias) bias += (size_t)el * p.N;
  }
  float ag[GEMV_ROWS], au[GEMV_ROWS];
  RowPtrs rg[GEMV_ROWS], ru[GEMV_ROWS];
  int grow[GEMV_ROWS];
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r) {
    const int f = min(f0 + r, F - 1);
    grow[r] = 32 * (f >> 4) + (f & 15);
    rg[r] = row_ptrs<FMT>(w, grow[r], p.K);
    ru[r] = row_ptrs<FMT>(w, grow[r] + 16, p.K);
    ag[r] = au[r] = 0.f;
  }
  const int nkb = owned ? p.K / 32 : 0;
  for (int kb = lane; kb < nkb; kb += 32) {
    float xv[32], wv[32];
    const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)kb * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(xp + i);
      xv[8 * i + 0] = bf16_lo(v.x); xv[8 * i + 1] = bf16_hi(v.x); xv[8 * i + 2] = bf16_lo(v.y); xv[8 * i + 3] = bf16_hi(v.y);
      xv[8 * i + 4] = bf16_lo(v.z); xv[8 * i + 5] = bf16_hi(v.z); xv[8 * i + 6] = bf16_lo(v.w); xv[8 * i + 7] = bf16_hi(v.w);
    }
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      decode32_f32<FMT>(rg[r], kb, wv);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) s = fmaf(wv[i], xv[i], s);
      ag[r] += s;
      decode32_f32<FMT>(ru[r], kb, wv);
      s = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) s = fmaf(wv[i], xv[i], s);
      au[r] += s;
    }
  }
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r) { ag[r] = warp_sum(ag[r]); au[r] = warp_sum(au[r]); }
  if (lane != 0) return;
  for (int r = 0; r < GEMV_ROWS && f0 + r < F; ++r) {
    const float g = ag[r] + (bias ? bias[grow[r]] : 0.f), u = au[r] + (bias ? bias[grow[r] + 16] : 0.f);
    const float v = owned ? gemv_act(p.act, g, u, p.act_alpha, p.act_limit) : 0.f;
    if (p.out_f32) ((float*)p.y)[(size_t)slot * F + f0 + r] = v;
    else ((__nv_bfloat16*)p.y)[(size_t)slot * F + f0 + r] = __float2bfloat16(v);
  }
}

// Batched-decode MoE GEMV: blockIdx.y is a local expert; its weights are streamed once and multiplied with every row of
// the compact packing that was routed to it (GRP_MM rows per pass; more rows take further passes).  A warp owns four weight
// rows: four outputs in plain mode, or the gate and up rows of two features in gated mode.
constexpr int GRP_MM = 8;

struct GroupParams {
  WeightRef w;
  const __nv_bfloat16* x;    // rows addressed through x_index (gate|up: token rows in place) or by packed position (down)
  const int* x_index;        // [packed rows] or null
  __nv_bfloat16* y;          // [packed rows][N_out]
  const float* bias;         // [E_local][N] or null
  const int* counts;         // [E] rows per expert
  const int* seg_start;      // [E+1] first packed row of each expert
  int e_lo, N, K, act;
  float act_alpha, act_limit;
};

template <int FMT, bool GATED>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_group_kernel(const GroupParams p) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int el = blockIdx.y, e = p.e_lo + el;
  const int cnt = p.counts[e];
  if (cnt == 0) return;
  const int start = p.seg_start[e];
  const int unit = blockIdx.x * GEMV_WARPS + warp;          // plain: 4 consecutive rows; gated: 2 consecutive features
  const int F = p.N / 2;
  int rows[4];
  if (GATED) {
    const int f0 = unit * 2;
    if (f0 >= F) return;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int f = min(f0 + j, F - 1);
      rows[j] = 32 * (f >> 4) + (f & 15);
      rows[2 + j] = rows[j] + 16;
    }
  } else {
    if (unit * 4 >= p.N) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) rows[j] = min(unit * 4 + j, p.N - 1);
  }
  const WeightRef w = expert_weight<FMT>(p.w, el, p.N, p.K);
  const float* bias = p.bias ? p.bias + (size_t)el * p.N : nullptr;
  RowPtrs rp[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) rp[r] = row_ptrs<FMT>(w, rows[r], p.K);
  const int nkb = p.K / 32;
  for (int pass = 0; pass < cnt; pass += GRP_MM) {
    const int mc = min(GRP_MM, cnt - pass);
    const __nv_bfloat16* xr[GRP_MM];
#pragma unroll
    for (int m = 0; m < GRP_MM; ++m) {
      const int pr = start + pass + min(m, mc - 1);
      xr[m] = p.x + (size_t)(p.x_index ? p.x_index[pr] : pr) * p.K;
    }
    float acc[4][GRP_MM];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int m = 0; m < GRP_MM; ++m) acc[r][m] = 0.f;
    for (int kb = lane; kb < nkb; kb += 32) {
      float wv[4][32];
#pragma unroll
      for (int r = 0; r < 4; ++r) decode32_f32<FMT>(rp[r], kb, wv[r]);
#pragma unroll
      for (int m = 0; m < GRP_MM; ++m) {
        if (m < mc) {
          const uint4* xp = reinterpret_cast<const uint4*>(xr[m] + (size_t)kb * 32);
          float xv[32];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 v = __ldg(xp + i);
            xv[8 * i + 0] = bf16_lo(v.x); xv[8 * i + 1] = bf16_hi(v.x); xv[8 * i + 2] = bf16_lo(v.y); xv[8 * i + 3] = bf16_hi(v.y);
            xv[8 * i + 4] = bf16_lo(v.z); xv[8 * i + 5] = bf16_hi(v.z); xv[8 * i + 6] = bf16_lo(v.w); xv[8 * i + 7] = bf16_hi(v.w);
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) s = fmaf(wv[r][i], xv[i], s);
            acc[r][m] += s;
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int m = 0; m < GRP_MM; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < GRP_MM; ++m) {
        if (m >= mc) break;
        const size_t orow = (size_t)(start + pass + m);
        if (GATED) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int f = unit * 2 + j;
            if (f >= F) break;
            const float g = acc[j][m] + (bias ? bias[rows[j]] : 0.f), u = acc[2 + j][m] + (bias ? bias[rows[2 + j]] : 0.f);
            p.y[orow * F + f] = __float2bfloat16(gemv_act(p.act, g, u, p.act_alpha, p.act_limit));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = unit * 4 + j;
            if (n >= p.N) break;
            p.y[orow * p.N + n] = __float2bfloat16(acc[j][m] + (bias ? bias[n] : 0.f));
          }
        }
      }
    }
  }
}

template <int FMT>
static int launch_group(const GroupParams& p, int n_experts, cudaStream_t st) {
  if (p.act != 0) {
    const int units = (p.N / 2 + 1) / 2;
    launch_pdl(gemv_group_kernel<FMT, true>, dim3(dim3((units + GEMV_WARPS - 1) / GEMV_WARPS, n_experts)), dim3(GEMV_WARPS * 32), 0, st, p);
  } else {
    const int units = (p.N + 3) / 4;
    launch_pdl(gemv_group_kernel<FMT, false>, dim3(dim3((units + GEMV_WARPS - 1) / GEMV_WARPS, n_experts)), dim3(GEMV_WARPS * 32), 0, st, p);
  }
  return (int)cudaGetLastError();
}

template <int FMT>
static int launch_gemv(const GemvParams& p, int slots, cudaStream_t st) {
  if (p.act != 0) {
    const int F = p.N / 2;
    dim3 grid((F + GEMV_WARPS * GEMV_ROWS - 1) / (GEMV_WARPS * GEMV_ROWS), slots);
    launch_pdl(gemv_gated_kernel<FMT>, dim3(grid), dim3(GEMV_WARPS * 32), 0, st, p);
    return (int)cudaGetLastError();
  }
  dim3 grid((p.N + GEMV_WARPS * GEMV_ROWS - 1) / (GEMV_WARPS * GEMV_ROWS), p.slot_expert ? slots : 1);
  if (p.slot_expert || p.M == 1) launch_pdl(gemv_kernel<FMT, 1>, dim3(grid), dim3(GEMV_WARPS * 32), 0, st, p);
  else if (p.M <= 4) launch_pdl(gemv_kernel<FMT, 4>, dim3(grid), dim3(GEMV_WARPS * 32), 0, st, p);
  else launch_pdl(gemv_kernel<FMT, 8>, dim3(grid), dim3(GEMV_WARPS * 32), 0, st, p);
  return (int)cudaGetLastError();
}

}  // namespace mx

// Whole-matrix decode to bf16 (one thread per 32-element block).  Prefill chunks of a quantised dense layer decode the weight
// once into a scratch matrix and run the TMA-fed bf16 GEMM on it: the in-kernel decode of the tensor-core GEMM repeats for every
// 128-row tile of activations and bounds it near 460 TFLOP/s, the bf16 kernel runs at about 1100.
namespace mx {
template <int FMT>
__global__ void __launch_bounds__(256) dequant_bf16_kernel(WeightRef w, long long N, int K, __nv_bfloat16* __restrict__ out) {
  pdl_prologue();
  const int kbs = K / 32;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * kbs) return;
  const long long n = i / kbs;
  const int kb = (int)(i - n * kbs);
  const RowPtrs rp = row_ptrs<FMT>(w, n, K);
  float v[32];
  decode32_f32<FMT>(rp, kb, v);
  uint4* o = reinterpret_cast<uint4*>(out + n * K + (long long)kb * 32);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = make_uint4(pack_bf16(v[8 * j], v[8 * j + 1]), pack_bf16(v[8 * j + 2], v[8 * j + 3]), pack_bf16(v[8 * j + 4], v[8 * j + 5]),
                      pack_bf16(v[8 * j + 6], v[8 * j + 7]));
}
}  // namespace mx

MX_HOST_API int mx_dequant_bf16(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, long long N, int K, void* out,
                                cudaStream_t st) {
  using namespace mx;
  if (N <= 0 || K <= 0) return 0;
  if (K % 32 || ((wfmt == WF_Q4K || wfmt == WF_Q6K) && K % 256)) return -103;
  const long long blocks = N * (K / 32);
  const unsigned grid = (unsigned)((blocks + 255) / 256);
  const WeightRef w{w0, w1, w2, w3};
  switch (wfmt) {
    case WF_Q8: launch_pdl(dequant_bf16_kernel<WF_Q8>, dim3(grid), dim3(256), 0, st, w, N, K, (__nv_bfloat16*)out); break;
    case WF_Q4K: launch_pdl(dequant_bf16_kernel<WF_Q4K>, dim3(grid), dim3(256), 0, st, w, N, K, (__nv_bfloat16*)out); break;
    case WF_Q6K: launch_pdl(dequant_bf16_kernel<WF_Q6K>, dim3(grid), dim3(256), 0, st, w, N, K, (__nv_bfloat16*)out); break;
    case WF_MXFP4: launch_pdl(dequant_bf16_kernel<WF_MXFP4>, dim3(grid), dim3(256), 0, st, w, N, K, (__nv_bfloat16*)out); break;
    default: return -100;
  }
  return (int)cudaGetLastError();
}

// Dense: y[M][N] from x[M][K], M <= 8.   Expert: y[slots][N] with slot_expert != null.
// With act != 0 the weight holds interleaved gate/up rows (N = 2F) and y is [rows][F]; in that
// mode every activation row is a "slot" (dense callers pass slots = M and slot_expert = null).
static int gemv_impl(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, void* y,
                     const float* bias, int M, int N, int K, int out_f32, int act, float act_alpha, float act_limit,
                     const int* slot_expert, const float* slot_scale, int slots, int x_div, const mx::PeerOut* peer, cudaStream_t stream);

MX_HOST_API int mx_gemv(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, void* y,
                        const float* bias, int M, int N, int K, int out_f32, int act, float act_alpha, float act_limit,
                        const int* slot_expert, const float* slot_scale, int slots, int x_div, cudaStream_t stream) {
  return gemv_impl(wfmt, w0, w1, w2, w3, x, y, bias, M, N, K, out_f32, act, act_alpha, act_limit, slot_expert, slot_scale, slots, x_div, nullptr, stream);
}

// Expert-major GEMV over a compact packing (see gemv_group_kernel).  counts / seg_start are indexed by global expert id.
MX_HOST_API int mx_gemv_group(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, const int* x_index, void* y,
                              const float* bias, int N, int K, int act, float act_alpha, float act_limit, const int* counts, const int* seg_start,
                              int e_lo, int n_experts, cudaStream_t stream) {
  using namespace mx;
  if (N <= 0 || K <= 0 || n_experts <= 0) return 0;
  if (K % 32) return -102;
  if ((wfmt == WF_Q4K || wfmt == WF_Q6K) && (K % 256)) return -103;
  if (act != 0 && (N % 32)) return -104;
  GroupParams p;
  p.w = WeightRef{w0, w1, w2, w3}; p.x = (const __nv_bfloat16*)x; p.x_index = x_index; p.y = (__nv_bfloat16*)y; p.bias = bias;
  p.counts = counts; p.seg_start = seg_start; p.e_lo = e_lo; p.N = N; p.K = K; p.act = act; p.act_alpha = act_alpha; p.act_limit = act_limit;
  switch (wfmt) {
    case WF_BF16: return launch_group<WF_BF16>(p, n_experts, stream);
    case WF_Q8: return launch_group<WF_Q8>(p, n_experts, stream);
    case WF_Q4K: return launch_group<WF_Q4K>(p, n_experts, stream);
    case WF_Q6K: return launch_group<WF_Q6K>(p, n_experts, stream);
    case WF_MXFP4: return launch_group<WF_MXFP4>(p, n_experts, stream);
    default: return -100;
  }
}

static int g_e_lo = 0, g_e_hi = 1 << 30;
// Expert-parallel variant of the expert mode: the weight stack holds experts [e_lo, e_hi) only.
MX_HOST_API int mx_gemv_experts(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, void* y,
                                const float* bias, int N, int K, int out_f32, int act, float act_alpha, float act_limit,
                                const int* slot_expert, const float* slot_scale, int slots, int x_div, int e_lo, int e_hi, cudaStream_t stream) {
  g_e_lo = e_lo; g_e_hi = e_hi;
  const int rc = gemv_impl(wfmt, w0, w1, w2, w3, x, y, bias, 1, N, K, out_f32, act, act_alpha, act_limit, slot_expert, slot_scale, slots, x_div, nullptr, stream);
  g_e_lo = 0; g_e_hi = 1 << 30;
  return rc;
}

namespace mx {
PeerOut make_peer_out(const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket);
int gemv_stream_try(int wfmt, const WeightRef& w, const void* x, void* y, const float* bias, int M, int N, int K, int out_f32, int act,
                    float act_alpha, float act_limit, const int* slot_expert, const float* slot_scale, int slots, int x_div, int e_lo,
                    int e_hi, const PeerOut* peer, cudaStream_t st);
}
// 0: pick per case (the streaming kernel where it measured faster: bf16, Q8, Q4_K and Q6_K matrices and the gated MXFP4 expert GEMV),
// 1: register-streamed kernels only, 2: streaming kernel wherever it applies (tests, A/B timing)
static int g_gemv_path = 0;
// Q4_K / Q6_K rows shorter than this leave most lanes of the streaming kernel without a 64-element granule
static int g_kq_stream_min_k = 1024;
MX_HOST_API void mx_gemv_set_path(int path) { g_gemv_path = path; }

// Row-parallel GEMV fused with the all-reduce: fp32 partials [M][N] land in every rank's inbox (see comm.cuh).
MX_HOST_API int mx_gemv_allreduce(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, const float* bias, int M,
                                  int N, int K, const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket,
                                  cudaStream_t stream) {
  if ((long long)M * N * 4 > slot_bytes) return -140;
  mx::PeerOut po = mx::make_peer_out(inbox, world, my_rank, slot_bytes, seq, ticket);
  return gemv_impl(wfmt, w0, w1, w2, w3, x, nullptr, bias, M, N, K, 1, 0, 0.f, 0.f, nullptr, nullptr, 0, 1, &po, stream);
}

static int gemv_impl(int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const void* x, void* y,
                     const float* bias, int M, int N, int K, int out_f32, int act, float act_alpha, float act_limit,
                     const int* slot_expert, const float* slot_scale, int slots, int x_div, const mx::PeerOut* peer, cudaStream_t stream) {
  using namespace mx;
  if (N <= 0 || K <= 0) return 0;
  if (K % 32 && !(wfmt == WF_BF16 && K % 8 == 0 && act == 0)) return -102;
  if ((wfmt == WF_Q4K || wfmt == WF_Q6K) && (K % 256)) return -103;
  if (!slot_expert && act == 0 && (M < 1 || M > GEMV_MAX_M)) return -106;
  if (g_gemv_path == 2 || (g_gemv_path == 0 && (wfmt == WF_BF16 || wfmt == WF_Q8 || (wfmt == WF_Q4K && K >= g_kq_stream_min_k) ||
                                                (wfmt == WF_Q6K && act == 0 && K >= g_kq_stream_min_k) || (wfmt == WF_MXFP4 && act != 0)))) {
    const int rc = gemv_stream_try(wfmt, WeightRef{w0, w1, w2, w3}, x, y, bias, M, N, K, out_f32, act, act_alpha, act_limit, slot_expert,
                                   slot_scale, slots, x_div, g_e_lo, g_e_hi, peer, stream);
    if (rc != 1) return rc;
  }
  GemvParams p;
  p.w = WeightRef{w0, w1, w2, w3};
  p.x = (const __nv_bfloat16*)x; p.y = y; p.bias = bias;
  p.slot_expert = slot_expert; p.slot_scale = slot_scale; p.x_div = x_div > 0 ? x_div : 1;
  p.e_lo = g_e_lo; p.e_hi = g_e_hi;
  p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32;
  p.act = act; p.act_alpha = act_alpha; p.act_limit = act_limit;
  if (peer) p.peer = *peer; else p.peer.world = 0;
  const int ns = (slot_expert || act != 0) ? (slots > 0 ? slots : M) : 1;
  switch (wfmt) {
    case WF_BF16: return launch_gemv<WF_BF16>(p, ns, stream);
    case WF_Q8: return launch_gemv<WF_Q8>(p, ns, stream);
    case WF_Q4K: return launch_gemv<WF_Q4K>(p, ns, stream);
    case WF_Q6K: return launch_gemv<WF_Q6K>(p, ns, stream);
    case WF_MXFP4: return launch_gemv<WF_MXFP4>(p, ns, stream);
    default: return -100;
  }
}
