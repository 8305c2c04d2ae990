// Streaming GEMV for decode (M <= 8 activation rows): persistent CTAs pull the weight matrix through a shared-memory
// ring with bulk asynchronous copies (cp.async.bulk + mbarrier transaction counts), one producer warp feeding
// 4-8 consumer warps.  A weight row block is one contiguous run per plane, so a stage is one or two bulk copies;
// the bytes in flight per SM are set by the ring (about 100 KB), not by registers or occupancy, which is what a
// 1-3 us kernel needs to get near HBM speed.  Rows longer than one chunk are cut along K: a stage is then RB row segments
// that are not contiguous, fetched by one tiled TMA load per plane (the plane as a 2-D byte tensor) -- one bulk copy per
// segment is bound by the rate of copy requests (about 120 cycles each), not by bytes.  Formats: bf16, Q8 (int8 + fp16 scale per 32), MXFP4 (E2M1 nibbles +
// e8m0 scale per 32), Q4_K (native 144-byte blocks) and Q6_K (four planes).  Q8, Q4_K and Q6_K codes meet block-scaled 16-bit
// activations in dp4a (exact integer partial sums, see the staging code).  MXFP4 rows are multiplied in packed fp16: the E2M1 codes become f16x2 words by byte permutes,
// the activation row is staged once as f16 scaled into range, 16-term partial sums run in HFMA2 and are folded
// into fp32 with the block scale.
//
// Modes (same contract as the register-streamed kernels in gemv.cu, which remain the path for the
// shapes this kernel does not take):
//   dense : y[m][n] for m < M, all rows share each decoded weight
//   slots : one activation row per slot (MoE decode: slot -> expert id -> weight slab; slots of experts owned by
//           another rank give zeros), optional gated activation over 16-row interleaved gate/up rows
// Fused epilogues: bias, per-slot scale, SwiGLU / clamped SwiGLU / GeGLU, stores into every rank's all-reduce inbox.
//
// Fused prologue (dense mode, bf16 / Q8 weights): the activation rows are formed in the kernel as RMSNorm(x + delta) * w from the fp32
// residual rows, where delta is a bf16 tensor or the expert combine sum_k cw[k] * yp[pos[k]]; every CTA computes the few rows for
// itself (they are a few KB and sit in L2), CTA 0 also writes the updated residual to a second buffer (other CTAs still read the old
// one) and, when asked, the normalised rows.  Fused tail (router GEMV): the CTA that finishes last (an atomic ticket) reads the
// logits, picks the top-k experts per token and writes the token rows as MXFP8 pair tiles for the block-scaled expert GEMM.
//
// Reference parity: src/ops/gemv_fp16.cpp:64, gemv_q8dot.cpp:276-680, gemv_mxfp4.cpp:94-323, moe_fused.cpp:101-541.
#include <cstring>
#include "common.cuh"
#include "comm.cuh"
#include "dequant.cuh"
#include "host_util.h"
#include "moe_route.cuh"
#include "mxfp8.cuh"

namespace mx {

static int g_gs_bf16_wide = 0;    // bf16 matrices with eight consumer warps per CTA (mx_gemv_stream_set_bf16_wide: A/B timing)
static int g_gs_tma = 1;          // tiled TMA loads for chunked stages (mx_gemv_stream_set_tma: A/B timing)

constexpr int GS_MAX_STAGES = 4;
constexpr int GS_MAX_XROWS = 8;
constexpr int GS_MAX_CK = 8;      // pairs per token the fused combine + norm prologue takes
constexpr int GS_NORM_MAX_K = 4096;   // row length the fused norm prologue holds in registers (8 float4 per thread at 128 threads)
constexpr int GS_NORM_MAX_M = 2;      // rows: they are normalised one after the other, so more rows go through the separate kernel

// Q8 weights against block-scaled 16-bit activations in dp4a: chosen inside this file for WF_Q8 launches without the norm prologue
// or the router tail (those write and read the activation rows as bf16)
constexpr int WF_Q8I = 16;

// bf16 with eight consumer warps per CTA instead of four (chosen at run time, see g_gs_bf16_wide)
constexpr int WF_BF16W = 17;
__host__ __device__ constexpr bool gs_is_bf16(int f) { return f == WF_BF16 || f == WF_BF16W; }

template <int FMT> struct GsCfg;
template <> struct GsCfg<WF_BF16> { static constexpr int WARPS = 4, RPW = 1; };
template <> struct GsCfg<WF_BF16W> { static constexpr int WARPS = 8, RPW = 1; };
template <> struct GsCfg<WF_Q8> { static constexpr int WARPS = 8, RPW = 1; };
template <> struct GsCfg<WF_MXFP4> { static constexpr int WARPS = 8, RPW = 2; };
template <> struct GsCfg<WF_Q4K> { static constexpr int WARPS = 8, RPW = 2; };
template <> struct GsCfg<WF_Q8I> { static constexpr int WARPS = 8, RPW = 2; };
template <> struct GsCfg<WF_Q6K> { static constexpr int WARPS = 8, RPW = 2; };

// activation rows = RMSNorm(x + delta_scale * delta) * w
struct GsNorm {
  const float* x;               // [M][K] fp32 residual rows; null: the kernel reads bf16 rows from GsParams::x
  float* x_out;                 // x + delta (a buffer other than x), written by CTA 0; null when there is no delta
  const __nv_bfloat16* delta;   // [M][K] or null
  const __nv_bfloat16* yp;      // combine form of delta: packed expert outputs [rows][K] ...
  const int* pos;               // ... [M][ck] row of yp per (token, slot) pair, < 0: no contribution
  const float* cw;              // ... [M][ck] weights
  int ck;
  const float* w;               // [K]
  float eps, delta_scale;
  int one_plus_w;
  __nv_bfloat16* h_out;         // optional: the normalised rows [M][K], written by CTA 0
};
// router tail: y holds fp32 logits [M][N]
struct GsRoute {
  int* ticket;                  // null: no tail
  const float* bias;
  int Kt, renorm;
  int* topk_idx;                // [M][Kt]
  float* topk_w;                // [M][w_copies][Kt]
  int w_copies;
  uint8_t* xq;                  // [M * Kt][KB * 128] e4m3: one row per (token, slot) pair
  uint8_t* sfx;                 // scale atoms [KB][max_tiles][512], pair r is row 0 of tile r
  int KB, max_tiles;
};

struct GsParams {
  GsNorm norm;
  GsRoute route;
  WeightRef w;
  const __nv_bfloat16* x;   // [n_xrows][K]
  void* y;
  const float* bias;
  const int* slot_expert;
  const float* slot_scale;
  int x_div, e_lo, e_hi;
  int M, N, K;
  int out_f32, act;
  float act_alpha, act_limit;
  int slots;                // slot mode: number of slots; dense mode: 1
  int slot_mode;            // 1: activation row = slot / x_div and one output row per slot
  int n_xrows;
  int KC, nkc;              // k chunk in elements (whole rows unless bf16 rows are very long) and chunks per row
  int nblk;                 // row blocks (plain) or feature blocks (gated) per slot
  int nst;                  // ring depth (2..4), chosen so that two CTAs fit an SM where possible
  int use_tma;              // chunked rows: one tiled TMA load per plane and stage (tensor maps over the planes) instead of one bulk copy per row
  long long tma_rows;       // rows the tensor maps cover (experts x N)
  int* status;
  PeerOut peer;
};

template <int FMT> __host__ __device__ __forceinline__ int gs_row_bytes0(int K) {
  return gs_is_bf16(FMT) ? K * 2 : ((FMT == WF_Q8 || FMT == WF_Q8I) ? K : (FMT == WF_Q4K ? K / 256 * 144 : K / 2));      // MXFP4 nibbles, Q6_K low nibbles
}
template <int FMT> __host__ __device__ __forceinline__ int gs_row_bytes1(int K) {
  return (gs_is_bf16(FMT) || FMT == WF_Q4K) ? 0 : ((FMT == WF_Q8 || FMT == WF_Q8I) ? q8_d_stride(K) * 2 : (FMT == WF_Q6K ? K / 4 : mxfp4_e_stride(K)));
}
// Q6_K only: the int8 sub-block scales and the fp16 block scales
template <int FMT> __host__ __device__ __forceinline__ int gs_row_bytes2(int K) { return FMT == WF_Q6K ? K / 16 : 0; }
template <int FMT> __host__ __device__ __forceinline__ int gs_row_bytes3(int K) { return FMT == WF_Q6K ? q6k_d_stride(K) * 2 : 0; }
// bytes of one row inside a stage: the whole row, or its k chunk for the formats that are chunked (bf16, Q4_K, Q8 in the dp4a form)
template <int FMT> __host__ __device__ __forceinline__ int gs_stage_row0(int K, int KC) {
  return gs_is_bf16(FMT) ? KC * 2 : (FMT == WF_Q4K ? KC / 256 * 144 : (FMT == WF_Q8I ? KC : (FMT == WF_Q6K ? KC / 2 : gs_row_bytes0<FMT>(K))));
}
template <int FMT> __host__ __device__ __forceinline__ int gs_stage_row1(int K, int KC) {
  return (FMT == WF_Q8I && KC != K) ? KC / 16 : (FMT == WF_Q6K ? KC / 4 : gs_row_bytes1<FMT>(K));
}
template <int FMT> __host__ __device__ __forceinline__ int gs_stage_row2(int K, int KC) { return FMT == WF_Q6K ? KC / 16 : 0; }
// (the fp16 block scales of a Q6_K row are a few 16-byte words: every chunk of the row brings the whole run)
template <int FMT> __host__ __device__ __forceinline__ int gs_stage_row_all(int K, int KC) {
  return gs_stage_row0<FMT>(K, KC) + gs_stage_row1<FMT>(K, KC) + gs_stage_row2<FMT>(K, KC) + gs_row_bytes3<FMT>(K);
}
// bytes of one staged activation row.  Q4_K: nine planes of K/64 (+1 pad) 16-byte words, see the staging code in the kernel.
template <int FMT> __host__ __device__ __forceinline__ int gs_xplane_step(int K) {
  return (FMT == WF_Q4K || FMT == WF_Q6K) ? (K >> 6) + 1 : (FMT == WF_Q8I ? ((K >> 5) | 1) : 0);
}
template <int FMT> __host__ __device__ __forceinline__ int gs_xrow_bytes(int K) {
  return FMT == WF_Q4K ? 9 * gs_xplane_step<FMT>(K) * 16
                       : (FMT == WF_Q6K ? 10 * gs_xplane_step<FMT>(K) * 16 : (FMT == WF_Q8I ? 5 * gs_xplane_step<FMT>(K) * 16 : K * 2));
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

__device__ __forceinline__ float gs_act(int act, float g, float u, float alpha, float limit) {
  if (act == 1) return g / (1.f + __expf(-g)) * u;
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t) * u;
}

// Eight E2M1 codes (nibble i of w = code i) -> four f16x2 words (codes 0|1, 2|3, 4|5, 6|7) by byte permutes: every
// E2M1 value is an f16 whose low byte is zero, so one 8-entry byte table holds the magnitudes and the sign lands on
// bit 7 of the same byte.
__device__ __forceinline__ void e2m1x8_to_f16x2_lut(uint32_t w, uint32_t (&o)[4]) {
  const uint32_t se = __byte_perm(w << 4, 0u, 0xBA98);      // byte b = 0xFF if code 2b   is negative
  const uint32_t so = __byte_perm(w, 0u, 0xBA98);           // byte b = 0xFF if code 2b+1 is negative
  const uint32_t sel = w & 0x77777777u;
  {
    const uint32_t sg = __byte_perm(se, so, 0x5140);                     // signs of codes 0,1,2,3
    const uint32_t hi = __byte_perm(0x3E3C3800u, 0x46444240u, sel) | (sg & 0x80808080u);
    o[0] = __byte_perm(hi, 0u, 0x1404);
    o[1] = __byte_perm(hi, 0u, 0x3424);
  }
  {
    const uint32_t sg = __byte_perm(se, so, 0x7362);                     // signs of codes 4,5,6,7
    const uint32_t hi = __byte_perm(0x3E3C3800u, 0x46444240u, sel >> 16) | (sg & 0x80808080u);
    o[2] = __byte_perm(hi, 0u, 0x1404);
    o[3] = __byte_perm(hi, 0u, 0x3424);
  }
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float f16x2_sum(uint32_t v) {
  const __half2 h = *reinterpret_cast<const __half2*>(&v);
  return __low2float(h) + __high2float(h);
}

// signed byte i of (v ^ 0x80808080) as float: 2^23 + u is exact, so is the subtraction
template <int I>
__device__ __forceinline__ float s8_to_float(uint32_t vx) {
  return __uint_as_float(__byte_perm(vx, 0x4B000000u, 0x7440 | I)) - 8388736.f;      // [b_I, 0, 0, 0x4B]
}

// ---- granules: the unit of work of a lane.  Lane l owns granules l, l+32, ... of every row, so consecutive lanes read
// consecutive 16-byte words of the weight row (no bank conflicts) and, with one activation row, keep their slice of x
// in registers for the whole kernel.
template <int FMT> struct Gran;
template <> struct Gran<WF_BF16> { static constexpr int GE = 8, XR = 4, NGMAX = 16; };     // 8 bf16 = one 16-byte word
template <> struct Gran<WF_BF16W> : Gran<WF_BF16> {};
template <> struct Gran<WF_Q8> { static constexpr int GE = 16, XR = 8, NGMAX = 8; };       // 16 int8
template <> struct Gran<WF_MXFP4> { static constexpr int GE = 32, XR = 16, NGMAX = 4; };   // 32 nibbles
template <> struct Gran<WF_Q4K> { static constexpr int GE = 64, XR = 36, NGMAX = 1; };     // 32 bytes of a Q4_K block: two sub-blocks
template <> struct Gran<WF_Q6K> { static constexpr int GE = 64, XR = 40, NGMAX = 1; };     // four 16-element sub-blocks
template <> struct Gran<WF_Q8I> { static constexpr int GE = 32, XR = 17, NGMAX = 3; };     // one Q8 block

// The MXFP4 path keeps its f16 activation row in four planes (plane i holds elements 8i..8i+7 of every 32-element
// granule), so that consecutive lanes read consecutive 16-byte words of each plane.
// The Q4_K path holds the row as block-scaled 16-bit integers split into a high and a low int8 (see the staging code), in
// eight planes plus a ninth with the scales and sums of the granule's two sub-blocks.  g counts granules from the row start.
template <int FMT>
__device__ __forceinline__ void load_xg(const uint8_t* __restrict__ xrow, int g, int K, uint32_t (&xr)[Gran<FMT>::XR]) {
  constexpr bool PLANES = FMT == WF_MXFP4 || FMT == WF_Q4K || FMT == WF_Q6K || FMT == WF_Q8I;
  const uint4* p = reinterpret_cast<const uint4*>(xrow) + (PLANES ? g : g * (Gran<FMT>::XR / 4));
  const int step = FMT == WF_MXFP4 ? (K >> 5) : (PLANES ? gs_xplane_step<FMT>(K) : 1);
#pragma unroll
  for (int i = 0; i < Gran<FMT>::XR / 4; ++i) {
    const uint4 v = p[i * step];
    xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
  }
  if constexpr (FMT == WF_Q8I) xr[16] = *reinterpret_cast<const uint32_t*>(p + 4 * step);      // the block's scale (first word of the last plane)
}

// decoded weight granule, ready to be multiplied with any number of activation rows
template <int FMT> struct WG;
template <> struct WG<WF_BF16> { uint4 v; };
template <> struct WG<WF_BF16W> : WG<WF_BF16> {};
template <> struct WG<WF_Q8> { float w[16]; float d; };
template <> struct WG<WF_MXFP4> { uint32_t t[16]; float sc; };
template <> struct WG<WF_Q6K> { uint32_t ev[8], od[8]; float ds[4]; };          // 6-bit codes of the even / odd elements, d * sub-block scale
template <> struct WG<WF_Q8I> { uint32_t q[8]; float d; };
template <> struct WG<WF_Q4K> { uint32_t a[8], b[8]; float dA, dB, mA, mB; };   // 4-bit codes as bytes (sub-blocks 2j / 2j+1), d * scale, dmin * min

// the second pair of planes and the first block of the chunk (index into the row's block scales) are Q6_K's
struct GsPlanes23 {
  const uint8_t* w2;
  const uint8_t* w3;
  int dblk0;
};

template <int FMT>
__device__ __forceinline__ void decode_g(const uint8_t* __restrict__ w0, const uint8_t* __restrict__ w1, const GsPlanes23& w23, int g, WG<FMT>& o) {
  if constexpr (gs_is_bf16(FMT)) {
    o.v = reinterpret_cast<const uint4*>(w0)[g];
  } else if constexpr (FMT == WF_Q8) {
    const uint4 a = reinterpret_cast<const uint4*>(w0)[g];
    o.d = __half2float(reinterpret_cast<const __half*>(w1)[g >> 1]);
    const uint32_t q[4] = {a.x ^ 0x80808080u, a.y ^ 0x80808080u, a.z ^ 0x80808080u, a.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o.w[4 * i] = s8_to_float<0>(q[i]); o.w[4 * i + 1] = s8_to_float<1>(q[i]); o.w[4 * i + 2] = s8_to_float<2>(q[i]); o.w[4 * i + 3] = s8_to_float<3>(q[i]);
    }
  } else if constexpr (FMT == WF_Q6K) {
    // granule g = 64 elements: 32 bytes of low nibbles (byte i = e[2i] | e[2i+1] << 4), four words of high bit pairs (one per 16
    // elements: byte b holds e[2b], e[2b+1], e[8+2b], e[9+2b] from bit 0 up), four int8 scales, the block's fp16 scale
    const uint4 l0 = reinterpret_cast<const uint4*>(w0)[2 * g], l1 = reinterpret_cast<const uint4*>(w0)[2 * g + 1];
    const uint4 hv = reinterpret_cast<const uint4*>(w1)[g];
    const uint32_t scw = reinterpret_cast<const uint32_t*>(w23.w2)[g];
    const float d = __half2float(reinterpret_cast<const __half*>(w23.w3)[w23.dblk0 + (g >> 2)]);
    // int8 -> float: 2^23 + (s ^ 0x80) - (2^23 + 128)
    const uint32_t su = scw ^ 0x80808080u;
    o.ds[0] = d * s8_to_float<0>(su); o.ds[1] = d * s8_to_float<1>(su); o.ds[2] = d * s8_to_float<2>(su); o.ds[3] = d * s8_to_float<3>(su);
    const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t h = hw[i >> 1] >> ((i & 1) * 4);
      o.ev[i] = (lw[i] & 0x0F0F0F0Fu) | ((h & 0x03030303u) << 4);
      o.od[i] = ((lw[i] >> 4) & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
    }
  } else if constexpr (FMT == WF_Q8I) {
    const uint4 a = reinterpret_cast<const uint4*>(w0)[2 * g], b = reinterpret_cast<const uint4*>(w0)[2 * g + 1];
    o.d = __half2float(reinterpret_cast<const __half*>(w1)[g]);
    o.q[0] = a.x; o.q[1] = a.y; o.q[2] = a.z; o.q[3] = a.w; o.q[4] = b.x; o.q[5] = b.y; o.q[6] = b.z; o.q[7] = b.w;
  } else if constexpr (FMT == WF_Q4K) {
    // granule g = 64 elements: group j = g & 3 of block g >> 2.  Byte i of the 32-byte group holds element i of sub-block 2j in its
    // low nibble and element i of sub-block 2j+1 in its high nibble.
    const uint8_t* blk = w0 + (size_t)(g >> 2) * 144;
    const int j = g & 3;
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
    const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * j), q1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * j);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    // the 6-bit scales and minima of the two sub-blocks, two bytes each (same packing as q4k_scale_min)
    const int sh = (j & 1) * 16;
    const uint32_t s0 = hdr.y >> sh, s1 = hdr.z >> sh, s2 = hdr.w >> sh;
    const uint32_t sc2 = j < 2 ? (s0 & 0x3F3Fu) : ((s2 & 0x0F0Fu) | ((s0 >> 2) & 0x3030u));
    const uint32_t mn2 = j < 2 ? (s1 & 0x3F3Fu) : (((s2 >> 4) & 0x0F0Fu) | ((s1 >> 2) & 0x3030u));
    o.dA = d * (__uint_as_float(0x4B000000u | (sc2 & 0xFFu)) - 8388608.f);
    o.dB = d * (__uint_as_float(0x4B000000u | (sc2 >> 8)) - 8388608.f);
    o.mA = dmin * (__uint_as_float(0x4B000000u | (mn2 & 0xFFu)) - 8388608.f);
    o.mB = dmin * (__uint_as_float(0x4B000000u | (mn2 >> 8)) - 8388608.f);
    const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o.a[i] = q[i] & 0x0F0F0F0Fu;
      o.b[i] = (q[i] >> 4) & 0x0F0F0F0Fu;
    }
  } else {
    const uint4 v = reinterpret_cast<const uint4*>(w0)[g];
    o.sc = e8m0_f32(w1[g]);
    const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t4[4];
      e2m1x8_to_f16x2_lut(q[i], t4);
      o.t[4 * i] = t4[0]; o.t[4 * i + 1] = t4[1]; o.t[4 * i + 2] = t4[2]; o.t[4 * i + 3] = t4[3];
    }
  }
}

template <int FMT>
__device__ __forceinline__ float dot_g(const WG<FMT>& w, const uint32_t (&xr)[Gran<FMT>::XR], float xscale) {
  if constexpr (gs_is_bf16(FMT)) {
    float s = bf16_lo(w.v.x) * bf16_lo(xr[0]);
    s = fmaf(bf16_hi(w.v.x), bf16_hi(xr[0]), s);
    s = fmaf(bf16_lo(w.v.y), bf16_lo(xr[1]), s); s = fmaf(bf16_hi(w.v.y), bf16_hi(xr[1]), s);
    s = fmaf(bf16_lo(w.v.z), bf16_lo(xr[2]), s); s = fmaf(bf16_hi(w.v.z), bf16_hi(xr[2]), s);
    s = fmaf(bf16_lo(w.v.w), bf16_lo(xr[3]), s); s = fmaf(bf16_hi(w.v.w), bf16_hi(xr[3]), s);
    return s;
  } else if constexpr (FMT == WF_Q8) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s0 = fmaf(w.w[2 * i], bf16_lo(xr[i]), s0);
      s1 = fmaf(w.w[2 * i + 1], bf16_hi(xr[i]), s1);
    }
    return (s0 + s1) * w.d;
  } else if constexpr (FMT == WF_Q6K) {
    // per 16-element sub-block: exact integer dot product of the codes with the 16-bit activations, then
    // d * scale * (D * activation scale - 32 * sum of the activations)
    float r = 0.f;
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
      int dh = 0, dl = 0;
#pragma unroll
      for (int c = 2 * sb; c < 2 * sb + 2; ++c) {
        dh = __dp4a((int)w.ev[c], (int)xr[4 * c], dh);
        dh = __dp4a((int)w.od[c], (int)xr[4 * c + 1], dh);
        dl = __dp4a((int)w.ev[c], (int)xr[4 * c + 2], dl);
        dl = __dp4a((int)w.od[c], (int)xr[4 * c + 3], dl);
      }
      r = fmaf(w.ds[sb], fmaf((float)(dh * 256 + dl), __uint_as_float(xr[32 + (sb >> 1)]), -32.f * __uint_as_float(xr[36 + sb])), r);
    }
    return r;
  } else if constexpr (FMT == WF_Q8I) {
    int ah = 0, al = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int pa = 4 * (k >> 1) + (k & 1);
      ah = __dp4a((int)w.q[k], (int)xr[pa], ah);
      al = __dp4a((int)w.q[k], (int)xr[pa + 2], al);
    }
    return (float)(ah * 256 + al) * (w.d * __uint_as_float(xr[16]));
  } else if constexpr (FMT == WF_Q4K) {
    // exact integer dot products of the 4-bit codes with the high and the low byte of the 16-bit activations; the
    // minima multiply the plain sums of the activations
    int ah = 0, al = 0, bh = 0, bl = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int pa = 4 * (k >> 1) + (k & 1), pb = 16 + pa;
      ah = __dp4a((int)w.a[k], (int)xr[pa], ah);
      al = __dp4a((int)w.a[k], (int)xr[pa + 2], al);
      bh = __dp4a((int)w.b[k], (int)xr[pb], bh);
      bl = __dp4a((int)w.b[k], (int)xr[pb + 2], bl);
    }
    const float fa = (float)(ah * 256 + al) * __uint_as_float(xr[32]), fb = (float)(bh * 256 + bl) * __uint_as_float(xr[33]);
    return fmaf(w.dA, fa, fmaf(w.dB, fb, -fmaf(w.mA, __uint_as_float(xr[34]), w.mB * __uint_as_float(xr[35]))));
  } else {
    uint32_t a0 = 0u, a1 = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a0 = hfma2_u32(w.t[2 * i], xr[2 * i], a0);
      a1 = hfma2_u32(w.t[2 * i + 1], xr[2 * i + 1], a1);
    }
    return (f16x2_sum(a0) + f16x2_sum(a1)) * (w.sc * xscale);
  }
}

// one weight row (one k chunk of it) against MM activation rows; CACHED: the lane's x granules are in registers
template <int FMT, int MM, bool CACHED, int NG>
__device__ __forceinline__ void gs_row(const uint8_t* __restrict__ w0, const uint8_t* __restrict__ w1, const GsPlanes23& w23, int ng, int lane,
                                       const uint32_t (&xc)[CACHED ? NG : 1][Gran<FMT>::XR], const uint8_t* __restrict__ xs, int K, int gbase,
                                       const float* __restrict__ xscale, float (&acc)[MM]) {
  if constexpr (CACHED) {
#pragma unroll
    for (int j = 0; j < NG; ++j) {
      const int g = lane + 32 * j;
      if (g < ng) {
        WG<FMT> wg;
        decode_g<FMT>(w0, w1, w23, g, wg);
        acc[0] += dot_g<FMT>(wg, xc[j], 1.f);
      }
    }
  } else {
#pragma unroll 1
    for (int g = lane; g < ng; g += 32) {
      WG<FMT> wg;
      decode_g<FMT>(w0, w1, w23, g, wg);
      {
#pragma unroll
        for (int m = 0; m < MM; ++m) {
          uint32_t xr[Gran<FMT>::XR];
          load_xg<FMT>(xs + (size_t)m * gs_xrow_bytes<FMT>(K), gbase + g, K, xr);
          acc[m] += dot_g<FMT>(wg, xr, FMT == WF_MXFP4 ? xscale[m] : 1.f);
        }
      }
    }
  }
}

// NG: granules per lane and row chunk (compile time, so the activation slice stays in registers); two CTAs per SM
template <int FMT, int MM, bool GATED, int NG>
__global__ void __launch_bounds__((GsCfg<FMT>::WARPS + 1) * 32, 2)
gemv_stream_kernel(const GsParams p, const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, const __grid_constant__ CUtensorMap tm2) {
  constexpr int WARPS = GsCfg<FMT>::WARPS, RPW = GsCfg<FMT>::RPW, RB = WARPS * RPW, FB = RB / 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K;
  const int g0 = gs_row_bytes0<FMT>(K), g1 = gs_row_bytes1<FMT>(K), g2 = gs_row_bytes2<FMT>(K), g3 = gs_row_bytes3<FMT>(K);      // global row strides
  const int r0b = gs_stage_row0<FMT>(K, p.KC), r1b = gs_stage_row1<FMT>(K, p.KC), r2b = gs_stage_row2<FMT>(K, p.KC), r3b = g3;   // bytes per row inside a stage
  const int plane1_off = RB * r0b, plane2_off = plane1_off + RB * r1b, plane3_off = plane2_off + RB * r2b;
  const int stage_bytes = RB * (r0b + r1b + r2b + r3b);
  const int xrow_bytes = gs_xrow_bytes<FMT>(K);
  // the stages start on a 128-byte boundary of the shared window (tiled TMA loads want it; the host adds the slack)
  const int x_bytes = ((p.n_xrows * xrow_bytes + 127) & ~127) + (int)((128u - (smem_u32(smem) & 127u)) & 127u);
  uint8_t* xs = smem;
  uint8_t* stages = smem + x_bytes;
  const int NST = p.nst;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stages + NST * stage_bytes);
  float* xscale = reinterpret_cast<float*>(bars + 2 * GS_MAX_STAGES);
  volatile int* abort_flag = reinterpret_cast<int*>(xscale + GS_MAX_XROWS);
  const uint32_t bar0 = smem_u32(bars);
  // Programmatic dependent launch: the weights are not produced by any kernel, so the producer warp starts to fill the ring
  // while the previous kernel is still running; everything that depends on earlier kernels (activations, expert ids, the
  // collective's sequence word, all global stores) comes after pdl_wait().
  pdl_launch_dependents();
  int next_seq = 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(bar0 + 8 * s, 1);
      mbar_init(bar0 + 8 * (GS_MAX_STAGES + s), WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int units = p.slots * p.nblk;
  const int F = p.N / 2;

  if (warp == WARPS) {
    // ------------------------------------------------------------ producer warp: lane 0 waits for a free stage and announces the
    // bytes; whole-row-block copies are issued by lane 0, the per-row copies of a k chunk by one lane per row (a single lane
    // issues about one bulk copy per 120 cycles, which bounds a chunked matrix well below the memory rate)
    {
      int it = 0;
      bool ok = true;
      if (p.slot_expert) pdl_wait();          // the expert ids come from the router kernel
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int slot = u / p.nblk, blk = u - slot * p.nblk;
        const uint8_t* b0 = (const uint8_t*)p.w.p0;
        const uint8_t* b1 = (const uint8_t*)p.w.p1;
        const uint8_t* b2 = (const uint8_t*)p.w.p2;
        const uint8_t* b3 = (const uint8_t*)p.w.p3;
        int tma_row0 = 0;          // first row of this slot's matrix in the tensor maps
        if (p.slot_expert) {
          const int e = p.slot_expert[slot];
          if (e < p.e_lo || e >= p.e_hi) continue;
          tma_row0 = (e - p.e_lo) * p.N;
          b0 += (size_t)(e - p.e_lo) * p.N * g0;
          b1 += (size_t)(e - p.e_lo) * p.N * g1;
          b2 += (size_t)(e - p.e_lo) * p.N * g2;
          b3 += (size_t)(e - p.e_lo) * p.N * g3;
        }
        for (int kc = 0; kc < p.nkc && ok; ++kc, ++it) {
          const int s = it % NST;
          const uint32_t full = bar0 + 8 * s, empty = bar0 + 8 * (GS_MAX_STAGES + s);
          if (it >= NST) {
            if (lane == 0) ok = mbar_wait(empty, ((it / NST) & 1) ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          }
          if (!ok) break;
          const uint32_t dst = smem_u32(stages + (size_t)s * stage_bytes);
          if (GATED) {
            const int f0 = blk * FB, nf = min(FB, F - f0);
            const int grow = 32 * (f0 >> 4) + (f0 & 15);
            if (p.use_tma) {
              // two boxes of FB rows per plane (rows past the block's last feature are loaded and ignored; rows past the matrix read zeros)
              if (lane == 0) {
                mbar_expect_tx(full, 2u * FB * (r0b + r1b));
                tma_load_2d(dst, &tm0, full, kc * (r0b >> 3), tma_row0 + grow);
                tma_load_2d(dst + FB * r0b, &tm0, full, kc * (r0b >> 3), tma_row0 + grow + 16);
                if (r1b) {
                  tma_load_2d(dst + plane1_off, &tm1, full, kc * (r1b >> 3), tma_row0 + grow);
                  tma_load_2d(dst + plane1_off + FB * r1b, &tm1, full, kc * (r1b >> 3), tma_row0 + grow + 16);
                }
              }
              continue;
            }
            if (lane == 0) mbar_expect_tx(full, 2u * nf * (r0b + r1b));
            __syncwarp();
            if (p.nkc == 1) {
              if (lane == 0) {
                bulk_g2s(dst, b0 + (size_t)grow * g0, nf * r0b, full);
                bulk_g2s(dst + FB * r0b, b0 + (size_t)(grow + 16) * g0, nf * r0b, full);
              }
            } else {
              // k chunk of every gate row (lanes 0..nf-1) and of every up row (lanes 16..16+nf-1), both planes
              const int r = lane & 15, up = lane >> 4;
              if (r < nf) {
                bulk_g2s(dst + (up * FB + r) * r0b, b0 + (size_t)(grow + 16 * up + r) * g0 + (size_t)kc * r0b, r0b, full);
                if (r1b) bulk_g2s(dst + plane1_off + (up * FB + r) * r1b, b1 + (size_t)(grow + 16 * up + r) * g1 + (size_t)kc * r1b, r1b, full);
              }
            }
            if (r1b && lane == 0 && p.nkc == 1) {
              bulk_g2s(dst + plane1_off, b1 + (size_t)grow * g1, nf * r1b, full);
              bulk_g2s(dst + plane1_off + FB * r1b, b1 + (size_t)(grow + 16) * g1, nf * r1b, full);
            }
          } else {
            const int row0 = blk * RB, nr = min(RB, p.N - row0);
            if (p.use_tma) {
              if (lane == 0) {
                mbar_expect_tx(full, (uint32_t)RB * (r0b + r1b + r2b) + (uint32_t)nr * r3b);
                tma_load_2d(dst, &tm0, full, kc * (r0b >> 3), tma_row0 + row0);
                if (r1b) tma_load_2d(dst + plane1_off, &tm1, full, kc * (r1b >> 3), tma_row0 + row0);
                if (r2b) tma_load_2d(dst + plane2_off, &tm2, full, kc * (r2b >> 3), tma_row0 + row0);
                if (r3b) bulk_g2s(dst + plane3_off, b3 + (size_t)row0 * g3, nr * r3b, full);
              }
              continue;
            }
            if (lane == 0) mbar_expect_tx(full, (uint32_t)nr * (r0b + r1b + r2b + r3b));
            __syncwarp();
            if (p.nkc == 1) {
              if (lane == 0) {
                bulk_g2s(dst, b0 + (size_t)row0 * g0, nr * r0b, full);
                if (r1b) bulk_g2s(dst + plane1_off, b1 + (size_t)row0 * g1, nr * r1b, full);
                if (r2b) bulk_g2s(dst + plane2_off, b2 + (size_t)row0 * g2, nr * r2b, full);
              }
            } else {
              // lanes 0..15: plane 0 (and 2) of row `lane`; lanes 16..31: plane 1 of row `lane - 16`
              const int r = lane & 15, hi = lane >> 4;
              for (int rr = r; rr < nr; rr += 16) {
                if (hi == 0) {
                  bulk_g2s(dst + rr * r0b, b0 + (size_t)(row0 + rr) * g0 + (size_t)kc * r0b, r0b, full);
                  if (r2b) bulk_g2s(dst + plane2_off + rr * r2b, b2 + (size_t)(row0 + rr) * g2 + (size_t)kc * r2b, r2b, full);
                } else if (r1b) {
                  bulk_g2s(dst + plane1_off + rr * r1b, b1 + (size_t)(row0 + rr) * g1 + (size_t)kc * r1b, r1b, full);
                }
              }
            }
            if (r3b && lane == 0) bulk_g2s(dst + plane3_off, b3 + (size_t)row0 * g3, nr * r3b, full);     // whole runs of block scales, every chunk
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    pdl_wait();
    next_seq = p.peer.world ? *p.peer.seq + 1 : 0;
    // stage the activation rows once (bf16 as they are; MXFP4 path: f16 scaled so that the row maximum sits near 2^9)
    if constexpr (FMT == WF_MXFP4) {
      // one warp per activation row; a lane keeps its 16-byte chunks in registers between the maximum and the conversion
      for (int m = warp; m < p.n_xrows; m += WARPS) {
        const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * K);
        const int nch = K >> 3;
        constexpr int CH = 16;                                   // chunks per lane: K <= 4096 (checked by the host)
        uint4 v[CH];
        float mx = 0.f;
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int c = lane + 32 * i;
          v[i] = c < nch ? __ldg(xr + c) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const uint32_t q[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) mx = fmaxf(mx, fmaxf(fabsf(bf16_lo(q[j])), fabsf(bf16_hi(q[j]))));
        }
        mx = warp_max(mx);
        int ex = 0;
        if (mx > 0.f) { frexpf(mx, &ex); }                       // mx = f * 2^ex, f in [0.5, 1)
        // x * 2^sh has its maximum in [2^8, 2^9): sixteen products of magnitude <= 6 * 2^9 cannot overflow an f16 sum
        const int sh = max(-24, min(24, 9 - ex));
        const float up = exp2f((float)sh);
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * K * 2);
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int c = lane + 32 * i;
          if (c < nch) {
            const uint32_t q[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2 h = __floats2half2_rn(bf16_lo(q[j]) * up, bf16_hi(q[j]) * up);
              o[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            dst[(c & 3) * (K >> 5) + (c >> 2)] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        if (lane == 0) xscale[m] = exp2f((float)-sh);
      }
    } else if constexpr (FMT == WF_Q4K || FMT == WF_Q6K || FMT == WF_Q8I) {
      // Each 32-element sub-block of a row becomes 16-bit integers X = rint(x * 32512 / amax), split as X = 256 h + l with h, l in
      // int8, so that a weight code times an activation is two exact dp4a terms.  A thread converts one 8-element chunk and its
      // three neighbours hold the rest of the sub-block.  Layout of a row: plane c (0..CPG-1) holds, for every granule, the words
      // {h[0..3], h[4..7], l[0..3], l[4..7]} of the granule's chunk c; the last plane holds the scales and then the sums of the
      // granule's sub-blocks (Q4_K: two sub-blocks in a 64-element granule; Q8: one).  Q6_K: a chunk's even elements fill the first
      // word of h and of l, its odd elements the second (the order in which the 6-bit codes are assembled); the second to last plane
      // holds the two scales, the last the sums of the four 16-element sub-blocks.
      constexpr int CPG = Gran<FMT>::GE / 8, NSUB = CPG / 4;
      const int nch = K >> 3, pstep = gs_xplane_step<FMT>(K);
      for (int m = 0; m < p.n_xrows; ++m) {
        const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * K);
        uint4* row = reinterpret_cast<uint4*>(xs + (size_t)m * xrow_bytes);
        for (int c0 = 0; c0 < nch; c0 += WARPS * 32) {          // every lane of a warp runs the loop body: the shuffles are warp wide
          const int c = c0 + threadIdx.x;
          const bool live = c < nch;
          const uint4 v = live ? __ldg(xr + c) : make_uint4(0u, 0u, 0u, 0u);
          const uint32_t q[4] = {v.x, v.y, v.z, v.w};
          float f[8];
          float amax = 0.f, sum = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            f[2 * i] = bf16_lo(q[i]);
            f[2 * i + 1] = bf16_hi(q[i]);
            amax = fmaxf(amax, fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1])));
            sum += f[2 * i] + f[2 * i + 1];
          }
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          const float sum16 = sum;
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          const float inv = amax > 0.f ? 32512.f / amax : 0.f;
          uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int X = __float2int_rn(f[i] * inv);
            const int h = (X + 128) >> 8, l = X - (h << 8);
            const int at = FMT == WF_Q6K ? (i & 1) * 4 + (i >> 1) : i;          // byte of the two-word group that element i goes to
            hw[at >> 2] |= (uint32_t)(h & 0xFF) << (8 * (at & 3));
            lw[at >> 2] |= (uint32_t)(l & 0xFF) << (8 * (at & 3));
          }
          const int g = c / CPG, cc = c % CPG;
          if (live) {
            row[cc * pstep + g] = make_uint4(hw[0], hw[1], lw[0], lw[1]);
            float* aux = reinterpret_cast<float*>(row + CPG * pstep + g);
            if constexpr (FMT == WF_Q6K) {
              if ((c & 3) == 0) aux[cc >> 2] = amax * (1.f / 32512.f);
              if ((c & 1) == 0) reinterpret_cast<float*>(row + (CPG + 1) * pstep + g)[cc >> 1] = sum16;
            } else if ((c & 3) == 0) {
              aux[cc >> 2] = amax * (1.f / 32512.f);
              aux[NSUB + (cc >> 2)] = sum;
            }
          }
        }
      }
    } else if (p.norm.x) {
      // residual add + RMSNorm in place of a separate launch.  All consumer threads work on one row at a time and keep their
      // elements in registers between the sum of squares and the scaling (K <= GS_NORM_MAX_K, checked by the host), so a row
      // costs one round trip to L2; rows follow one another, which is why the host sends only a couple of rows this way.
      const GsNorm& nm = p.norm;
      const bool writer = blockIdx.x == 0;
      constexpr int NT = WARPS * 32, NV = GS_NORM_MAX_K / (4 * NT);
      float* red = xscale;                      // GS_MAX_XROWS floats, unused by these formats
      for (int m = 0; m < p.n_xrows; ++m) {
        const float* xr = nm.x + (size_t)m * K;
        int pos[GS_MAX_CK];
        float cwv[GS_MAX_CK];
#pragma unroll
        for (int k = 0; k < GS_MAX_CK; ++k) {
          const bool live = nm.yp && k < nm.ck;
          pos[k] = live ? nm.pos[(size_t)m * nm.ck + k] : -1;
          cwv[k] = live ? nm.cw[(size_t)m * nm.ck + k] : 0.f;
        }
        float4 v[NV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int i = (threadIdx.x + j * NT) * 4;
          v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (i < K) {
            v[j] = *reinterpret_cast<const float4*>(xr + i);
            if (nm.yp) {
              float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int k = 0; k < GS_MAX_CK; ++k) {
                if (pos[k] < 0) continue;
                const uint2 yv = *reinterpret_cast<const uint2*>(nm.yp + (size_t)pos[k] * K + i);
                d.x = fmaf(cwv[k], bf16_lo(yv.x), d.x); d.y = fmaf(cwv[k], bf16_hi(yv.x), d.y);
                d.z = fmaf(cwv[k], bf16_lo(yv.y), d.z); d.w = fmaf(cwv[k], bf16_hi(yv.y), d.w);
              }
              v[j].x += d.x * nm.delta_scale; v[j].y += d.y * nm.delta_scale; v[j].z += d.z * nm.delta_scale; v[j].w += d.w * nm.delta_scale;
            } else if (nm.delta) {
              const uint2 dv = *reinterpret_cast<const uint2*>(nm.delta + (size_t)m * K + i);
              v[j].x += bf16_lo(dv.x) * nm.delta_scale; v[j].y += bf16_hi(dv.x) * nm.delta_scale;
              v[j].z += bf16_lo(dv.y) * nm.delta_scale; v[j].w += bf16_hi(dv.y) * nm.delta_scale;
            }
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
          }
        }
        ss = warp_sum(ss);
        consumer_sync(NT);                      // (the previous row's readers of `red` are done)
        if (lane == 0) red[warp] = ss;
        consumer_sync(NT);
        float tot = 0.f;
#pragma unroll
        for (int wv = 0; wv < WARPS; ++wv) tot += red[wv];
        const float inv = rsqrtf(tot / K + nm.eps);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int i = (threadIdx.x + j * NT) * 4;
          if (i < K) {
            float4 g = *reinterpret_cast<const float4*>(nm.w + i);
            if (nm.one_plus_w) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
            const uint2 o = make_uint2(pack_bf16(v[j].x * inv * g.x, v[j].y * inv * g.y), pack_bf16(v[j].z * inv * g.z, v[j].w * inv * g.w));
            *reinterpret_cast<uint2*>(xs + ((size_t)m * K + i) * 2) = o;
            if (writer) {
              if (nm.x_out) *reinterpret_cast<float4*>(nm.x_out + (size_t)m * K + i) = v[j];
              if (nm.h_out) *reinterpret_cast<uint2*>(nm.h_out + (size_t)m * K + i) = o;
            }
          }
        }
      }
    } else {
      const int n16 = p.n_xrows * K / 8;
      for (int i = threadIdx.x; i < n16; i += WARPS * 32) reinterpret_cast<uint4*>(xs)[i] = __ldg(reinterpret_cast<const uint4*>(p.x) + i);
    }
    consumer_sync(WARPS * 32);

    int it = 0;
    bool ok = true;
    constexpr bool CACHED = MM == 1 && FMT != WF_MXFP4;      // MXFP4 decoding needs the registers: x comes from shared memory
    uint32_t xc[CACHED ? NG : 1][Gran<FMT>::XR];
    int x_tag = -1;                                         // (activation row, k chunk) held in xc
    const int ng = p.KC / Gran<FMT>::GE;
    // A k chunk of at most 16 granules would leave half of the lanes idle: the two half-warps take the warp's two rows side by side
    // (each lane accumulates for its own row; the warp-wide sums of the epilogue then see zeros from the other half).
    constexpr bool HALF_OK = (FMT == WF_Q4K || FMT == WF_Q6K) && (GATED || RPW == 2);
    const bool half = HALF_OK && ng <= 16;
    const int xl = half ? (lane & 15) : lane;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int slot = u / p.nblk, blk = u - slot * p.nblk;
      bool owned = true;
      int el = 0;
      if (p.slot_expert) {
        const int e = p.slot_expert[slot];
        owned = e >= p.e_lo && e < p.e_hi;
        el = owned ? e - p.e_lo : 0;
      }
      const int xrow = p.slot_mode ? slot / p.x_div : 0;
      const uint8_t* xbase = xs + (size_t)xrow * xrow_bytes;
      float acc[GATED ? 2 : RPW][MM];
#pragma unroll
      for (int r = 0; r < (GATED ? 2 : RPW); ++r)
#pragma unroll
        for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;
      if (owned && ok) {
        for (int kc = 0; kc < p.nkc; ++kc, ++it) {
          if (CACHED && x_tag != xrow * p.nkc + kc) {
            x_tag = xrow * p.nkc + kc;
#pragma unroll
            for (int j = 0; j < NG; ++j)
              if (xl + 32 * j < ng) load_xg<FMT>(xbase, kc * ng + xl + 32 * j, K, xc[j]);
          }
          const int s = it % NST;
          ok = mbar_wait(bar0 + 8 * s, (it / NST) & 1, p.status, ERR_MBAR_TIMEOUT_EPILOGUE, abort_flag);
          if (!ok) break;
          const uint8_t* st = stages + (size_t)s * stage_bytes;
          if (half) {
            if constexpr (HALF_OK) {
              const int hr = lane >> 4;
              const int srow = GATED ? (hr == 0 ? 0 : FB) + warp : warp * RPW + hr;
              const GsPlanes23 w23{st + plane2_off + (size_t)srow * r2b, st + plane3_off + (size_t)srow * r3b, kc * (p.KC >> 8)};
              float a[MM];
#pragma unroll
              for (int m = 0; m < MM; ++m) a[m] = 0.f;
              gs_row<FMT, MM, CACHED, NG>(st + (size_t)srow * r0b, st + plane1_off + (size_t)srow * r1b, w23, ng, xl, xc, xbase, K, kc * ng,
                                      xscale + xrow, a);
#pragma unroll
              for (int m = 0; m < MM; ++m) {
                acc[0][m] += hr == 0 ? a[m] : 0.f;
                acc[1][m] += hr == 1 ? a[m] : 0.f;
              }
            }
          } else
#pragma unroll
          for (int r = 0; r < (GATED ? 2 : RPW); ++r) {
            // gated: the warp owns one feature of the block; its gate row sits at `warp`, its up row FB rows further
            const int srow = GATED ? (r == 0 ? 0 : FB) + warp : warp * RPW + r;
            const GsPlanes23 w23{st + plane2_off + (size_t)srow * r2b, st + plane3_off + (size_t)srow * r3b, kc * (p.KC >> 8)};
            gs_row<FMT, MM, CACHED, NG>(st + (size_t)srow * r0b, st + plane1_off + (size_t)srow * r1b, w23, ng, lane, xc, xbase, K, kc * ng,
                                    xscale + xrow, acc[r]);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar0 + 8 * (GS_MAX_STAGES + s));
        }
      }
      // ---- epilogue of this unit
#pragma unroll
      for (int r = 0; r < (GATED ? 2 : RPW); ++r)
#pragma unroll
        for (int m = 0; m < MM; ++m) acc[r][m] = warp_sum(acc[r][m]);
      if (lane == 0) {
        const float oscale = p.slot_scale ? p.slot_scale[slot] : 1.f;
        if (GATED) {
          const int f = blk * FB + warp;
          if (f < F) {
            const int grow = 32 * (f >> 4) + (f & 15);
            const float* bias = p.bias ? p.bias + (size_t)el * p.N : nullptr;
            const float g = acc[0][0] + (bias ? bias[grow] : 0.f), uu = acc[1][0] + (bias ? bias[grow + 16] : 0.f);
            const float v = owned ? gs_act(p.act, g, uu, p.act_alpha, p.act_limit) * oscale : 0.f;
            if (p.out_f32) ((float*)p.y)[(size_t)slot * F + f] = v;
            else ((__nv_bfloat16*)p.y)[(size_t)slot * F + f] = __float2bfloat16(v);
          }
        } else {
#pragma unroll
          for (int r = 0; r < RPW; ++r) {
            const int n = blk * RB + warp * RPW + r;
            if (n >= p.N) continue;
            const float* bias = p.bias ? p.bias + (size_t)el * p.N : nullptr;
#pragma unroll
            for (int m = 0; m < MM; ++m) {
              if (!p.slot_mode && m >= p.M) break;
              const size_t orow = p.slot_mode ? (size_t)slot : (size_t)m;
              const float v = owned ? (acc[r][m] + (bias ? bias[n] : 0.f)) * oscale : 0.f;
              if (p.peer.world) {
                for (int d = 0; d < p.peer.world; ++d) reinterpret_cast<float*>(peer_slot(p.peer, d, next_seq))[orow * p.N + n] = v;
              } else if (p.out_f32) ((float*)p.y)[orow * p.N + n] = v;
              else ((__nv_bfloat16*)p.y)[orow * p.N + n] = __float2bfloat16(v);
            }
          }
        }
      }
    }
  }
  if (p.peer.world) {
    pdl_wait();                               // (producer warp: its lanes take part in the block-wide publish)
    peer_publish(p.peer, next_seq);
  }
  if (p.route.ticket) {
    // ---- router tail: the last CTA to finish routes the tokens and writes their MXFP8 pair tiles
    __shared__ int s_last;
    pdl_wait();
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int prev = atomicAdd(p.route.ticket, 1);
      s_last = prev == (int)gridDim.x - 1;
      if (s_last) *p.route.ticket = 0;        // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const GsRoute& rt = p.route;
    for (int t = warp; t < p.M; t += WARPS + 1) route_token_warp((const float*)p.y, rt.bias, t, p.N, rt.Kt, rt.renorm, rt.topk_idx, rt.topk_w, rt.w_copies);
    // xs holds the normalised bf16 rows this CTA multiplied: one thread per (row, 32-element block)
    const int Kp = rt.KB * MXF_KBLOCK, nblk = rt.KB * 4;
    for (int u = threadIdx.x; u < p.M * nblk; u += blockDim.x) {
      const int t = u / nblk, blk = u - t * nblk, k0 = blk * 32;
      float v[32];
      float amax = 0.f;
      if (k0 < K) {
        const uint4* src = reinterpret_cast<const uint4*>(xs + ((size_t)t * K + k0) * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 raw = src[i];
          const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            v[8 * i + 2 * jj] = bf16_lo(w4[jj]);
            v[8 * i + 2 * jj + 1] = bf16_hi(w4[jj]);
            amax = fmaxf(amax, fmaxf(fabsf(v[8 * i + 2 * jj]), fabsf(v[8 * i + 2 * jj + 1])));
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      float inv;
      const uint32_t eb = mxfp8_scale(amax, &inv);
      const uint4 lo = make_uint4(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv), e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                                  e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv), e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
      const uint4 hi = make_uint4(e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv), e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv),
                                  e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv), e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv));
      for (int k = 0; k < rt.Kt; ++k) {
        const size_t r = (size_t)t * rt.Kt + k;
        uint4* d = reinterpret_cast<uint4*>(rt.xq + r * Kp + k0);
        d[0] = lo;
        d[1] = hi;
        rt.sfx[((size_t)(blk >> 2) * rt.max_tiles + r) * SF_ATOM + sf_atom_offset(0, blk & 3)] = (uint8_t)eb;
      }
    }
  }
}

template <int FMT, int MM, bool GATED, int NG>
static int gs_launch(const GsParams& p, int smem, cudaStream_t st) {
  constexpr int THREADS = (GsCfg<FMT>::WARPS + 1) * 32;
  static DeviceOnce attr_done;
  if (attr_done.pending()) {
    cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<FMT, MM, GATED, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done.mark();
  }
  const int units = p.slots * p.nblk;
  const int per_sm = smem <= 113 * 1024 ? 2 : 1;
  const int grid = min(units, sm_count() * per_sm);
  // Chunked rows: a stage is RB row segments that are not contiguous in memory.  One tiled TMA load per plane fetches them all
  // (the planes as 2-D byte tensors [rows][row bytes], box = chunk bytes x rows of the stage); segments wider than a box (bf16) and
  // expert stacks of unknown extent keep the per-row bulk copies.
  CUtensorMap tm[3];
  std::memset(tm, 0, sizeof(tm));
  GsParams q = p;
  q.use_tma = 0;
  if (g_gs_tma && p.nkc > 1 && p.tma_rows > 0) {
    constexpr int RB = GsCfg<FMT>::WARPS * GsCfg<FMT>::RPW;
    const uint32_t box_rows = GATED ? RB / 2 : RB;
    const int cb[3] = {gs_stage_row0<FMT>(p.K, p.KC), gs_stage_row1<FMT>(p.K, p.KC), gs_stage_row2<FMT>(p.K, p.KC)};
    const int rbytes[3] = {gs_row_bytes0<FMT>(p.K), gs_row_bytes1<FMT>(p.K), gs_row_bytes2<FMT>(p.K)};
    const void* base[3] = {p.w.p0, p.w.p1, p.w.p2};
    bool ok = true;
    for (int i = 0; i < 3 && ok; ++i) {
      if (!cb[i]) continue;
      // the tensor's rows are the used bytes of each plane row (chunks x chunk bytes); the pitch is the plane's row stride
      ok = cb[i] <= 2048 && make_tmap_bytes(&tm[i], base[i], (uint64_t)cb[i] * p.nkc, (uint64_t)p.tma_rows, (uint64_t)rbytes[i], (uint32_t)cb[i], box_rows) == 0;
    }
    q.use_tma = ok ? 1 : 0;
  }
  launch_pdl(gemv_stream_kernel<FMT, MM, GATED, NG>, dim3(grid), dim3(THREADS), (size_t)smem, st, q, tm[0], tm[1], tm[2]);
  return (int)cudaGetLastError();
}

template <int FMT, int NG>
static int gs_dispatch_ng(GsParams& p, int smem, bool gated, cudaStream_t st) {
  if (gated) {
    if constexpr (FMT == WF_Q6K || GsCfg<FMT>::RPW != 2) return 1;       // no gated form (four planes, or one row per warp)
    else return gs_launch<FMT, 1, true, NG>(p, smem, st);
  }
  if (p.slot_mode || p.M == 1) return gs_launch<FMT, 1, false, NG>(p, smem, st);
  if (FMT == WF_MXFP4) return 1;
  if (p.M <= 2) return gs_launch<FMT, 2, false, NG>(p, smem, st);
  if (p.M <= 4) return gs_launch<FMT, 4, false, NG>(p, smem, st);
  return gs_launch<FMT, 8, false, NG>(p, smem, st);
}

template <int FMT>
static int gs_dispatch(GsParams& p, cudaStream_t st) {
  constexpr int WARPS = GsCfg<FMT>::WARPS, RPW = GsCfg<FMT>::RPW, RB = WARPS * RPW;
  const bool gated = p.act != 0;
  p.KC = p.K; p.nkc = 1;
  if (gs_is_bf16(FMT) && p.K > 4096) {
    int n = (p.K + 4095) / 4096;
    while (n < 64 && (p.K % n || (p.K / n) % 8)) ++n;
    if (p.K % n) return 1;
    p.nkc = n; p.KC = p.K / n;
  }
  if ((FMT == WF_Q4K || FMT == WF_Q6K || FMT == WF_Q8I) && p.K > 32 * Gran<FMT>::NGMAX * Gran<FMT>::GE) {
    // whole 256-element blocks per chunk, as few chunks as possible: the per-row copies of a chunked matrix are bound by the
    // rate of bulk-copy requests, not by bytes (chunks of at most 1024 elements are taken by half-warps, see the consumer loop)
    int n = 2;
    while (n < 64 && (p.K % n || (p.K / n) % 256 || p.K / n > 32 * Gran<FMT>::NGMAX * Gran<FMT>::GE)) ++n;
    if (n >= 64) return 1;
    p.nkc = n; p.KC = p.K / n;
  }
  if (p.KC / Gran<FMT>::GE > 32 * Gran<FMT>::NGMAX || p.KC % Gran<FMT>::GE) return 1;
  if (gated && p.nkc > 1 && gs_row_bytes1<FMT>(p.K) && FMT != WF_Q8I) return 1;
  if (FMT == WF_MXFP4 && p.K > 4096) return 1;
  p.nblk = gated ? (p.N / 2 + RB / 2 - 1) / (RB / 2) : (p.N + RB - 1) / RB;
  const int stage = RB * gs_stage_row_all<FMT>(p.K, p.KC);
  const int fixed = ((p.n_xrows * gs_xrow_bytes<FMT>(p.K) + 127) & ~127) + 128 + 2 * GS_MAX_STAGES * 8 + GS_MAX_XROWS * 4 + 16;
  p.nst = GS_MAX_STAGES;
  while (p.nst > 2 && fixed + p.nst * stage > 113 * 1024) --p.nst;        // two CTAs per SM when three stages still fit
  if (fixed + p.nst * stage > 113 * 1024) p.nst = min(GS_MAX_STAGES, max(2, (200 * 1024 - fixed) / stage));
  const int smem = fixed + p.nst * stage;
  if (smem > 200 * 1024 || p.nst < 2) return 1;
  // granules per lane: 3/4 of the maximum covers K <= 3072 with a quarter fewer registers
  constexpr int NGS = Gran<FMT>::NGMAX * 3 / 4;
  if constexpr (NGS >= 1) {
    if (p.KC / Gran<FMT>::GE <= 32 * NGS) return gs_dispatch_ng<FMT, NGS>(p, smem, gated, st);
  }
  return gs_dispatch_ng<FMT, Gran<FMT>::NGMAX>(p, smem, gated, st);
}

// Returns 0 when the kernel was launched, 1 when the shape / format is not taken by this path (the caller falls
// back to the register-streamed kernels), a CUDA error code otherwise.
static int gemv_stream_fused(int wfmt, const WeightRef& w, const void* x, void* y, const float* bias, int M, int N, int K, int out_f32, int act,
                             float act_alpha, float act_limit, const int* slot_expert, const float* slot_scale, int slots, int x_div, int e_lo,
                             int e_hi, const PeerOut* peer, const GsNorm* norm, const GsRoute* route, cudaStream_t st);

int gemv_stream_try(int wfmt, const WeightRef& w, const void* x, void* y, const float* bias, int M, int N, int K, int out_f32, int act,
                    float act_alpha, float act_limit, const int* slot_expert, const float* slot_scale, int slots, int x_div, int e_lo,
                    int e_hi, const PeerOut* peer, cudaStream_t st) {
  return gemv_stream_fused(wfmt, w, x, y, bias, M, N, K, out_f32, act, act_alpha, act_limit, slot_expert, slot_scale, slots, x_div, e_lo, e_hi, peer,
                           nullptr, nullptr, st);
}

static int gemv_stream_fused(int wfmt, const WeightRef& w, const void* x, void* y, const float* bias, int M, int N, int K, int out_f32, int act,
                             float act_alpha, float act_limit, const int* slot_expert, const float* slot_scale, int slots, int x_div, int e_lo,
                             int e_hi, const PeerOut* peer, const GsNorm* norm, const GsRoute* route, cudaStream_t st) {
  if (wfmt != WF_BF16 && wfmt != WF_Q8 && wfmt != WF_MXFP4 && wfmt != WF_Q4K && wfmt != WF_Q6K) return 1;
  if (K % 32 && !(wfmt == WF_BF16 && K % 8 == 0)) return 1;
  if ((wfmt == WF_Q4K || wfmt == WF_Q6K) && K % 256) return 1;
  if (act != 0 && wfmt != WF_MXFP4 && wfmt != WF_Q4K && !(wfmt == WF_Q8 && !norm && !route)) return 1;      // gated epilogue: one feature per warp needs RPW == 2
  if (act != 0 && (N % 32)) return 1;
  GsParams p;
  p.w = w; p.x = (const __nv_bfloat16*)x; p.y = y; p.bias = bias; p.slot_expert = slot_expert; p.slot_scale = slot_scale;
  p.x_div = x_div > 0 ? x_div : 1; p.e_lo = e_lo; p.e_hi = e_hi; p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32; p.act = act;
  p.act_alpha = act_alpha; p.act_limit = act_limit; p.status = status_word();
  p.slot_mode = (slot_expert != nullptr || act != 0) ? 1 : 0;
  p.slots = p.slot_mode ? (slots > 0 ? slots : M) : 1;
  p.n_xrows = p.slot_mode ? (p.slots + p.x_div - 1) / p.x_div : M;
  if (p.n_xrows < 1 || p.n_xrows > GS_MAX_XROWS) return 1;
  // every plane row must start on a 16-byte boundary for the bulk copies
  const int rb0 = wfmt == WF_BF16 ? K * 2 : (wfmt == WF_Q8 ? K : (wfmt == WF_Q4K ? K / 256 * 144 : K / 2));
  if (rb0 % 16) return 1;
  if (((uintptr_t)w.p0 & 15) || (w.p1 && ((uintptr_t)w.p1 & 15)) || ((uintptr_t)x & 15)) return 1;
  if (wfmt == WF_Q6K && (!w.p2 || !w.p3 || ((uintptr_t)w.p2 & 15) || ((uintptr_t)w.p3 & 15))) return 1;
  p.use_tma = 0;
  p.tma_rows = slot_expert ? ((e_hi > e_lo && e_hi - e_lo <= 65536) ? (long long)(e_hi - e_lo) * N : 0) : N;
  if (peer) p.peer = *peer; else p.peer.world = 0;
  if (norm) p.norm = *norm; else p.norm.x = nullptr;
  if (route) p.route = *route; else p.route.ticket = nullptr;
  if ((norm || route) && (wfmt == WF_MXFP4 || wfmt == WF_Q4K || wfmt == WF_Q6K || p.slot_mode)) return 1;
  switch (wfmt) {
    case WF_BF16: return g_gs_bf16_wide ? gs_dispatch<WF_BF16W>(p, st) : gs_dispatch<WF_BF16>(p, st);
    case WF_Q8: return (norm || route) ? gs_dispatch<WF_Q8>(p, st) : gs_dispatch<WF_Q8I>(p, st);
    case WF_Q4K: return gs_dispatch<WF_Q4K>(p, st);
    case WF_Q6K: return gs_dispatch<WF_Q6K>(p, st);
    default: return gs_dispatch<WF_MXFP4>(p, st);
  }
}

}  // namespace mx
MX_HOST_API void mx_gemv_stream_set_tma(int on) { mx::g_gs_tma = on ? 1 : 0; }
MX_HOST_API void mx_gemv_stream_set_bf16_wide(int on) { mx::g_gs_bf16_wide = on ? 1 : 0; }
namespace mx {

// One ticket word per launch of a router GEMV with the routing tail; launches rotate through the words (see attention.cu).
constexpr int GS_TICKET_SLOTS = 8;
static __device__ int g_gs_tickets[GS_TICKET_SLOTS];

}  // namespace mx

using namespace mx;

// y[M][N] = (RMSNorm(x + delta_scale * delta) * norm_w) W^T + bias for M <= 2 rows of at most 4096 elements, W bf16 or Q8 (dense, one expert).
//   x fp32 [M][K]; delta: bf16 [M][K] (delta != null), or the expert combine sum_k cw[m][k] * yp[pos[m][k]] (yp != null, ck <= 8), or none.
//   x_out (required with a delta, must not alias x): the updated residual; h_out (optional): the normalised rows as bf16.
//   route (E = N experts, fp32 logits in y): topk_idx [M][Kt], topk_w [M][w_copies][Kt] and the rows as MXFP8 pair tiles xq / sfx (see mx_moe_route_quant).
// Returns 1 when the shape or format is not taken (the caller runs the separate kernels instead).
MX_HOST_API int mx_gemv_norm(int wfmt, const void* w0, const void* w1, const float* x, float* x_out, const void* delta, const void* yp, const int* pos,
                             const float* cw, int ck, const float* norm_w, float eps, int one_plus_w, float delta_scale, void* h_out, void* y,
                             const float* bias, int M, int N, int K, int out_f32, int route, const float* route_bias, int Kt, int renorm,
                             int* topk_idx, float* topk_w, int w_copies, void* xq, void* sfx, int max_tiles, cudaStream_t st) {
  if (M < 1 || M > GS_NORM_MAX_M || K % 8 || K > GS_NORM_MAX_K || ck > GS_MAX_CK) return 1;
  if ((delta || yp) && (!x_out || x_out == x)) return -150;
  GsNorm nm;
  nm.x = x; nm.x_out = (delta || yp) ? x_out : nullptr; nm.delta = yp ? nullptr : (const __nv_bfloat16*)delta;
  nm.yp = (const __nv_bfloat16*)yp; nm.pos = pos; nm.cw = cw; nm.ck = yp ? ck : 0;
  nm.w = norm_w; nm.eps = eps; nm.delta_scale = delta_scale; nm.one_plus_w = one_plus_w; nm.h_out = (__nv_bfloat16*)h_out;
  GsRoute rt;
  rt.ticket = nullptr;
  if (route) {
    if (!out_f32 || N > 1024 || Kt > 32 || Kt > N || K % 32 || max_tiles < M * Kt) return -151;
    static int* base[64] = {nullptr};
    static unsigned turn[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!base[dev]) {
      void* a = nullptr;
      if (cudaGetSymbolAddress(&a, g_gs_tickets) != cudaSuccess) return -152;
      base[dev] = (int*)a;
    }
    rt.ticket = base[dev] + turn[dev]++ % GS_TICKET_SLOTS;
    rt.bias = route_bias; rt.Kt = Kt; rt.renorm = renorm; rt.topk_idx = topk_idx; rt.topk_w = topk_w; rt.w_copies = w_copies < 1 ? 1 : w_copies;
    rt.xq = (uint8_t*)xq; rt.sfx = (uint8_t*)sfx; rt.KB = (K + MXF_KBLOCK - 1) / MXF_KBLOCK; rt.max_tiles = max_tiles;
  }
  return gemv_stream_fused(wfmt, WeightRef{w0, w1, nullptr, nullptr}, x, y, bias, M, N, K, out_f32, 0, 0.f, 0.f, nullptr, nullptr, 0, 1, 0, 1 << 30,
                           nullptr, &nm, route ? &rt : nullptr, st);
}
