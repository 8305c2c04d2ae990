// EXL3 (trellis-coded) linear layers: y = had128(had128(x * suh) W_rot) * svh.
//
//   hadamard128_kernel   block-diagonal, normalised 128-point Sylvester Hadamard transform of activation rows with the
//                        per-feature sign / scale vector folded in before (suh) or after (svh, + bias): one warp per
//                        128-element run, four elements per lane (two butterfly stages in registers, five by shuffles)
//   exl3_dequant_kernel  trellis -> W_rot as bf16 [N][K], the operand of the tensor-core GEMM for prefill-sized batches
//   exl3_gemv_kernel     acc[M][N] = xh[M][K] W_rot for M <= 8 rows with the weights decoded in registers (decode steps)
//
// The trellis holds one cyclic bit stream of 256 * bits bits per 16 x 16 tile; weight t of the tile is the 16-bit window
// ending at bit (t + 1) * bits (most significant bit of each 32-bit word first), hashed into two fp16 values whose fp16 sum
// is the weight.  Lane l of a warp decodes the eight weights t = 8 l .. 8 l + 7, which sit at rows {2 (l % 4), +1, +8, +9}
// of columns {l / 4, l / 4 + 8} of the tile (the layout of a tensor-core fragment), so a tile's 32 lanes cover it exactly.
//
// Reference parity: src/ops/gemv_exl3.cpp:66,162 (decode GEMV), src/ops/hadamard.cpp:36,84 (transform),
// src/core/exl3_decode.cpp (bit extraction and codebook); host twin: csrc/host/exl3.cpp.
#include "common.cuh"
#include "host_util.h"

namespace mx {

constexpr int EXL3_MAX_M = 8;

__device__ __forceinline__ float exl3_code_value(uint32_t code) {
  uint32_t x = code * 89226354u + 64248484u;
  x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
  const __half lo = __ushort_as_half((unsigned short)(x & 0xffffu)), hi = __ushort_as_half((unsigned short)(x >> 16));
  return __half2float(__hadd(lo, hi));
}

// The warp holds the tile's 8 * bits words (word j in lane j % 32, register j / 32); returns this lane's eight weights.
// WIDE: more than 4 bits per weight, i.e. more than 32 words per tile (the second register is in use).
// The eight windows of a lane are consecutive: they cover bits [start, start + 7 bits + 16) of the cyclic stream with
// start = 8 lane bits + bits - 16, i.e. at most 75 bits (three words) up to 4 bits per weight and 103 bits (four words) above.  The lane
// fetches those words once by shuffles and cuts its windows out of them with funnel shifts.
template <bool WIDE>
__device__ __forceinline__ void exl3_decode8(uint32_t w_lo, uint32_t w_hi, int bits, int lane, float (&v)[8]) {
  constexpr int NW = WIDE ? 4 : 3;
  const int nwords = bits * 8;
  int start = lane * 8 * bits + bits - 16;
  if (start < 0) start += nwords * 32;
  const int wb = start >> 5, off0 = start & 31;
  uint32_t w[NW];
#pragma unroll
  for (int k = 0; k < NW; ++k) {
    int idx = wb + k;
    if (idx >= nwords) idx -= nwords;
    uint32_t a = __shfl_sync(0xffffffffu, w_lo, idx & 31);
    if constexpr (WIDE) {
      const uint32_t b = __shfl_sync(0xffffffffu, w_hi, idx & 31);
      a = idx < 32 ? a : b;
    }
    w[k] = a;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int o = off0 + j * bits;                 // first bit of window j inside w[]
    const int k = o >> 5;                          // <= 1 (2 when WIDE)
    uint32_t hi, lo;
    if constexpr (WIDE) {
      hi = k == 0 ? w[0] : (k == 1 ? w[1] : w[2]);
      lo = k == 0 ? w[1] : (k == 1 ? w[2] : w[3]);
    } else {
      hi = k == 0 ? w[0] : w[1];
      lo = k == 0 ? w[1] : w[2];
    }
    const uint32_t code = __funnelshift_l(lo, hi, o & 31) >> 16;       // bits [o, o + 16), most significant bit first
    v[j] = exl3_code_value(code);
  }
}

__device__ __forceinline__ void exl3_load_tile(const uint32_t* __restrict__ tile, int nwords, int lane, uint32_t& w_lo, uint32_t& w_hi) {
  w_lo = lane < nwords ? __ldg(tile + lane) : 0u;
  w_hi = lane + 32 < nwords ? __ldg(tile + lane + 32) : 0u;
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(128) hadamard128_kernel(const TI* __restrict__ x, const float* __restrict__ pre, const float* __restrict__ post,
                                                          const float* __restrict__ bias, TO* __restrict__ y, long long nruns, int n, int ldx, int ldy,
                                                          int nsum, long long sum_stride) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long run = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (run >= nruns) return;
  const int per_row = n >> 7;
  const long long row = run / per_row;
  const int col = (int)(run - row * per_row) * 128 + lane * 4;
  float v[4];
  if constexpr (sizeof(TI) == 2) {
    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + row * ldx + col);
    v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
  } else {
    const float4 r = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + row * ldx + col);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    for (int sidx = 1; sidx < nsum; ++sidx) {          // partial sums of a K-split product, added in a fixed order
      const float4 q = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + sidx * sum_stride + row * ldx + col);
      v[0] += q.x; v[1] += q.y; v[2] += q.z; v[3] += q.w;
    }
  }
  if (pre) {
    const float4 s = *reinterpret_cast<const float4*>(pre + col);
    v[0] *= s.x; v[1] *= s.y; v[2] *= s.z; v[3] *= s.w;
  }
  {
    const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
    v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? o - v[i] : v[i] + o;
    }
  }
  constexpr float NORM = 0.08838834764831845f;       // 1 / sqrt(128)
  float4 s = make_float4(1.f, 1.f, 1.f, 1.f), b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (post) s = *reinterpret_cast<const float4*>(post + col);
  if (bias) b = *reinterpret_cast<const float4*>(bias + col);
  v[0] = fmaf(v[0] * NORM, s.x, b.x); v[1] = fmaf(v[1] * NORM, s.y, b.y); v[2] = fmaf(v[2] * NORM, s.z, b.z); v[3] = fmaf(v[3] * NORM, s.w, b.w);
  if constexpr (sizeof(TO) == 2) {
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + row * ldy + col) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row * ldy + col) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

__global__ void __launch_bounds__(256) exl3_dequant_kernel(const uint32_t* __restrict__ trellis, int tile_k, int tile_n, int bits,
                                                           __nv_bfloat16* __restrict__ out) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long tile = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tile >= (long long)tile_k * tile_n) return;
  const int ki = (int)(tile / tile_n), ni = (int)(tile - (long long)ki * tile_n);
  const int nwords = bits * 8;
  uint32_t w_lo, w_hi;
  exl3_load_tile(trellis + tile * nwords, nwords, lane, w_lo, w_hi);
  float v[8];
  if (bits > 4) exl3_decode8<true>(w_lo, w_hi, bits, lane, v);
  else exl3_decode8<false>(w_lo, w_hi, bits, lane, v);
  const size_t K = (size_t)tile_k * 16;
  const int r0 = (lane & 3) * 2, c0 = lane >> 2;
  __nv_bfloat16* o0 = out + ((size_t)ni * 16 + c0) * K + (size_t)ki * 16 + r0;
  __nv_bfloat16* o1 = o0 + 8 * K;
  *reinterpret_cast<uint32_t*>(o0) = pack_bf16(v[0], v[1]);
  *reinterpret_cast<uint32_t*>(o0 + 8) = pack_bf16(v[2], v[3]);
  *reinterpret_cast<uint32_t*>(o1) = pack_bf16(v[4], v[5]);
  *reinterpret_cast<uint32_t*>(o1 + 8) = pack_bf16(v[6], v[7]);
}

// One CTA per (tile column, K range): 16 outputs over a slice of the K tiles.  Its eight warps stride over the slice's tiles, UNROLL
// tiles in flight per warp (one 128-byte load each at 4 bits per weight), and meet in shared memory; the CTA writes its partial sums
// to part[range][m][n], and the Hadamard kernel that follows adds the ranges (a fixed order: results do not depend on scheduling).
constexpr int EXL3_UNROLL = 4;

template <int MM, bool WIDE>
__global__ void __launch_bounds__(256) exl3_gemv_kernel(const uint32_t* __restrict__ trellis, int tile_k, int tile_n, int bits,
                                                        const __nv_bfloat16* __restrict__ xh, float* __restrict__ part, int M, int tiles_per_range) {
  pdl_prologue();
  __shared__ float red[8][MM][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ni = blockIdx.x;
  const int k_lo = blockIdx.y * tiles_per_range, k_hi = min(tile_k, k_lo + tiles_per_range);
  const int nwords = bits * 8;
  const size_t K = (size_t)tile_k * 16;
  const int r0 = (lane & 3) * 2;
  float s0[MM], s1[MM];
#pragma unroll
  for (int m = 0; m < MM; ++m) s0[m] = s1[m] = 0.f;
  for (int kb = k_lo + warp; kb < k_hi; kb += 8 * EXL3_UNROLL) {
    uint32_t w_lo[EXL3_UNROLL], w_hi[EXL3_UNROLL];
#pragma unroll
    for (int u = 0; u < EXL3_UNROLL; ++u) {
      const int ki = kb + 8 * u;
      w_lo[u] = w_hi[u] = 0u;
      if (ki < k_hi) {
        const uint32_t* tile = trellis + ((size_t)ki * tile_n + ni) * nwords;
        if (lane < nwords) w_lo[u] = __ldg(tile + lane);
        if (WIDE && lane + 32 < nwords) w_hi[u] = __ldg(tile + lane + 32);
      }
    }
#pragma unroll
    for (int u = 0; u < EXL3_UNROLL; ++u) {
      const int ki = kb + 8 * u;
      if (ki >= k_hi) break;                  // (uniform over the warp)
      float v[8];
      exl3_decode8<WIDE>(w_lo[u], w_hi[u], bits, lane, v);
#pragma unroll
      for (int m = 0; m < MM; ++m) {
        if (m < M) {
          const __nv_bfloat16* xp = xh + (size_t)m * K + (size_t)ki * 16 + r0;
          const uint32_t xa = __ldg(reinterpret_cast<const uint32_t*>(xp)), xb = __ldg(reinterpret_cast<const uint32_t*>(xp + 8));
          const float x0 = bf16_lo(xa), x1 = bf16_hi(xa), x2 = bf16_lo(xb), x3 = bf16_hi(xb);
          s0[m] += v[0] * x0 + v[1] * x1 + v[2] * x2 + v[3] * x3;
          s1[m] += v[4] * x0 + v[5] * x1 + v[6] * x2 + v[7] * x3;
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MM; ++m) {
    s0[m] += __shfl_xor_sync(0xffffffffu, s0[m], 1); s0[m] += __shfl_xor_sync(0xffffffffu, s0[m], 2);
    s1[m] += __shfl_xor_sync(0xffffffffu, s1[m], 1); s1[m] += __shfl_xor_sync(0xffffffffu, s1[m], 2);
    if ((lane & 3) == 0) {
      red[warp][m][lane >> 2] = s0[m];
      red[warp][m][(lane >> 2) + 8] = s1[m];
    }
  }
  __syncthreads();
  const size_t N = (size_t)tile_n * 16;
  for (int i = threadIdx.x; i < MM * 16; i += 256) {
    const int m = i >> 4, c = i & 15;
    if (m >= M) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][m][c];
    part[((size_t)blockIdx.y * M + m) * N + (size_t)ni * 16 + c] = s;
  }
}

}  // namespace mx

using namespace mx;

// y[rows][n] = had128(x * pre) * post + bias over every aligned run of 128 elements; x bf16 or fp32 (row stride ldx), y bf16 or fp32 (row stride ldy).
// nsum > 1 (fp32 input only): x is the sum of nsum matrices sum_stride elements apart.
MX_HOST_API int mx_hadamard128_cuda(const void* x, int x_f32, const float* pre, const float* post, const float* bias, void* y, int y_f32, long long rows,
                                    int n, int ldx, int ldy, int nsum, long long sum_stride, cudaStream_t st) {
  if (rows <= 0 || n <= 0) return 0;
  if (n % 128 || ldx % 4 || ldy % 4 || nsum < 1 || (nsum > 1 && (!x_f32 || sum_stride % 4))) return -160;
  const long long nruns = rows * (n / 128);
  const dim3 grid((unsigned)((nruns + 3) / 4)), block(128);
  if (x_f32 && y_f32) launch_pdl(hadamard128_kernel<float, float>, grid, block, 0, st, (const float*)x, pre, post, bias, (float*)y, nruns, n, ldx, ldy, nsum, sum_stride);
  else if (x_f32) launch_pdl(hadamard128_kernel<float, __nv_bfloat16>, grid, block, 0, st, (const float*)x, pre, post, bias, (__nv_bfloat16*)y, nruns, n, ldx, ldy, nsum, sum_stride);
  else if (y_f32) launch_pdl(hadamard128_kernel<__nv_bfloat16, float>, grid, block, 0, st, (const __nv_bfloat16*)x, pre, post, bias, (float*)y, nruns, n, ldx, ldy, nsum, sum_stride);
  else launch_pdl(hadamard128_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)x, pre, post, bias, (__nv_bfloat16*)y, nruns, n, ldx, ldy, nsum, sum_stride);
  return (int)cudaGetLastError();
}

// out: W_rot as bf16 [N][K] (N = 16 tile_n, K = 16 tile_k)
MX_HOST_API int mx_exl3_dequant_bf16(const void* trellis, int tile_k, int tile_n, int bits, void* out, cudaStream_t st) {
  if (tile_k <= 0 || tile_n <= 0) return 0;
  if (bits < 1 || bits > 8) return -161;
  const long long tiles = (long long)tile_k * tile_n;
  launch_pdl(exl3_dequant_kernel, dim3((unsigned)((tiles + 7) / 8)), dim3(256), 0, st, (const uint32_t*)trellis, tile_k, tile_n, bits, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

// part[ranges][M][N] (fp32): partial sums of xh[M][K] (bf16) W_rot over `ranges` slices of the K tiles (see mx_exl3_gemv_ranges), M <= 8
MX_HOST_API int mx_exl3_gemv_ranges(int tile_k, int tile_n) {
  // enough CTAs for about four per SM, at least eight tiles (one per warp) in a range, at most eight ranges
  const int want = (4 * sm_count() + tile_n - 1) / tile_n;
  int r = want < 1 ? 1 : (want > 8 ? 8 : want);
  while (r > 1 && tile_k / r < 8) --r;
  return r;
}

template <int MM>
static void exl3_gemv_launch(const uint32_t* t, int tile_k, int tile_n, int bits, const __nv_bfloat16* x, float* part, int M, int ranges, cudaStream_t st) {
  const int per = (tile_k + ranges - 1) / ranges;
  const dim3 grid((unsigned)tile_n, (unsigned)ranges), block(256);
  if (bits > 4) launch_pdl(exl3_gemv_kernel<MM, true>, grid, block, 0, st, t, tile_k, tile_n, bits, x, part, M, per);
  else launch_pdl(exl3_gemv_kernel<MM, false>, grid, block, 0, st, t, tile_k, tile_n, bits, x, part, M, per);
}

MX_HOST_API int mx_exl3_gemv(const void* trellis, int tile_k, int tile_n, int bits, const void* xh, float* part, int M, int ranges, cudaStream_t st) {
  if (tile_k <= 0 || tile_n <= 0 || M <= 0) return 0;
  if (bits < 1 || bits > 8 || M > EXL3_MAX_M || ranges < 1 || ranges > tile_k) return -162;
  const uint32_t* t = (const uint32_t*)trellis;
  const __nv_bfloat16* x = (const __nv_bfloat16*)xh;
  if (M == 1) exl3_gemv_launch<1>(t, tile_k, tile_n, bits, x, part, M, ranges, st);
  else if (M <= 2) exl3_gemv_launch<2>(t, tile_k, tile_n, bits, x, part, M, ranges, st);
  else if (M <= 4) exl3_gemv_launch<4>(t, tile_k, tile_n, bits, x, part, M, ranges, st);
  else exl3_gemv_launch<8>(t, tile_k, tile_n, bits, x, part, M, ranges, st);
  return (int)cudaGetLastError();
}
