// Gated DeltaNet scan in chunked (WY) form on the tensor cores: prefill-sized sequences.
//
// The recurrence per head (state S [v = 128][k = 128], fp32):   S <- e^g S;  d = (v - S k) beta;  S <- S + d k^T;  o = S q
// is a chain of T dependent rank-1 updates in the sequential kernel (deltanet.cu).  Over a chunk of C = 64 tokens with the
// cumulative log-decay G_i = g_0 + ... + g_i it has the closed form
//     (I + A) U = beta V - diag(beta e^G) K S0^T,        A_ij = beta_i e^{G_i - G_j} (k_i . k_j) for j < i  (strictly lower)
//     O = diag(e^G) Q S0^T + M U,                        M_ij = e^{G_i - G_j} (q_i . k_j) for j <= i
//     S = e^{G_last} S0 + U^T diag(e^{G_last - G}) K
// so that only three small matrix products per chunk depend on the running state.  Two kernels:
//
//   dn_chunk_prep_kernel  one CTA per (chunk, v-head), all chunks in parallel.  L2-normalises q and k, forms the gates, K K^T and Q K^T
//       with one tcgen05.mma (M = 128: K rows then Q rows; N = 64; accumulator in TMEM), then solves (I + A) W = [beta V | beta e^G K]
//       by forward substitution in fp32 (one thread per right-hand-side column, the column in registers) and writes the chunk's
//       operands as ready-made shared-memory images (128-byte-swizzled K-major tiles): [e^G Q ; W_k], M, (e^{G_last - G} K)^T, W_v.
//   dn_chunk_scan_kernel  one CTA per (sequence, v-head, half of the v columns), chunks in order.  The state slice lives in registers
//       (thread = k index, 64 v columns each) and goes to shared memory as a bf16 hi + lo pair (an MN-major B operand) once per
//       chunk.  Per chunk:  [e^G Q ; W_k] S0^T -> TMEM (rows 0..63 start the output, rows 64..127 are W_k S0^T);  U = W_v - W_k S0^T
//       -> bf16 tile;  M U accumulates onto the output rows and (e^{G_last - G} K)^T U gives the state increment, both in one MMA
//       batch;  the threads fold the increment into their registers.  The next chunk's images arrive by bulk copies meanwhile.
//
// Rows past a sequence's end are padded with beta = 0, g = 0, k = q = v = 0 (identity steps).  The kernel keeps no per-position
// checkpoints: speculative verify batches (a few tokens) stay on the sequential kernel.  Every wait is bounded (status word).
//
// Reference parity: research/05_deltanet_math.md:349-367 (the chunked form), src/ops/deltanet.cpp:410-480 (the sequential original).
#include "common.cuh"
#include "host_util.h"

namespace mx {

using bf16 = __nv_bfloat16;

constexpr int DC = 64;            // chunk length
constexpr int DD = 128;           // head width (k and v)
constexpr int DC_VS = 64;         // v columns per scan CTA
// workspace of one (chunk, head): byte offsets
constexpr int WS_A1 = 0;          // [e^G Q ; W_k]: 128 x 128 bf16 as two K atoms of 16 KiB
constexpr int WS_MQK = 32768;     // M: 64 x 64 bf16, rows 0..63 of one K atom (8 KiB)
constexpr int WS_KDT = 40960;     // (e^{G_last - G} K)^T: 128 x 64 bf16, one K atom (16 KiB)
constexpr int WS_WV = 57344;      // W_v fp32 as [v half][column quad 16][row 64][4] (32 KiB)
constexpr int WS_BYTES = 90112;

struct ChunkParams {
  const bf16* qkv; int ld, q_off, k_off, v_off;
  const bf16* ab; int ab_ld;
  const int* a_idx; const int* b_idx; const int* k_of_v;
  const float* ssm_a; const float* dt_bias;
  const int* cu_q; int B, n_v;
  float q_scale, eps;
  uint8_t* ws; float* egl; int max_chunks;
  float* state; const int* slots; float* out;
  int* status;
};

// chunk index -> (sequence, first token, live rows); false: past the last chunk
__device__ __forceinline__ bool dc_locate(const int* __restrict__ cu_q, int B, int ci, int& b, int& t0, int& n) {
  int base = 0;
  for (b = 0; b < B; ++b) {
    const int len = cu_q[b + 1] - cu_q[b];
    const int nc = (len + DC - 1) / DC;
    if (ci < base + nc) {
      const int c = ci - base;
      t0 = cu_q[b] + c * DC;
      n = min(DC, len - c * DC);
      return true;
    }
    base += nc;
  }
  return false;
}

// ------------------------------------------------------------------------------------------------ prep
struct PrepSmem {
  static constexpr int AK = 0;                 // [K ; Q] normalised, bf16, two K atoms (32 KiB)
  static constexpr int A1 = 32768;             // image of [e^G Q ; W_k]
  static constexpr int KDT = 65536;            // image of (e^{G_last - G} K)^T
  static constexpr int MISC = 81920;           // barrier, TMEM slot, abort flag
  static constexpr int TOTAL = MISC + 256 + 1024;
};

// (shared-window load: a pointer derived from the aligned dynamic base would compile to a generic load)
__device__ __forceinline__ float lds_bf16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return __uint_as_float((uint32_t)v << 16);
}

__global__ void __launch_bounds__(256, 2) dn_chunk_prep_kernel(const ChunkParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  // Arrays the threads read in their inner loops are static: the dynamic window's pointers come from integer arithmetic (the 1024-byte
  // alignment), so dereferencing them compiles to generic loads, which take the long-latency path.
  __shared__ __align__(16) float sA[DC * DC];                          // A, fp32
  __shared__ float sg[DC], sbeta[DC];                                  // g then G (cumulative), beta
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PrepSmem::MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  pdl_prologue();
  int b, t0, n;
  if (!dc_locate(p.cu_q, p.B, blockIdx.x, b, t0, n)) return;            // whole CTA, before any barrier / TMEM use
  const int kh = p.k_of_v[h];
  if (tid == 0) { mbar_init(smem_u32(bar), 1); *abort_flag = 0; fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), 64); tmem_relinquish(); }

  // A warp owns rows warp, warp + 8, ...; their loads are issued together and before the gate arithmetic, so that the eight rows cost
  // one trip to memory and that trip overlaps the gates and their prefix sum.
  uint2 qraw[DC / 8], kraw[DC / 8], vraw[DC / 8];
#pragma unroll
  for (int it = 0; it < DC / 8; ++it) {
    const int r = warp + 8 * it;
    qraw[it] = kraw[it] = vraw[it] = make_uint2(0u, 0u);
    if (r < n) {
      const bf16* row = p.qkv + (size_t)(t0 + r) * p.ld + lane * 4;
      qraw[it] = *reinterpret_cast<const uint2*>(row + p.q_off + kh * DD);
      kraw[it] = *reinterpret_cast<const uint2*>(row + p.k_off + kh * DD);
      vraw[it] = *reinterpret_cast<const uint2*>(row + p.v_off + h * DD);
    }
  }
  // gates
  if (tid < DC) {
    float g = 0.f, be = 0.f;
    if (tid < n) {
      const float a = __bfloat162float(p.ab[(size_t)(t0 + tid) * p.ab_ld + p.a_idx[h]]) + p.dt_bias[h];
      const float bb = __bfloat162float(p.ab[(size_t)(t0 + tid) * p.ab_ld + p.b_idx[h]]);
      g = p.ssm_a[h] * (fmaxf(a, 0.f) + log1pf(__expf(-fabsf(a))));       // softplus
      be = 1.f / (1.f + __expf(-bb));
    }
    sg[tid] = g;
    sbeta[tid] = be;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 0) {                       // inclusive prefix sum of the 64 gates: lane l holds elements 2l and 2l + 1
    const float g0 = sg[2 * lane], g1 = sg[2 * lane + 1];
    float v = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    sg[2 * lane] = v - g1;
    sg[2 * lane + 1] = v;
  }
  __syncthreads();
  const float Gl = sg[DC - 1];

  // rows: L2 norms, the [K ; Q] operand, e^G Q and (e^{G_last - G} K)^T
#pragma unroll
  for (int it = 0; it < DC / 8; ++it) {
    const int r = warp + 8 * it;
    const float q[4] = {bf16_lo(qraw[it].x), bf16_hi(qraw[it].x), bf16_lo(qraw[it].y), bf16_hi(qraw[it].y)};
    const float k[4] = {bf16_lo(kraw[it].x), bf16_hi(kraw[it].x), bf16_lo(kraw[it].y), bf16_hi(kraw[it].y)};
    const float iq = rsqrtf(warp_sum(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]) + p.eps) * p.q_scale;
    const float ik = rsqrtf(warp_sum(k[0] * k[0] + k[1] * k[1] + k[2] * k[2] + k[3] * k[3]) + p.eps);
    const float eg = __expf(sg[r]), ed = __expf(Gl - sg[r]);
    const uint32_t atom = (uint32_t)(lane >> 4) * 16384u, chunk = (lane & 15) >> 1, half = (lane & 1) * 8;
    *reinterpret_cast<uint2*>(smem + PrepSmem::AK + atom + sw128_offset(r, chunk) + half) =
        make_uint2(pack_bf16(k[0] * ik, k[1] * ik), pack_bf16(k[2] * ik, k[3] * ik));
    *reinterpret_cast<uint2*>(smem + PrepSmem::AK + atom + sw128_offset(64 + r, chunk) + half) =
        make_uint2(pack_bf16(q[0] * iq, q[1] * iq), pack_bf16(q[2] * iq, q[3] * iq));
    *reinterpret_cast<uint2*>(smem + PrepSmem::A1 + atom + sw128_offset(r, chunk) + half) =
        make_uint2(pack_bf16(q[0] * iq * eg, q[1] * iq * eg), pack_bf16(q[2] * iq * eg, q[3] * iq * eg));
#pragma unroll
    for (int i = 0; i < 4; ++i)          // transposed: element (k index, position r)
      *reinterpret_cast<bf16*>(smem + PrepSmem::KDT + sw128_offset(lane * 4 + i, r >> 3) + (r & 7) * 2) = __float2bfloat16(k[i] * ik * ed);
    // the raw v row waits in rows 64..127 of the [e^G Q ; W_k] image (W_k lands there after the substitution has read it)
    *reinterpret_cast<uint2*>(smem + PrepSmem::A1 + atom + 8192 + r * 128 + (lane & 15) * 8) = vraw[it];
  }
  fence_proxy_async();
  __syncthreads();

  // K K^T (rows 0..63) and Q K^T (rows 64..127)
  const uint32_t mbar = smem_u32(bar);
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, DC, 0, 0);
#pragma unroll
    for (int kk = 0; kk < DD / 16; ++kk) {
      const uint32_t off = sbase + PrepSmem::AK + (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem_base, umma_desc_k_sw128(off), umma_desc_k_sw128(off), idesc, kk != 0);
    }
    umma_commit(mbar);
  }
  const bool ok = mbar_wait(mbar, 0, p.status, ERR_MBAR_TIMEOUT_EPILOGUE, abort_flag, 32);
  tc_fence_after();
  uint8_t* ws = p.ws + ((size_t)blockIdx.x * p.n_v + h) * WS_BYTES;
  {
    // accumulator rows: warps w and w + 4 share TMEM lanes 32 (w % 4) .. + 31 and take columns 0..31 and 32..63
    const int row = (warp & 3) * 32 + lane, col0 = (warp >> 2) * 32;
    uint32_t c[32];
    if (ok) {
      tmem_ld_32x32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + col0, c);
      tmem_ld_wait();
    }
    if (ok && row < DC) {
      const int i = row;
      const float Gi = sg[i], bi = sbeta[i];
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4) {
        float a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = col0 + jj + u;
          a[u] = j < i ? bi * __expf(Gi - sg[j]) * __uint_as_float(c[jj + u]) : 0.f;
        }
        *reinterpret_cast<float4*>(sA + i * DC + col0 + jj) = make_float4(a[0], a[1], a[2], a[3]);
      }
    } else if (ok) {
      const int i = row - DC;
      const float Gi = sg[i];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float m[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int j = col0 + 8 * ch + u;
          m[u] = j <= i ? __expf(Gi - sg[j]) * __uint_as_float(c[8 * ch + u]) : 0.f;
        }
        *reinterpret_cast<uint4*>(ws + WS_MQK + sw128_offset(i, (col0 >> 3) + ch)) =
            make_uint4(pack_bf16(m[0], m[1]), pack_bf16(m[2], m[3]), pack_bf16(m[4], m[5]), pack_bf16(m[6], m[7]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // (I + A) W = [beta V | beta e^G K]: thread c owns column c of the right-hand side.  (Runs also after a wait that ran out: the block
  // contains a barrier, and what it then writes is never read, the status word being set.)
  {
    float w[DC];
    const int c = tid;
    // right-hand sides from shared memory: the staged v rows, and the normalised k rows of the [K ; Q] operand (rows past the
    // sequence's end are zero in both, and so is their beta)
    if (c < DD) {
      const uint32_t va = sbase + PrepSmem::A1 + (uint32_t)(c >> 6) * 16384u + 8192u + (c & 63) * 2;
#pragma unroll
      for (int i = 0; i < DC; ++i) w[i] = sbeta[i] * lds_bf16(va + i * 128);
    } else {
      const int e = c - DD;
      const uint32_t ka = sbase + PrepSmem::AK + (uint32_t)(e >> 6) * 16384u + (e & 7) * 2;
#pragma unroll
      for (int i = 0; i < DC; ++i) w[i] = sbeta[i] * __expf(sg[i]) * lds_bf16(ka + sw128_offset(i, (e & 63) >> 3));
    }
    __syncthreads();                     // every v row has been read: W_k may overwrite them
#pragma unroll
    for (int i = 1; i < DC; ++i) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int j = 0; j < (i & ~3); j += 4) {
        const float4 a = *reinterpret_cast<const float4*>(sA + i * DC + j);
        a0 = fmaf(a.x, w[j], a0); a1 = fmaf(a.y, w[j + 1], a1); a2 = fmaf(a.z, w[j + 2], a2); a3 = fmaf(a.w, w[j + 3], a3);
      }
#pragma unroll
      for (int j = (i & ~3); j < i; ++j) a0 = fmaf(sA[i * DC + j], w[j], a0);
      w[i] -= (a0 + a1) + (a2 + a3);
    }
    if (c < DD) {
      float* wv = reinterpret_cast<float*>(ws + WS_WV) + ((size_t)((c >> 6) * 16 + ((c & 63) >> 2)) * DC) * 4 + (c & 3);
#pragma unroll
      for (int i = 0; i < DC; ++i) wv[i * 4] = w[i];
    } else {
      const int e = c - DD;
      const uint32_t atom = (uint32_t)(e >> 6) * 16384u, chunk = (e & 63) >> 3, sub = (e & 7) * 2;
#pragma unroll
      for (int i = 0; i < DC; ++i)
        *reinterpret_cast<bf16*>(smem + PrepSmem::A1 + atom + sw128_offset(64 + i, chunk) + sub) = __float2bfloat16(w[i]);
    }
  }
  __syncthreads();
  if (ok) {
    const uint4* s1 = reinterpret_cast<const uint4*>(smem + PrepSmem::A1);
    uint4* d1 = reinterpret_cast<uint4*>(ws + WS_A1);
    for (int i = tid; i < 32768 / 16; i += 256) d1[i] = s1[i];
    const uint4* s2 = reinterpret_cast<const uint4*>(smem + PrepSmem::KDT);
    uint4* d2 = reinterpret_cast<uint4*>(ws + WS_KDT);
    for (int i = tid; i < 16384 / 16; i += 256) d2[i] = s2[i];
    if (tid == 0) p.egl[(size_t)blockIdx.x * p.n_v + h] = __expf(Gl);
  }
  if (warp == 0) tmem_dealloc(tmem_base, 64);
}

// ------------------------------------------------------------------------------------------------ scan
struct ScanSmem {
  static constexpr int A1 = 0;                 // per stage
  static constexpr int A2 = 32768;             // M in rows 0..63 of the atom, zeros in rows 64..127
  static constexpr int KDT = 49152;
  static constexpr int WV = 65536;             // this CTA's half of W_v (16 KiB)
  static constexpr int STAGE = 81920;
  static constexpr int LOAD_BYTES = 32768 + 8192 + 16384 + 16384;
  static constexpr int SHI = 2 * STAGE;        // state slice, bf16 high part: [k 128][v 64] (MN-major B)
  static constexpr int SLO = SHI + 16384;
  static constexpr int U = SLO + 16384;        // U: [position 64][v 64] bf16 (MN-major B)
  static constexpr int BARS = U + 8192;
  static constexpr int TOTAL = BARS + 256 + 1024;
  static_assert(TOTAL <= 232448, "shared memory plan exceeds 227 KB");
};

__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void dc_bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(128, 1) dn_chunk_scan_kernel(const ChunkParams p) {
  using L = ScanSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
  const uint32_t bar_load = smem_u32(bars), bar_mma = bar_load + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x >> 1, vs = blockIdx.x & 1, b = blockIdx.y;
  const int t_begin = p.cu_q[b], len = p.cu_q[b + 1] - t_begin;
  if (len <= 0) return;                                  // whole CTA, before any barrier / TMEM use
  const int nc = (len + DC - 1) / DC;
  int cb = 0;                                            // index of this sequence's first chunk
  for (int i = 0; i < b; ++i) cb += (p.cu_q[i + 1] - p.cu_q[i] + DC - 1) / DC;

  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_load + 8, 1); mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), 128); tmem_relinquish(); }
  // rows 64..127 of both M atoms stay zero (their products land on accumulator rows nobody reads again)
  for (int i = tid; i < 2 * 8192 / 16; i += 128) {
    const int stg = i / (8192 / 16), o = i % (8192 / 16);
    reinterpret_cast<uint4*>(smem + stg * L::STAGE + L::A2 + 8192)[o] = make_uint4(0, 0, 0, 0);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_lane = (uint32_t)(warp * 32) << 16;
  pdl_prologue();                                        // the images come from the prep kernel

  // thread = k index; registers hold S[v = vs * 64 + j][k] for j = 0..63
  float S[DC_VS];
  float* sp = p.state + (((size_t)p.slots[b] * p.n_v + h) * DD + vs * DC_VS) * DD + tid;
#pragma unroll
  for (int j = 0; j < DC_VS; ++j) S[j] = sp[(size_t)j * DD];

  auto issue_load = [&](int c) {
    const int stg = c & 1;
    const uint8_t* ws = p.ws + ((size_t)(cb + c) * p.n_v + h) * WS_BYTES;
    const uint32_t dst = sbase + stg * L::STAGE, bar = bar_load + 8 * stg;
    mbar_expect_tx(bar, L::LOAD_BYTES);
    dc_bulk(dst + L::A1, ws + WS_A1, 32768, bar);
    dc_bulk(dst + L::A2, ws + WS_MQK, 8192, bar);
    dc_bulk(dst + L::KDT, ws + WS_KDT, 16384, bar);
    dc_bulk(dst + L::WV, ws + WS_WV + vs * 16384, 16384, bar);
  };
  if (tid == 0) issue_load(0);

  constexpr uint32_t idesc = umma_idesc_bf16(128, DC_VS, 0, 1);          // B operands are MN-major (v contiguous)
  uint32_t mma_phase = 0;
  bool ok = true;
  for (int c = 0; c < nc && ok; ++c) {
    const int stg = c & 1;
    const uint32_t st = sbase + stg * L::STAGE;
    // the state slice as a bf16 pair: row k = this thread, 64 v values = 128 bytes per part
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float a = S[8 * ch + 2 * q], bq = S[8 * ch + 2 * q + 1];
        const bf16 ah = __float2bfloat16(a), bh = __float2bfloat16(bq);
        hi[q] = pack_bf16(__bfloat162float(ah), __bfloat162float(bh));
        lo[q] = pack_bf16(a - __bfloat162float(ah), bq - __bfloat162float(bh));
      }
      *reinterpret_cast<uint4*>(smem + L::SHI + sw128_offset(tid, ch)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(smem + L::SLO + sw128_offset(tid, ch)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      if (c + 1 < nc) issue_load(c + 1);                 // that stage's last readers (the MMAs of chunk c - 1) have completed
      if (mbar_wait(bar_load + 8 * stg, (c >> 1) & 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag)) {
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
          for (int kk = 0; kk < DD / 16; ++kk)
            umma_bf16(tmem_base, umma_desc_k_sw128(st + L::A1 + (kk >> 2) * 16384 + (kk & 3) * 32),
                      umma_desc_mn_sw128(sbase + (part ? L::SLO : L::SHI) + kk * 2048, DD * 128, 1024), idesc, (part | kk) != 0);
        umma_commit(bar_mma);
      }
    }
    if (!(ok = mbar_wait(bar_mma, mma_phase, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag, 32))) break;
    mma_phase ^= 1;
    tc_fence_after();
    // (every thread that reads the copied W_v observes the copy's barrier itself; thread 0 has seen it complete, so this returns at once)
    if (!(ok = mbar_wait(bar_load + 8 * stg, (c >> 1) & 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
    if (warp >= 2) {
      // U = W_v - W_k S0^T for position i, as one 128-byte row of the U tile
      const int i = tid - DC;
      uint32_t c0[32], c1[32];
      tmem_ld_32x32(tmem_base + tm_lane, c0);
      tmem_ld_32x32(tmem_base + tm_lane + 32, c1);
      tmem_ld_wait();
      const uint32_t wv = st + L::WV + i * 16;          // (shared-window loads: a pointer derived from the aligned base would be generic)
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const float4 w0 = lds_f4(wv + (2 * ch) * DC * 16), w1 = lds_f4(wv + (2 * ch + 1) * DC * 16);
        const uint32_t* src = ch < 4 ? c0 : c1;
        const int o = (ch & 3) * 8;
        *reinterpret_cast<uint4*>(smem + L::U + sw128_offset(i, ch)) =
            make_uint4(pack_bf16(w0.x - __uint_as_float(src[o]), w0.y - __uint_as_float(src[o + 1])),
                       pack_bf16(w0.z - __uint_as_float(src[o + 2]), w0.w - __uint_as_float(src[o + 3])),
                       pack_bf16(w1.x - __uint_as_float(src[o + 4]), w1.y - __uint_as_float(src[o + 5])),
                       pack_bf16(w1.z - __uint_as_float(src[o + 6]), w1.w - __uint_as_float(src[o + 7])));
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < DC / 16; ++kk)               // output rows += M U
        umma_bf16(tmem_base, umma_desc_k_sw128(st + L::A2 + kk * 32), umma_desc_mn_sw128(sbase + L::U + kk * 2048, DC * 128, 1024), idesc, 1);
#pragma unroll
      for (int kk = 0; kk < DC / 16; ++kk)               // state increment, transposed: [k][v]
        umma_bf16(tmem_base + DC_VS, umma_desc_k_sw128(st + L::KDT + kk * 32), umma_desc_mn_sw128(sbase + L::U + kk * 2048, DC * 128, 1024), idesc, kk != 0);
      umma_commit(bar_mma);
    }
    if (!(ok = mbar_wait(bar_mma, mma_phase, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag, 32))) break;
    mma_phase ^= 1;
    tc_fence_after();
    const int n = min(DC, len - c * DC);
    if (warp < 2) {
      uint32_t c0[32], c1[32];
      tmem_ld_32x32(tmem_base + tm_lane, c0);
      tmem_ld_32x32(tmem_base + tm_lane + 32, c1);
      tmem_ld_wait();
      if (tid < n) {
        float4* o = reinterpret_cast<float4*>(p.out + (size_t)(t_begin + c * DC + tid) * p.n_v * DD + h * DD + vs * DC_VS);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = make_float4(__uint_as_float(c0[4 * j]), __uint_as_float(c0[4 * j + 1]), __uint_as_float(c0[4 * j + 2]), __uint_as_float(c0[4 * j + 3]));
          o[8 + j] = make_float4(__uint_as_float(c1[4 * j]), __uint_as_float(c1[4 * j + 1]), __uint_as_float(c1[4 * j + 2]), __uint_as_float(c1[4 * j + 3]));
        }
      }
    }
    {
      const float eg = p.egl[(size_t)(cb + c) * p.n_v + h];
      uint32_t d0[32], d1[32];
      tmem_ld_32x32(tmem_base + tm_lane + DC_VS, d0);
      tmem_ld_32x32(tmem_base + tm_lane + DC_VS + 32, d1);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        S[j] = fmaf(eg, S[j], __uint_as_float(d0[j]));
        S[32 + j] = fmaf(eg, S[32 + j], __uint_as_float(d1[j]));
      }
    }
  }
  if (ok) {
#pragma unroll
    for (int j = 0; j < DC_VS; ++j) sp[(size_t)j * DD] = S[j];
  } else {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);     // a wait ran out: let copies in flight land before shared memory is released
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 128);
}

}  // namespace mx

using namespace mx;

// Bytes of workspace and number of per-(chunk, head) scalars for T tokens in B sequences (chunks <= T / 64 + B).
MX_HOST_API long long mx_deltanet_chunk_ws_bytes(int T, int B, int n_v) { return (long long)(T / DC + B) * n_v * WS_BYTES; }

// Chunked scan: same contract as mx_deltanet_scan without checkpoints.  `ws` holds mx_deltanet_chunk_ws_bytes(T, B, n_v) bytes
// (16-byte aligned), `egl` (T / 64 + B) * n_v floats.
MX_HOST_API int mx_deltanet_scan_chunked(const void* qkv, int ld, int q_off, int k_off, int v_off, const void* ab, int ab_ld, const int* a_idx,
                                         const int* b_idx, const int* k_of_v, const float* ssm_a, const float* dt_bias, float* state,
                                         const int* slots, const int* cu_q, int B, int T, int n_v, int head_dim, float q_scale, float eps,
                                         float* out, void* ws, float* egl, cudaStream_t st) {
  if (B <= 0 || n_v <= 0 || T <= 0) return 0;
  if (head_dim != DD || (ld & 3) || (q_off & 3) || (k_off & 3) || (v_off & 3) || ((uintptr_t)ws & 15)) return -101;
  ChunkParams p;
  p.qkv = (const bf16*)qkv; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.ab = (const bf16*)ab; p.ab_ld = ab_ld; p.a_idx = a_idx; p.b_idx = b_idx; p.k_of_v = k_of_v;
  p.ssm_a = ssm_a; p.dt_bias = dt_bias; p.cu_q = cu_q; p.B = B; p.n_v = n_v; p.q_scale = q_scale; p.eps = eps;
  p.ws = (uint8_t*)ws; p.egl = egl; p.max_chunks = T / DC + B;
  p.state = state; p.slots = slots; p.out = out; p.status = status_word();
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(dn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PrepSmem::TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ScanSmem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured.mark();
  }
  launch_pdl(dn_chunk_prep_kernel, dim3(p.max_chunks, n_v), dim3(256), (size_t)PrepSmem::TOTAL, st, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  launch_pdl(dn_chunk_scan_kernel, dim3(n_v * 2, B), dim3(128), (size_t)ScanSmem::TOTAL, st, p);
  return (int)cudaGetLastError();
}
