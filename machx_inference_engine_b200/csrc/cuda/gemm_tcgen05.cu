// Persistent warp-specialised GEMM for sm_100a: C[M,N] = A[M,K] * W[N,K]^T (+ epilogue).
//
//   * A (bf16 activations, K-contiguous) arrives through TMA into 128-byte-swizzled tiles.
//   * W is either bf16 (also TMA) or a quantised runtime layout (Q8 / Q4_K / Q6_K planes /
//     MXFP4 planes) that eight producer warps decode in registers straight into the swizzled
//     B tile -- the weights are never materialised as fp16/bf16 in global memory.
//   * One elected thread issues tcgen05.mma (M=128, N=BN, K=16 per instruction); fp32
//     accumulators live in TMEM, double buffered so the epilogue of tile i overlaps the main
//     loop of tile i+1.
//   * Four epilogue warps read TMEM with tcgen05.ld and apply bias / activation / row scale.
//   * The same kernel runs grouped (MoE) problems: a per-m-tile expert id selects the weight
//     slab, and the number of live m-tiles is read from device memory, so no host round trip.
//
// Reference parity: replaces gemm_fp16 / gemm_fp16_onednn / gemm_q4k_xmx / dequant_*_bt + GEMM
// (src/ops/gemm_fp16.cpp:64, gemm_onednn.cpp:76-111, gemm_q4k_xmx.cpp:129-432,
// dequant_kernels.cpp) and the dispatcher in src/model/dense_dispatch.hpp:562-754, and the MoE
// prefill GEMMs of src/ops/moe_fused.cpp:568-1961.  Ragged K and N are handled natively.
#include "common.cuh"
#include "dequant.cuh"
#include "host_util.h"

namespace mx {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kNumEpilogueWarps = 4;
constexpr int kNumDequantWarps = 8;

enum Act : int { ACT_NONE = 0, ACT_SWIGLU = 1, ACT_SWIGLU_OAI = 2, ACT_GEGLU = 3 };

struct GemmParams {
  int M, N, K;
  int num_m_tiles;              // host upper bound
  int num_n_tiles;
  const int* num_m_tiles_dev;   // grouped: live m-tile count (device), else null
  const int* tile_expert;       // grouped: expert id per m-tile, else null
  WeightRef w;
  void* C;                      // bf16 or fp32, leading dimension ldc (elements)
  int ldc;
  int out_f32;
  const float* bias;            // [N] or [E][N], nullable
  const float* row_scale;       // [M], nullable
  int act;
  float act_alpha, act_limit;
  int* status;
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // + barriers + alignment slack
};

__device__ __forceinline__ float act_apply(int act, float g, float u, float alpha, float limit) {
  if (act == ACT_SWIGLU) return g / (1.f + __expf(-g)) * u;
  if (act == ACT_SWIGLU_OAI) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  // GeGLU, tanh approximation
  const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
  return 0.5f * g * (1.f + t) * u;
}

template <int FMT, int BN, int STAGES>
__global__ void __launch_bounds__(FMT == WF_BF16 ? 192 : 448, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  constexpr bool kDequant = FMT != WF_BF16;
  constexpr uint32_t TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);   // power of two for BN in {32,64,128,256}
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  // barrier slots: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, kDequant ? 1 + kNumDequantWarps * 32 : 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kNumEpilogueWarps * 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = p.num_m_tiles_dev ? min(*p.num_m_tiles_dev, p.num_m_tiles) : p.num_m_tiles;
  const int total_tiles = m_tiles * p.num_n_tiles;
  const int k_iters = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      if (!kDequant) prefetch_tmap(&tmap_b);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int mt = t % m_tiles, nt = t / m_tiles;
        const int e = p.tile_expert ? p.tile_expert[mt] : 0;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
          const uint32_t a_dst = smem_base + s * L::STAGE_BYTES;
          mbar_expect_tx(bar_full + 8 * s, kDequant ? L::A_BYTES : L::STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, bar_full + 8 * s, k * BK, mt * BM);
          if (!kDequant) tma_load_3d(a_dst + L::A_BYTES, &tmap_b, bar_full + 8 * s, k * BK, nt * BN, e);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
      uint32_t it = 0, tile_n = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_n) {
        const uint32_t acc = tile_n & 1, acc_ph = (tile_n >> 1) & 1;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!(ok = mbar_wait(bar_full + 8 * s, ph, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * L::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + L::A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)   // 16 bf16 = 32 bytes per UMMA K step: +2 in the (addr>>4) field
            umma_bf16(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (k | kk) != 0);
          umma_commit(bar_empty + 8 * s);
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);
      }
    }
  } else if (warp < 2 + kNumEpilogueWarps) {
    // ------------------------------------------------ epilogue: TMEM -> registers -> global
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    uint32_t tile_n = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_n) {
      const int mt = t % m_tiles, nt = t / m_tiles;
      const int e = p.tile_expert ? p.tile_expert[mt] : 0;
      const uint32_t acc = tile_n & 1, acc_ph = (tile_n >> 1) & 1;
      if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, p.status, ERR_MBAR_TIMEOUT_EPILOGUE, abort_flag))) break;
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float rs = (p.row_scale && row_ok) ? p.row_scale[row] : 1.f;
      const float* bias = p.bias ? p.bias + (size_t)e * p.N : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c0, r);
        tmem_ld_wait();
        const int col0 = nt * BN + c0;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] = __uint_as_float(r[j]);
          if (bias && col0 + j < p.N) v[j] += bias[col0 + j];
        }
        if (p.act == ACT_NONE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= rs;
          if (p.out_f32) {
            float* out = (float*)p.C + (size_t)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) out[j] = v[j];
            }
          } else {
            __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                *reinterpret_cast<uint4*>(out + j) = make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                                                                pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) out[j] = __float2bfloat16(v[j]);
            }
          }
        } else {
          // gate/up are interleaved in groups of 16 columns: [g0..g15 | u0..u15]; 16 outputs per 32 inputs
          const int ocol0 = col0 >> 1;
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = act_apply(p.act, v[j], v[16 + j], p.act_alpha, p.act_limit) * rs;
          const int on = p.N >> 1;
          if (p.out_f32) {
            float* out = (float*)p.C + (size_t)row * p.ldc + ocol0;
            for (int j = 0; j < 16 && ocol0 + j < on; ++j) out[j] = o[j];
          } else {
            __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + ocol0;
            if (ocol0 + 16 <= on && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 16; j += 8)
                *reinterpret_cast<uint4*>(out + j) = make_uint4(pack_bf16(o[j], o[j + 1]), pack_bf16(o[j + 2], o[j + 3]),
                                                                pack_bf16(o[j + 4], o[j + 5]), pack_bf16(o[j + 6], o[j + 7]));
            } else {
              for (int j = 0; j < 16 && ocol0 + j < on; ++j) out[j] = __float2bfloat16(o[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
  } else if (kDequant) {
    // ------------------------------------------------ weight decode producers (8 warps)
    const int d = threadIdx.x - (2 + kNumEpilogueWarps) * 32;   // 0..255
    uint32_t it = 0;
    bool ok = true;
    constexpr int ROWS_PER_PASS = kNumDequantWarps * 32 / 2;      // two threads per row (32 k-elements each)
    const int half = d & 1;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int mt = t % m_tiles, nt = t / m_tiles;
      const int e = p.tile_expert ? p.tile_expert[mt] : 0;
      const WeightRef we = p.tile_expert ? expert_weight<FMT>(p.w, e, p.N, p.K) : p.w;
      for (int k = 0; k < k_iters; ++k, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, p.status, ERR_MBAR_TIMEOUT_DEQUANT, abort_flag))) break;
        uint8_t* b_tile = smem + s * L::STAGE_BYTES + L::A_BYTES;
        const int kb = k * 2 + half;                              // 32-element block index along K
        const bool k_ok = kb * 32 < p.K;
#pragma unroll 1
        for (int r0 = 0; r0 < BN; r0 += ROWS_PER_PASS) {
          const int rl = r0 + (d >> 1);
          if (rl < BN) {
            const int n = nt * BN + rl;
            uint32_t o[16];
            if (n < p.N && k_ok) {
              const RowPtrs rp = row_ptrs<FMT>(we, n, p.K);
              decode32_bf16<FMT>(rp, kb, o);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = 0u;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(b_tile + sw128_offset(rl, 4 * half + c)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
          }
        }
        fence_proxy_async();
        mbar_arrive(bar_full + 8 * s);
      }
    }
  }

  // ---------------------------------------------------- teardown
  if (*abort_flag) {
    // a wait ran out: give copies still in flight time to land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------
template <int FMT, int BN, int STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_kernel<FMT, BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, FMT == WF_BF16 ? 192 : 448, L::TOTAL, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

template <int BN, int STAGES>
static int dispatch_fmt(int fmt, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  switch (fmt) {
    case WF_BF16: return launch<WF_BF16, BN, STAGES>(ta, tb, p, st);
    case WF_Q8: return launch<WF_Q8, BN, STAGES>(ta, tb, p, st);
    case WF_Q4K: return launch<WF_Q4K, BN, STAGES>(ta, tb, p, st);
    case WF_Q6K: return launch<WF_Q6K, BN, STAGES>(ta, tb, p, st);
    case WF_MXFP4: return launch<WF_MXFP4, BN, STAGES>(ta, tb, p, st);
    default: return -100;
  }
}

}  // namespace mx

// C[M, N(/2 with act)] = A[M,K] * W[(E,)N,K]^T.
//   a          bf16 [M,K] row-major, 16-byte aligned, K % 8 == 0
//   wfmt/w0..w3  weight format and plane pointers (see WFormat); n_experts >= 1
//   tile_expert / num_m_tiles_dev: grouped mode (both null for a plain GEMM)
//   bn         32, 64 or 128 (tile width); the caller picks small tiles for small M
// Returns 0 or a CUDA / driver error code.
MX_HOST_API int mx_gemm(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, int n_experts,
                        void* c, int ldc, int out_f32, const float* bias, const float* row_scale, int act, float act_alpha,
                        float act_limit, int M, int N, int K, const int* tile_expert, const int* num_m_tiles_dev, int bn,
                        cudaStream_t stream) {
  using namespace mx;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8) return -101;
  if (wfmt != WF_BF16 && (K % 32)) return -102;
  if ((wfmt == WF_Q4K || wfmt == WF_Q6K) && (K % 256)) return -103;
  if (act != ACT_NONE && (N % 32)) return -104;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + bn - 1) / bn;
  p.num_m_tiles_dev = num_m_tiles_dev;
  p.tile_expert = tile_expert;
  p.w = WeightRef{w0, w1, w2, w3};
  p.C = c; p.ldc = ldc; p.out_f32 = out_f32;
  p.bias = bias; p.row_scale = row_scale;
  p.act = act; p.act_alpha = act_alpha; p.act_limit = act_limit;
  p.status = status_word();

  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)K * 2};
    uint32_t box[2] = {BK, BM};
    int r = make_tmap_bf16(&ta, a, 2, dims, strides, box, 1);
    if (r) return r;
  }
  if (wfmt == WF_BF16) {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)n_experts};
    uint64_t strides[2] = {(uint64_t)K * 2, (uint64_t)K * 2 * (uint64_t)N};
    uint32_t box[3] = {BK, (uint32_t)bn, 1};
    int r = make_tmap_bf16(&tb, w0, 3, dims, strides, box, 1);
    if (r) return r;
  } else {
    tb = ta;
  }
  switch (bn) {
    case 128: return dispatch_fmt<128, 6>(wfmt, ta, tb, p, stream);
    case 64: return dispatch_fmt<64, 8>(wfmt, ta, tb, p, stream);
    case 32: return dispatch_fmt<32, 8>(wfmt, ta, tb, p, stream);
    default: return -105;
  }
}
