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
#include "comm.cuh"
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
  void* C;                      // leading dimension ldc (elements)
  int ldc;
  int out_f32;                  // output kind: 0 bf16, 1 fp32, 2 fp16
  const float* bias;            // [N] or [E][N], nullable
  const float* row_scale;       // [M], nullable
  int act;
  float act_alpha, act_limit;
  int group_m;                  // tile rasterisation group (see tile_coords)
  int* status;
  PeerOut peer;                 // world > 0: the tile is stored into every rank's inbox (fused all-reduce), not into C
  // all-gather -> GEMM: A is a gather buffer whose row chunks are stored by their owner ranks (shard.cu); the TMA producer waits for
  // the owner's flag before it loads the first tile of a chunk, and m-tiles are walked starting at this rank's own chunk
  const int* a_flags;           // [world] flags of the gather buffer (this rank's copy), null = plain A
  const int* a_seq;             // device word: the sequence number the flags have to reach
  int a_rows_per_src, a_world, m_rot;
};

constexpr int kRawDepth = 10;   // k-iterations of packed weight bytes kept in flight per producer thread

// Shared-memory plan.  TMA-fed weights: one ring of SA stages holding an A tile and a B tile each.
// Decoded weights: the A ring (SA deep, TMA) is decoupled from a short B ring (SB deep, written by
// the decode warps) because their latencies differ; in front of the B ring sits the packed-byte
// ring (kRawDepth deep) that hides HBM latency for the weights.
template <int FMT, int BN, int SA, int SB>
struct SmemLayout {
  static constexpr bool kDequant = FMT != WF_BF16;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int A_OFFSET = 0;
  static constexpr int B_OFFSET = SA * A_BYTES;
  static constexpr int NB = kDequant ? SB : SA;
  static constexpr int BAR_OFFSET = B_OFFSET + NB * B_BYTES;
  static constexpr int RAW_THREADS = 2 * BN;
  static constexpr int RAW_MAIN = kDequant ? RAW_THREADS * RawSlot<FMT>::MAIN : 0;     // per stage: main bytes, then aux bytes
  static constexpr int RAW_STAGE = kDequant ? RAW_THREADS * (RawSlot<FMT>::MAIN + RawSlot<FMT>::AUX) : 0;
  static constexpr int RAW_OFFSET = BAR_OFFSET + 512;
  // Epilogue staging for peer stores (TMA-fed weights only; the decode configuration has no room): per epilogue warp 32 rows of
  // 128 bytes (+16 bytes of padding against bank conflicts), so that a store instruction covers four whole 128-byte row segments.
  static constexpr int STG_ROW = 144;
  static constexpr int STG_BYTES = kDequant ? 0 : 4 * 32 * STG_ROW;
  static constexpr int STG_OFFSET = RAW_OFFSET + kRawDepth * RAW_STAGE;
  static constexpr int TOTAL = STG_OFFSET + STG_BYTES + 1024;   // + alignment slack
  static_assert(TOTAL <= 232448, "shared memory plan exceeds 227 KB");
};

// Tile order.  Tiles are walked in groups of `group_m` m-tiles: inside a group the m index runs
// fastest, then n.  group_m = 1 (grouped / MoE problems) keeps one m-tile's activations hot in L2
// while its n-tiles stream the expert's weights exactly once; dense problems use a group of 8 so a
// wave of CTAs shares both a band of A and a band of W.
__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group_m, int& mt, int& nt, int m_rot = 0) {
  const int per_group = group_m * n_tiles;
  const int g = t / per_group, r = t - g * per_group;
  const int gm = min(group_m, m_tiles - g * group_m);
  mt = g * group_m + r % gm;
  nt = r / gm;
  if (m_rot) { mt += m_rot; if (mt >= m_tiles) mt -= m_tiles; }
}

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

template <int FMT, int BN, int SA, int SB>
__global__ void __launch_bounds__(FMT == WF_BF16 ? 192 : 448, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using L = SmemLayout<FMT, BN, SA, SB>;
  constexpr bool kDequant = FMT != WF_BF16;
  // k-blocks per barrier handshake.  The single MMA-issuing thread pays a fixed cost per wait / commit pair, which at one
  // 64-wide k-block per handshake exceeded the tensor time of a 128x128 tile: TMA-fed (bf16) weights hand over two blocks
  // at once (measured 973 -> 1103 TFLOP/s at 8192^3).  Decoded weights are bound by the decode warps, not by the
  // handshake (no gain measured), and keep the finer ring.
  constexpr int KS = (!kDequant && SA % 2 == 0) ? 2 : 1;
  constexpr int LA = SA / KS, LB = (kDequant ? SB : SA) / KS;      // logical ring depths
  constexpr uint32_t TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);   // power of two for BN in {32,64,128,256}
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  // barrier slots: full_a[SA], empty_a[SA], full_b[SB], empty_b[SB], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * SA;
  const uint32_t bar_bfull = bar_empty + 8 * SA, bar_bempty = bar_bfull + 8 * SB;
  const uint32_t bar_tfull = bar_bempty + 8 * SB, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SA + 2 * SB + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * SA + 2 * SB + 4) * 8 + 8 <= 512, "barrier block too small");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(bar_bfull + 8 * s, kNumDequantWarps);      // one arrival per decode warp
      mbar_init(bar_bempty + 8 * s, 1);
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
  const int next_seq = p.peer.world ? *p.peer.seq + 1 : 0;
  const int k_iters = (p.K + BK - 1) / BK;
  const int kl_iters = (k_iters + KS - 1) / KS;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (A always, B when it is bf16)
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      if (!kDequant) prefetch_tmap(&tmap_b);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int mt, nt;
        tile_coords(t, m_tiles, p.num_n_tiles, p.group_m, mt, nt, p.m_rot);
        const int e = p.tile_expert ? p.tile_expert[mt] : 0;
        if (p.a_flags) {
          // the rows of this m-tile come from one owner rank: wait (bounded) until that rank's stores have been published
          const int src = min((mt * BM) / p.a_rows_per_src, p.a_world - 1);
          const int want = *p.a_seq;
          if (ld_acquire_sys(p.a_flags + src) - want < 0) {
            const long long t0 = clock64();
            while (ld_acquire_sys(p.a_flags + src) - want < 0) {
              __nanosleep(64);
              if (*abort_flag || clock64() - t0 > 2000000000ll) { *abort_flag = 1; atomicCAS(p.status, 0, ERR_PEER_FLAG_TIMEOUT); ok = false; break; }
            }
            if (!ok) break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");      // the peer's stores, acquired above, before this thread's TMA reads
        }
        for (int kl = 0; kl < kl_iters; ++kl, ++it) {
          const uint32_t s = it % LA, ph = (it / LA) & 1;
          if (!(ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
          mbar_expect_tx(bar_full + 8 * s, KS * (kDequant ? L::A_BYTES : L::A_BYTES + L::B_BYTES));
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            // a k-block past the end of K is fetched all the same: the out-of-range box arrives as zeros
            const int k = kl * KS + j;
            const uint32_t ps = s * KS + j;
            tma_load_2d(smem_base + L::A_OFFSET + ps * L::A_BYTES, &tmap_a, bar_full + 8 * s, k * BK, mt * BM);
            if (!kDequant) tma_load_3d(smem_base + L::B_OFFSET + ps * L::B_BYTES, &tmap_b, bar_full + 8 * s, k * BK, nt * BN, e);
          }
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
        for (int kl = 0; kl < kl_iters; ++kl, ++it) {
          const uint32_t s = it % LA, ph = (it / LA) & 1;
          const uint32_t sb = kDequant ? it % LB : s, phb = (it / LB) & 1;
          if (!(ok = mbar_wait(bar_full + 8 * s, ph, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          if (kDequant && !(ok = mbar_wait(bar_bfull + 8 * sb, phb, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          tc_fence_after();
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            const uint64_t a_desc = umma_desc_k_sw128(smem_base + L::A_OFFSET + (s * KS + j) * L::A_BYTES);
            const uint64_t b_desc = umma_desc_k_sw128(smem_base + L::B_OFFSET + (sb * KS + j) * L::B_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)   // 16 bf16 = 32 bytes per UMMA K step: +2 in the (addr>>4) field
              umma_bf16(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kl | j | kk) != 0);
          }
          umma_commit(bar_empty + 8 * s);
          if (kDequant) umma_commit(bar_bempty + 8 * sb);
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
      int mt, nt;
      tile_coords(t, m_tiles, p.num_n_tiles, p.group_m, mt, nt, p.m_rot);
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
        if constexpr (!kDequant && BN >= 64) {
          // Fused all-reduce, TMA-fed weights: a thread owns one row, so direct stores put 32 different rows (16 bytes each) into
          // one instruction, which NVLink carries as 32 small packets.  The rows go through shared memory instead and leave as
          // 128-byte segments, four rows per instruction.
          if (p.peer.world && p.act == ACT_NONE && (p.N & 7) == 0 && (p.ldc & 7) == 0) {
            const int eb = p.out_f32 == 1 ? 4 : 2;                 // bytes per element of the inbox slot
            const int cpf = 128 / eb;                              // columns per 128-byte segment: 32 (fp32) or 64 (bf16 / fp16)
            uint8_t* stg = smem + L::STG_OFFSET + q * (32 * L::STG_ROW);
            uint8_t* mine = stg + lane * L::STG_ROW + (c0 % cpf) * eb;
            const bool live = row_ok && col0 < p.N;
            if (eb == 4) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) {
                  o4.x = (__uint_as_float(r[j]) + (bias && col0 + j < p.N ? bias[col0 + j] : 0.f)) * rs;
                  o4.y = (__uint_as_float(r[j + 1]) + (bias && col0 + j + 1 < p.N ? bias[col0 + j + 1] : 0.f)) * rs;
                  o4.z = (__uint_as_float(r[j + 2]) + (bias && col0 + j + 2 < p.N ? bias[col0 + j + 2] : 0.f)) * rs;
                  o4.w = (__uint_as_float(r[j + 3]) + (bias && col0 + j + 3 < p.N ? bias[col0 + j + 3] : 0.f)) * rs;
                }
                *reinterpret_cast<float4*>(mine + j * 4) = o4;
              }
            } else {
              const bool h = p.out_f32 == 2;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = live ? (__uint_as_float(r[j + i]) + (bias && col0 + j + i < p.N ? bias[col0 + j + i] : 0.f)) * rs : 0.f;
                *reinterpret_cast<uint4*>(mine + j * 2) = h ? make_uint4(pack_f16(t[0], t[1]), pack_f16(t[2], t[3]), pack_f16(t[4], t[5]), pack_f16(t[6], t[7]))
                                                            : make_uint4(pack_bf16(t[0], t[1]), pack_bf16(t[2], t[3]), pack_bf16(t[4], t[5]), pack_bf16(t[6], t[7]));
              }
            }
            if ((c0 + 32) % cpf == 0 || c0 + 32 >= BN) {
              __syncwarp();
              const int seg_col0 = nt * BN + (c0 / cpf) * cpf;     // first column of the staged segment
              const int piece = lane & 7;                           // 16-byte piece of the 128-byte segment
              const int pcol = seg_col0 + piece * (16 / eb);
              const int n_dst = peer_count(p.peer);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int rl = 4 * j + (lane >> 3);
                const int grow = mt * BM + q * 32 + rl;
                if (grow < p.M && pcol < p.N) {
                  const uint4 val = *reinterpret_cast<const uint4*>(stg + rl * L::STG_ROW + piece * 16);
                  const int dst0 = peer_first(p.peer, grow);
                  for (int dst = dst0; dst < dst0 + n_dst; ++dst)
                    *reinterpret_cast<uint4*>(peer_slot(p.peer, dst, next_seq) + ((size_t)grow * p.ldc + pcol) * eb) = val;
                }
              }
              __syncwarp();
            }
            continue;
          }
        }
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
          const int n_dst = p.peer.world ? peer_count(p.peer) : 1;
          const int dst0 = p.peer.world ? peer_first(p.peer, row) : 0;
          for (int dst = dst0; dst < dst0 + n_dst; ++dst) {
          void* cbase = p.peer.world ? (void*)peer_slot(p.peer, dst, next_seq) : p.C;
          if (p.out_f32 == 1) {
            float* out = (float*)cbase + (size_t)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) out[j] = v[j];
            }
          } else {
            const bool h = p.out_f32 == 2;
            __nv_bfloat16* out = (__nv_bfloat16*)cbase + (size_t)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                *reinterpret_cast<uint4*>(out + j) = h ? make_uint4(pack_f16(v[j], v[j + 1]), pack_f16(v[j + 2], v[j + 3]),
                                                                    pack_f16(v[j + 4], v[j + 5]), pack_f16(v[j + 6], v[j + 7]))
                                                       : make_uint4(pack_bf16(v[j], v[j + 1]), pack_bf16(v[j + 2], v[j + 3]),
                                                                    pack_bf16(v[j + 4], v[j + 5]), pack_bf16(v[j + 6], v[j + 7]));
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                if (h) ((__half*)out)[j] = __float2half(v[j]); else out[j] = __float2bfloat16(v[j]);
              }
            }
          }
          }
        } else {
          // gate/up are interleaved in groups of 16 columns: [g0..g15 | u0..u15]; 16 outputs per 32 inputs
          const int ocol0 = col0 >> 1;
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = act_apply(p.act, v[j], v[16 + j], p.act_alpha, p.act_limit) * rs;
          const int on = p.N >> 1;
          if (p.out_f32 == 1) {
            float* out = (float*)p.C + (size_t)row * p.ldc + ocol0;
            for (int j = 0; j < 16 && ocol0 + j < on; ++j) out[j] = o[j];
          } else {
            const bool h = p.out_f32 == 2;
            __nv_bfloat16* out = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + ocol0;
            if (ocol0 + 16 <= on && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 16; j += 8)
                *reinterpret_cast<uint4*>(out + j) = h ? make_uint4(pack_f16(o[j], o[j + 1]), pack_f16(o[j + 2], o[j + 3]),
                                                                    pack_f16(o[j + 4], o[j + 5]), pack_f16(o[j + 6], o[j + 7]))
                                                       : make_uint4(pack_bf16(o[j], o[j + 1]), pack_bf16(o[j + 2], o[j + 3]),
                                                                    pack_bf16(o[j + 4], o[j + 5]), pack_bf16(o[j + 6], o[j + 7]));
            } else {
              for (int j = 0; j < 16 && ocol0 + j < on; ++j) {
                if (h) ((__half*)out)[j] = __float2half(o[j]); else out[j] = __float2bfloat16(o[j]);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
  } else if (kDequant) {
    // ------------------------------------------------ weight decode producers (8 warps)
    // Thread d owns (row d>>1, k-half d&1) of every B tile.  Its packed bytes travel global ->
    // private shared slot with cp.async, kRawDepth k-iterations ahead (across tile boundaries), so
    // HBM latency is covered by the copies in flight instead of stalling the decode.
    const int d = threadIdx.x - (2 + kNumEpilogueWarps) * 32;   // 0..255
    const int half = d & 1, rl = d >> 1;
    const bool live = rl < BN;
    uint8_t* raw_base = smem + L::RAW_OFFSET + (live ? d : 0) * RawSlot<FMT>::MAIN;
    uint8_t* aux_base = smem + L::RAW_OFFSET + L::RAW_MAIN + (live ? d : 0) * RawSlot<FMT>::AUX;
    const uint32_t raw_base_u32 = smem_u32(raw_base), aux_base_u32 = smem_u32(aux_base);
    const int k_blocks = p.K / 32;                 // valid 32-element blocks along K
    // prefetch cursor: tile pt, k-iteration pk, ring slot ps; row pointers are recomputed once per tile
    int pt = blockIdx.x, pk = 0, ps = 0;
    RowPtrs prp = {nullptr, nullptr, nullptr, nullptr};
    bool prow_ok = false;
    auto prefetch_tile_setup = [&]() {
      prow_ok = false;
      if (pt < total_tiles && live) {
        int pmt, pnt;
        tile_coords(pt, m_tiles, p.num_n_tiles, p.group_m, pmt, pnt, p.m_rot);
        const int n = pnt * BN + rl;
        if (n < p.N) {
          const int pe = p.tile_expert ? p.tile_expert[pmt] : 0;
          prp = row_ptrs<FMT>(p.tile_expert ? expert_weight<FMT>(p.w, pe, p.N, p.K) : p.w, n, p.K);
          prow_ok = true;
        }
      }
    };
    auto issue_next = [&]() {
      if (prow_ok && 2 * pk + half < k_blocks) raw_issue<FMT>(raw_base_u32 + ps * L::RAW_STAGE, aux_base_u32 + ps * L::RAW_STAGE, prp, pk, half);
      cp_async_commit();
      ps = (ps + 1 == kRawDepth) ? 0 : ps + 1;
      if (++pk == k_iters) { pk = 0; pt += gridDim.x; prefetch_tile_setup(); }
    };
    prefetch_tile_setup();
#pragma unroll 1
    for (int i = 0; i < kRawDepth - 1; ++i) issue_next();
    uint32_t sb = 0, phb = 0;
    int cs = 0;                                    // consume slot in the raw ring
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int mt, nt;
      tile_coords(t, m_tiles, p.num_n_tiles, p.group_m, mt, nt, p.m_rot);
      const bool row_ok = live && nt * BN + rl < p.N;
      for (int kl = 0; kl < kl_iters && ok; ++kl) {
        if (!(ok = mbar_wait(bar_bempty + 8 * sb, phb ^ 1, p.status, ERR_MBAR_TIMEOUT_DEQUANT, abort_flag))) break;
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          const int k = kl * KS + j;
          uint32_t o[16];
          bool have = false;
          if (k < k_iters) {
            issue_next();
            cp_async_wait<kRawDepth - 1>();          // this iteration's bytes have landed in the slot
            if (live && row_ok && 2 * k + half < k_blocks) {
              raw_decode<FMT>(raw_base + cs * L::RAW_STAGE, aux_base + cs * L::RAW_STAGE, k, half, o);
              have = true;
            }
            cs = (cs + 1 == kRawDepth) ? 0 : cs + 1;
          }
          if (live) {
            if (!have) {
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = 0u;
            }
            uint8_t* b_tile = smem + L::B_OFFSET + (sb * KS + j) * L::B_BYTES;
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(b_tile + sw128_offset(rl, raw_chunk<FMT>(half, c))) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
          }
        }
        // every lane publishes its generic-proxy stores to the async proxy, then one lane arrives for the warp
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_bfull + 8 * sb);
        if (++sb == LB) { sb = 0; phb ^= 1; }
      }
    }
    cp_async_wait<0>();
  }

  // ---------------------------------------------------- teardown
  if (*abort_flag) {
    // a wait ran out: give copies still in flight time to land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (p.peer.world) peer_publish(p.peer, next_seq);
}

// ------------------------------------------------------------------------------------------
template <int FMT, int BN, int SA, int SB>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  using L = SmemLayout<FMT, BN, SA, SB>;
  auto kern = gemm_kernel<FMT, BN, SA, SB>;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured.mark();
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, FMT == WF_BF16 ? 192 : 448, L::TOTAL, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// SA: depth of the TMA ring (A, plus B when the weights are bf16).  QA/QB: depths of the A ring and
// of the decoded-B ring for quantised weights.
template <int BN, int SA, int QA, int QB>
static int dispatch_fmt(int fmt, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
  switch (fmt) {
    case WF_BF16: return launch<WF_BF16, BN, SA, 1>(ta, tb, p, st);
    case WF_Q8: return launch<WF_Q8, BN, QA - 1, QB - 2>(ta, tb, p, st);
    case WF_Q4K: return launch<WF_Q4K, BN, QA, QB - 1>(ta, tb, p, st);
    case WF_Q6K: return launch<WF_Q6K, BN, QA, QB - 1>(ta, tb, p, st);
    case WF_MXFP4: return launch<WF_MXFP4, BN, QA, QB>(ta, tb, p, st);
    default: return -100;
  }
}

}  // namespace mx

// C[M, N(/2 with act)] = A[M,K] * W[(E,)N,K]^T.
//   a          bf16 [M,K] row-major, 16-byte aligned, K % 8 == 0
//   out_f32    output kind: 0 bf16, 1 fp32, 2 fp16
//   wfmt/w0..w3  weight format and plane pointers (see WFormat); n_experts >= 1
//   tile_expert / num_m_tiles_dev: grouped mode (both null for a plain GEMM)
//   bn         32, 64 or 128 (tile width); the caller picks small tiles for small M
// Returns 0 or a CUDA / driver error code.
struct GatherIn { const int* flags; const int* seq; int rows_per_src, world, m_rot; };
static int gemm_impl(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, int n_experts,
                     void* c, int ldc, int out_f32, const float* bias, const float* row_scale, int act, float act_alpha,
                     float act_limit, int M, int N, int K, const int* tile_expert, const int* num_m_tiles_dev, int bn,
                     const mx::PeerOut* peer, cudaStream_t stream, const GatherIn* gin = nullptr);

MX_HOST_API int mx_gemm(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, int n_experts,
                        void* c, int ldc, int out_f32, const float* bias, const float* row_scale, int act, float act_alpha,
                        float act_limit, int M, int N, int K, const int* tile_expert, const int* num_m_tiles_dev, int bn,
                        cudaStream_t stream) {
  return gemm_impl(a, wfmt, w0, w1, w2, w3, n_experts, c, ldc, out_f32, bias, row_scale, act, act_alpha, act_limit, M, N, K, tile_expert,
                   num_m_tiles_dev, bn, nullptr, stream);
}

// all-gather -> GEMM: `a` is this rank's gather buffer [M,K]; rows [s * rows_per_src, (s + 1) * rows_per_src) are valid once
// flags[s] >= *seq.  m-tiles are taken starting at tile m_rot (this rank's own rows), so the math starts before the peers' rows
// have arrived.  Optional reduce-scatter epilogue as in mx_gemm_allreduce when world > 0.
MX_HOST_API int mx_gemm_gathered(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, void* c, int ldc,
                                 int out_f32, const float* bias, int act, float act_alpha, float act_limit, int M, int N, int K, int bn,
                                 const int* flags, const int* seq, int rows_per_src, int src_world, int m_rot, cudaStream_t stream) {
  GatherIn g{flags, seq, rows_per_src, src_world, m_rot};
  return gemm_impl(a, wfmt, w0, w1, w2, w3, 1, c, ldc, out_f32, bias, nullptr, act, act_alpha, act_limit, M, N, K, nullptr, nullptr, bn, nullptr,
                   stream, &g);
}

namespace mx { PeerOut make_peer_out(const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket); }

// Row-parallel GEMM fused with the all-reduce: every tcgen05 output tile is stored (bf16 when out_kind == 0,
// fp32 when 1) into slot [my_rank] of every rank's inbox straight from the epilogue registers; the last CTA
// publishes the sequence number.  The consumer is mx_comm_rmsnorm_reduce / mx_comm_reduce.
MX_HOST_API int mx_gemm_allreduce(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, const float* bias,
                                  int out_kind, int M, int N, int K, int bn, const void* const* inbox, int world, int my_rank,
                                  long long slot_bytes, int* seq, int* ticket, int rs_rows, cudaStream_t stream) {
  if ((long long)M * N * (out_kind == 1 ? 4 : 2) > slot_bytes) return -140;
  mx::PeerOut po = mx::make_peer_out(inbox, world, my_rank, slot_bytes, seq, ticket);
  po.rs_rows = rs_rows;
  return gemm_impl(a, wfmt, w0, w1, w2, w3, 1, nullptr, N, out_kind, bias, nullptr, 0, 0.f, 0.f, M, N, K, nullptr, nullptr, bn, &po, stream);
}

static int gemm_impl(const void* a, int wfmt, const void* w0, const void* w1, const void* w2, const void* w3, int n_experts,
                     void* c, int ldc, int out_f32, const float* bias, const float* row_scale, int act, float act_alpha,
                     float act_limit, int M, int N, int K, const int* tile_expert, const int* num_m_tiles_dev, int bn,
                     const mx::PeerOut* peer, cudaStream_t stream, const GatherIn* gin) {
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
  if (peer) p.peer = *peer; else p.peer.world = 0;
  p.group_m = tile_expert ? 1 : 8;
  p.status = status_word();
  p.a_flags = nullptr; p.a_seq = nullptr; p.a_rows_per_src = 0; p.a_world = 0; p.m_rot = 0;
  if (gin) {
    if (gin->rows_per_src % BM) return -106;            // a 128-row tile must not straddle two owners
    p.a_flags = gin->flags; p.a_seq = gin->seq; p.a_rows_per_src = gin->rows_per_src; p.a_world = gin->world;
    p.m_rot = gin->m_rot % p.num_m_tiles;
    p.group_m = 1;                                      // m-major walk: all n-tiles of a row chunk before the next chunk is needed
  }

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
    case 128: return dispatch_fmt<128, 6, 4, 6>(wfmt, ta, tb, p, stream);
    case 64: return dispatch_fmt<64, 8, 6, 4>(wfmt, ta, tb, p, stream);
    case 32: return dispatch_fmt<32, 8, 6, 4>(wfmt, ta, tb, p, stream);
    default: return -105;
  }
}
