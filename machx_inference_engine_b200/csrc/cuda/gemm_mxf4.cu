// Block-scaled MXFP4 grouped GEMM for sm_100a: the expert projections of gpt-oss on the 5th-generation
// tensor cores with nothing decoded on the ALUs.
//
//   * Weights stay packed E2M1 (4 bit) + e8m0 scale per 32 in global memory, repacked once at load time
//     into tiles of 192 rows x 128 elements (ops/weights.py: to_mxf4_tiles).  TMA (16U4_ALIGN16B tensor
//     map) expands a tile into the padded 8-bit containers that `tcgen05.mma.kind::mxf8f6f4.block_scale`
//     reads; the scale factors travel as 512-byte atoms (bulk copy -> shared memory -> `tcgen05.cp` -> TMEM).
//   * Activations are MXFP8 (e4m3 + e8m0 per 32): moe_quant_kernel produces them from the bf16 hidden rows
//     while they are gathered into expert order, and the gated first projection writes its output in that
//     form itself, so the second projection reads it without a pass in between.
//   * One instruction multiplies a 128-row token tile (M) with 192 weight rows (N) over 32 elements of K.
//     A tcgen05.mma of M = 128 occupies the tensor pipe for about 130 cycles however narrow N is (measured
//     here: 16- to 96-column instructions all took as long), so the weights sit on the wide N side: 192
//     rows per instruction keep the pipe's appetite (3 KiB of packed weights per instruction) above the
//     SM's share of HBM bandwidth.  192 = 96 gate rows + 96 up rows of the same features for the gated
//     pair (the activation then pairs column c with column c + 96 of one TMEM lane), or 192 consecutive
//     rows of the down projection; twice 192 accumulator columns leave room in TMEM for the scale factors.
//   * Token tiles are the packer's 128-row expert segments (prefill), or one (token, expert) pair per tile
//     (decode): rows beyond a tile's live count are never loaded or stored.
//   * Roles: one thread issues TMA / bulk copies for a ring of stages, one thread issues tcgen05.cp /
//     tcgen05.mma, four warps drain double-buffered accumulators.
//
// Reference parity: replaces the per-expert dequant + oneDNN GEMM chain of src/model/gptoss_tp.cpp:685-765
// and the MXFP4 GEMV family of src/ops/gemv_mxfp4.cpp:94-323 for the expert projections.
#include "common.cuh"
#include "host_util.h"
#include "moe_route.cuh"
#include "mxfp8.cuh"

#include <cuda_fp8.h>

namespace mx {

constexpr int XT_M = 128;        // token rows per tile (instruction M)
constexpr int XT_K = 128;        // elements of K per stage (4 instructions of K = 32)
constexpr int XT_N = 192;        // weight rows per tile (instruction N)
constexpr int XT_HALF = XT_N / 2;
constexpr int XT_FEW = 8;        // tiles with at most this many live rows take the epilogue that spreads one row over a warp

struct Mxf4Params {
  int N, K;                       // output features (dual: of gate and of up each), logical K
  int FB, KB;                     // feature blocks (96 features dual, 192 single), 128-element k blocks
  int KS, KBS;                    // single mode: K is cut into KS ranges of KBS k-blocks, range s writes its partial sums to rows
  long long split_rows;           // s * split_rows + row of `out` (the consumer adds them up); KS = 1: no split
  int dual;
  int max_tiles;                  // host bound on token tiles; scale atoms of the activations are [KB][max_tiles][512]
  int row_stride;                 // first row of token tile j is j * row_stride (128: padded expert segments, 1: one pair per tile)
  int e_lo, n_experts;            // tile_expert holds global expert ids; the bank holds experts [e_lo, e_lo + n_experts), other tiles are skipped
  const int* num_tiles_dev;       // live tile count (device), nullable
  const int* tile_expert;         // [max_tiles]
  const int* tile_valid;          // [max_tiles] live rows of each tile (1..128), nullable = default_valid
  int default_valid;
  const uint8_t* sfw;             // weight scale atoms [E][FB][KB][2][512]
  const uint8_t* sfx;             // activation scale atoms [KB][max_tiles][512]
  const float* bias0;             // [E][N] nullable (dual: gate)
  const float* bias1;             // dual: up
  __nv_bfloat16* out;             // single: [rows][ldo] bf16
  int ldo;
  uint8_t* oq;                    // dual: [rows][oq_ld] e4m3, the next projection's input
  uint8_t* osf;                   // dual: its scale atoms [oq_ld / 128][max_tiles][512]
  int oq_ld;
  int act;                        // dual: 1 SwiGLU, 2 clamped SwiGLU
  float act_alpha, act_limit;
  int* status;
};

struct XLayout {
  static constexpr int A_BYTES = XT_M * XT_K;                 // 16 KiB: 128 token rows x 128 e4m3
  static constexpr int B_BYTES = XT_N * XT_K;                 // 24 KiB: 192 weight rows x 128 one-byte containers
  static constexpr int A = 0;
  static constexpr int B = A_BYTES;
  static constexpr int SF = B + B_BYTES;                      // SFX (512), SFW (1024), pad
  static constexpr int STAGE = SF + 2048;
  static constexpr int STAGES = 5;
  static constexpr int BAR_OFFSET = STAGES * STAGE;
  static constexpr int EPI_OFFSET = BAR_OFFSET + 256;         // few-row epilogue: XT_FEW accumulator rows as fp32
  static constexpr int EPI_BYTES = XT_FEW * XT_N * 4;
  static constexpr int TOTAL = EPI_OFFSET + EPI_BYTES + 1024; // + alignment slack
  static_assert(STAGE % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(TOTAL <= 232448, "shared memory plan exceeds 227 KB");
};

// kind::mxf8f6f4 instruction descriptor: A = E4M3 (code 0) tokens, B = E2M1 (code 5) weights, ue8m0 scales, K-major operands,
// M = 128, N = 192.  The scale-factor ids (which byte of a scale column the instruction uses) are added per k-step.
constexpr uint32_t MXF4_IDESC = (0u << 7) | (5u << 10) | ((uint32_t)(XT_N >> 3) << 17) | (1u << 23) | ((uint32_t)(XT_M >> 4) << 24);
constexpr uint32_t MXF4_IDESC_KSTEP = (1u << 4) | (1u << 29);

// The loops of the two single-thread roles are written for instruction count: one thread issues every copy or every MMA of an SM.
template <bool ACC>
__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t tsfa, uint32_t tsfb, uint32_t acc = 1) {
  // K-major, 128-byte swizzle: the upper descriptor word is constant (stride 1024 B between 8-row groups, version 1, SWIZZLE_128B)
  constexpr uint32_t HI = (1024u >> 4) | (1u << 14) | (2u << 29);
  const uint64_t a = ((uint64_t)HI << 32) | a_lo, b = ((uint64_t)HI << 32) | b_lo;
  if constexpr (ACC) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(tsfa), "r"(tsfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(tsfa), "r"(tsfb)
        : "memory");
  }
}
// start-address word of a K-major SWIZZLE_128B operand descriptor
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16); }
// 32 rows x 16 bytes of shared memory -> 32 TMEM lanes x 4 columns, replicated into the four lane quarters
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint32_t smem_addr) {
  constexpr uint32_t HI = (128u >> 4) | (1u << 14);       // 128 bytes between 8-row groups, version 1, no swizzle
  const uint64_t d = ((uint64_t)HI << 32) | ((smem_addr & 0x3FFFF) >> 4);
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(d) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// barrier of the four epilogue warps
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

__device__ __forceinline__ float mxf4_act(int act, float g, float u, float alpha, float limit) {
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return __fdividef(g, 1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  return __fdividef(g, 1.f + __expf(-g)) * u;
}

// work item t -> (token tile j, feature block fb, k range ks); returns the tile's live rows (<= 0: nothing to do)
__device__ __forceinline__ int item_decode(const Mxf4Params& p, int t, int& j, int& fb, int& ks) {
  ks = 0;
  if (p.KS > 1) { ks = t % p.KS; t /= p.KS; }
  j = t / p.FB;
  fb = t - j * p.FB;
  const int e = p.tile_expert[j] - p.e_lo;
  if (e < 0 || e >= p.n_experts) return 0;
  return p.tile_valid ? p.tile_valid[j] : p.default_valid;
}

__global__ void __launch_bounds__(192, 1)
mxf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x16, const __grid_constant__ CUtensorMap tmap_x32,
                 const __grid_constant__ CUtensorMap tmap_x64, const __grid_constant__ CUtensorMap tmap_x128, const Mxf4Params p) {
  using L = XLayout;
  constexpr int S = L::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t SF_COL = 2 * XT_N;       // scale factors: four buffers of 16 columns behind the two accumulators
  static_assert(SF_COL + 64 <= TMEM_COLS, "TMEM plan");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * S;
  const uint32_t bar_tfull = bar_empty + 8 * S, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * S + 4) * 8 + 8 <= 256, "barrier block too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 128); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_prologue();           // everything below reads what earlier kernels of the stream wrote

  const int m_tiles = p.num_tiles_dev ? min(*p.num_tiles_dev, p.max_tiles) : p.max_tiles;
  const int total = m_tiles * p.FB * p.KS;

  if (warp == 0) {
    // ------------------------------------------------ producer: TMA tiles + bulk copies of the scale atoms
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      prefetch_tmap(&tmap_x128);
      uint32_t s = 0, ph = 1, st = smem_base, fbar = bar_full, ebar = bar_empty;     // ring cursor (ph: parity to wait for on `empty`)
      const size_t sfx_step = (size_t)p.max_tiles * SF_ATOM;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int j, fb, ks;
        const int nv = item_decode(p, t, j, fb, ks);
        if (nv <= 0) continue;
        const int kb0 = ks * p.KBS, kb1 = min(p.KB, kb0 + p.KBS);
        const int box = nv <= 16 ? 16 : (nv <= 32 ? 32 : (nv <= 64 ? 64 : 128));
        const CUtensorMap* tx = box == 16 ? &tmap_x16 : (box == 32 ? &tmap_x32 : (box == 64 ? &tmap_x64 : &tmap_x128));
        const long long wt = ((long long)(p.tile_expert[j] - p.e_lo) * p.FB + fb) * p.KB;   // first weight tile of this slab
        const int row0 = j * p.row_stride;
        // a packed-4-bit TMA load counts its packed bytes on the barrier (half of what it writes to shared memory)
        const uint32_t bytes = L::B_BYTES / 2 + 2 * SF_ATOM + box * XT_K + SF_ATOM;
        int wy = (int)((wt + kb0) * XT_N), kx = kb0 * XT_K;
        const uint8_t* sw = p.sfw + (wt + kb0) * (2 * SF_ATOM);
        const uint8_t* sx = p.sfx + (size_t)j * SF_ATOM + (size_t)kb0 * sfx_step;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(ebar, ph, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
          mbar_expect_tx(fbar, bytes);
          tma_load_2d(st + L::B, &tmap_w, fbar, 0, wy);
          tma_load_2d(st + L::A, tx, fbar, kx, row0);
          bulk_load(st + L::SF + SF_ATOM, sw, 2 * SF_ATOM, fbar);
          bulk_load(st + L::SF, sx, SF_ATOM, fbar);
          wy += XT_N; kx += XT_K; sw += 2 * SF_ATOM; sx += sfx_step;
          st += L::STAGE; fbar += 8; ebar += 8;
          if (++s == S) { s = 0; ph ^= 1; st = smem_base; fbar = bar_full; ebar = bar_empty; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t s = 0, ph = 0, st = smem_base, fbar = bar_full, ebar = bar_empty, sfsel = 0, item_n = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int j, fb, ks;
        if (item_decode(p, t, j, fb, ks) <= 0) continue;
        const int kb0 = ks * p.KBS, kb1 = min(p.KB, kb0 + p.KBS);
        const uint32_t acc = item_n & 1, acc_ph = (item_n >> 1) & 1;
        ++item_n;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * XT_N;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(fbar, ph, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          tc_fence_after();
          const uint32_t sf = tmem_base + SF_COL + sfsel;               // four scale buffers rotate between consecutive stages
          sfsel = (sfsel + 16) & 63;
          tmem_cp_sf(sf, st + L::SF);                                   // token scales: columns 0..3
          tmem_cp_sf(sf + 4, st + L::SF + SF_ATOM);                     // weight scales: rows 0..127 -> columns 4..7
          tmem_cp_sf(sf + 8, st + L::SF + 2 * SF_ATOM);                 //                rows 128..191 -> columns 8, 9
          const uint32_t a = desc_lo(st + L::A), b = desc_lo(st + L::B);
          umma_mxf4<false>(d, a, b, MXF4_IDESC, sf, sf + 4, (uint32_t)(kb - kb0));
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)        // 32 elements = 32 bytes per k-step: +2 in the descriptor's 16-byte units
            umma_mxf4<true>(d, a + 2 * kk, b + 2 * kk, MXF4_IDESC + kk * MXF4_IDESC_KSTEP, sf, sf + 4);
          umma_commit(ebar);
          st += L::STAGE; fbar += 8; ebar += 8;
          if (++s == S) { s = 0; ph ^= 1; st = smem_base; fbar = bar_full; ebar = bar_empty; }
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);
      }
    }
  } else {
    // ------------------------------------------------ epilogue: lane = token row, column = weight row (feature)
    const int q = warp & 3;
    const int rin = q * 32 + lane;                // row inside the token tile
    uint32_t item_n = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int j, fb, ks;
      const int nv = item_decode(p, t, j, fb, ks);
      if (nv <= 0) continue;
      const uint32_t acc = item_n & 1, acc_ph = (item_n >> 1) & 1;
      ++item_n;
      if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, p.status, ERR_MBAR_TIMEOUT_EPILOGUE, abort_flag, 64))) break;
      tc_fence_after();
      const int e = p.tile_expert[j] - p.e_lo;
      const bool row_ok = rin < nv;
      const size_t row = (size_t)j * p.row_stride + rin;
      const uint32_t tl = tmem_base + ((uint32_t)(q * 32) << 16) + acc * XT_N;
      if (nv <= XT_FEW) {
        // Few live rows (decode: one pair per tile; batched decode: a couple of rows per expert).  With lane = row only a few
        // threads of one warp would do the whole epilogue, so the rows go through shared memory and every warp takes
        // (row, 32- or 64-column block) items with lane = column.
        float* epi = reinterpret_cast<float*>(smem + L::EPI_OFFSET);
        if (q == 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < XT_N; c0 += 32) {
            uint32_t g[32];
            tmem_ld_32x32(tl + c0, g);
            tmem_ld_wait();
            if (lane < nv) {
              float4* d4 = reinterpret_cast<float4*>(epi + lane * XT_N + c0);
#pragma unroll
              for (int c = 0; c < 8; ++c)
                d4[c] = make_float4(__uint_as_float(g[4 * c]), __uint_as_float(g[4 * c + 1]), __uint_as_float(g[4 * c + 2]), __uint_as_float(g[4 * c + 3]));
            }
          }
        }
        epi_sync();
        tc_fence_before();
        mbar_arrive(bar_tempty + 8 * acc);         // the accumulator is free while the rows are finished from shared memory
        const int we = warp - 2;
        if (p.dual) {
          const float* bg = p.bias0 ? p.bias0 + (size_t)e * p.N : nullptr;
          const float* bu = p.bias1 ? p.bias1 + (size_t)e * p.N : nullptr;
          for (int it = we; it < nv * 3; it += 4) {
            const int r = it / 3, b = it - r * 3;
            const int f0 = fb * XT_HALF + b * 32;
            if (f0 >= p.N) continue;
            const size_t orow = (size_t)j * p.row_stride + r;
            const float gv = epi[r * XT_N + b * 32 + lane] + (bg ? __ldg(bg + f0 + lane) : 0.f);
            const float uv = epi[r * XT_N + XT_HALF + b * 32 + lane] + (bu ? __ldg(bu + f0 + lane) : 0.f);
            const float v = __bfloat162float(__float2bfloat16(mxf4_act(p.act, gv, uv, p.act_alpha, p.act_limit)));
            float inv;
            const uint32_t eb = mxfp8_scale(warp_max(fabsf(v)), &inv);
            p.oq[orow * p.oq_ld + f0 + lane] = (uint8_t)__nv_cvt_float_to_fp8(v * inv, __NV_SATFINITE, __NV_E4M3);
            const int blk = f0 >> 5;
            if (lane == 0) p.osf[((size_t)(blk >> 2) * p.max_tiles + j) * SF_ATOM + sf_atom_offset(r, blk & 3)] = (uint8_t)eb;
          }
          if (fb == p.FB - 1) {
            for (int it = we; it < nv; it += 4) {
              const size_t orow = (size_t)j * p.row_stride + it;
              for (int f0 = p.N; f0 < p.oq_ld; f0 += 32) {
                p.oq[orow * p.oq_ld + f0 + lane] = 0;
                const int blk = f0 >> 5;
                if (lane == 0) p.osf[((size_t)(blk >> 2) * p.max_tiles + j) * SF_ATOM + sf_atom_offset(it, blk & 3)] = 127;
              }
            }
          }
        } else {
          const float* bs = (p.bias0 && ks == 0) ? p.bias0 + (size_t)e * p.N : nullptr;
          for (int it = we; it < nv * 3; it += 4) {
            const int r = it / 3, b = it - r * 3;
            const int f = fb * XT_N + b * 64 + 2 * lane;
            if (f >= p.N) continue;
            __nv_bfloat16* orow = p.out + ((size_t)ks * p.split_rows + (size_t)j * p.row_stride + r) * p.ldo;
            const float v0 = epi[r * XT_N + b * 64 + 2 * lane] + (bs ? __ldg(bs + f) : 0.f);
            if (f + 1 < p.N) {
              const float v1 = epi[r * XT_N + b * 64 + 2 * lane + 1] + (bs ? __ldg(bs + f + 1) : 0.f);
              if ((p.ldo & 1) == 0) *reinterpret_cast<uint32_t*>(orow + f) = pack_bf16(v0, v1);
              else { orow[f] = __float2bfloat16(v0); orow[f + 1] = __float2bfloat16(v1); }
            } else {
              orow[f] = __float2bfloat16(v0);
            }
          }
        }
        epi_sync();                                // the next item's rows overwrite the staging buffer
        continue;
      }
      if (q * 32 < nv) {                           // warps whose 32 rows are all beyond the tile's live rows have nothing to read
        if (p.dual) {
          const float* bg = p.bias0 ? p.bias0 + (size_t)e * p.N : nullptr;
          const float* bu = p.bias1 ? p.bias1 + (size_t)e * p.N : nullptr;
#pragma unroll 1
          for (int c0 = 0; c0 < XT_HALF; c0 += 32) {
            uint32_t g[32], u[32];
            tmem_ld_32x32(tl + c0, g);
            tmem_ld_32x32(tl + XT_HALF + c0, u);
            tmem_ld_wait();
            const int f0 = fb * XT_HALF + c0;     // first output feature of this 32-column block (a multiple of 32)
            if (f0 >= p.N) break;
            if (!row_ok) continue;                // rows beyond the tile's live count hold whatever the last tile left in shared memory
            float v[32];
            float amax = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              // N is a multiple of 32: the whole block is inside the matrix
              const float gv = __uint_as_float(g[c]) + (bg ? __ldg(bg + f0 + c) : 0.f);
              const float uv = __uint_as_float(u[c]) + (bu ? __ldg(bu + f0 + c) : 0.f);
              v[c] = __bfloat162float(__float2bfloat16(mxf4_act(p.act, gv, uv, p.act_alpha, p.act_limit)));
              amax = fmaxf(amax, fabsf(v[c]));
            }
            {
              float inv;
              const uint32_t eb = mxfp8_scale(amax, &inv);
              uint4* dst = reinterpret_cast<uint4*>(p.oq + row * p.oq_ld + f0);
              dst[0] = make_uint4(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv), e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                                  e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv), e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
              dst[1] = make_uint4(e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv), e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv),
                                  e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv), e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv));
              const int blk = f0 >> 5;
              p.osf[((size_t)(blk >> 2) * p.max_tiles + j) * SF_ATOM + sf_atom_offset(rin, blk & 3)] = (uint8_t)eb;
            }
          }
          // the feature block that ends the row also writes the zero padding up to the next multiple of 128 (unit scale)
          if (row_ok && fb == p.FB - 1) {
            for (int f0 = p.N; f0 < p.oq_ld; f0 += 32) {
              uint4* dst = reinterpret_cast<uint4*>(p.oq + row * p.oq_ld + f0);
              dst[0] = make_uint4(0, 0, 0, 0);
              dst[1] = make_uint4(0, 0, 0, 0);
              const int blk = f0 >> 5;
              p.osf[((size_t)(blk >> 2) * p.max_tiles + j) * SF_ATOM + sf_atom_offset(rin, blk & 3)] = 127;
            }
          }
        } else {
          const float* bs = (p.bias0 && ks == 0) ? p.bias0 + (size_t)e * p.N : nullptr;
          __nv_bfloat16* out = p.out + ((size_t)ks * p.split_rows + row) * p.ldo;
#pragma unroll 1
          for (int c0 = 0; c0 < XT_N; c0 += 32) {
            uint32_t g[32];
            tmem_ld_32x32(tl + c0, g);
            tmem_ld_wait();
            const int f0 = fb * XT_N + c0;
            if (f0 >= p.N) break;
            if (!row_ok) continue;
            if (f0 + 32 <= p.N && (p.ldo & 7) == 0) {
#pragma unroll
              for (int c = 0; c < 32; c += 8) {
                float w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = __uint_as_float(g[c + i]) + (bs ? __ldg(bs + f0 + c + i) : 0.f);
                *reinterpret_cast<uint4*>(out + f0 + c) = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
              }
            } else {
#pragma unroll
              for (int c = 0; c < 32; ++c)
                if (f0 + c < p.N) out[f0 + c] = __float2bfloat16(__uint_as_float(g[c]) + (bs ? bs[f0 + c] : 0.f));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);      // a wait ran out: let copies in flight land before shared memory is released
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------ activation quantiser
// One CTA per destination row r: source row = src_index ? src_index[r] : r, divided by x_div (pair mode: K pairs share a token
// row); rows whose index is negative (tile padding) are skipped.  Thread i owns the 32-element block i of the row: amax -> e8m0
// scale -> 32 e4m3 bytes; the scale byte lands in the row's slot of the tile's scale atom.  Blocks between K and the padded
// KB * 128 are written as zeros with a unit scale.
__global__ void __launch_bounds__(128) moe_quant_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ src_index, int x_div,
                                                        const int* __restrict__ row_limit, int K, int KB, int max_tiles, int rows_per_tile,
                                                        uint8_t* __restrict__ xq, uint8_t* __restrict__ sfx) {
  pdl_prologue();
  const int r = blockIdx.x;
  if (row_limit && r >= row_limit[1]) return;
  int src = r;
  if (src_index) { src = src_index[r]; if (src < 0) return; }
  src /= x_div;
  const int Kp = KB * XT_K;
  const int tile = r / rows_per_tile, rin = r - tile * rows_per_tile;
  for (int blk = threadIdx.x; blk < KB * 4; blk += blockDim.x) {
    const int k0 = blk * 32;
    float v[32];
    float amax = 0.f;
    const bool live = k0 < K;           // K is a multiple of 32
    if (live) {
      const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)src * ldx + k0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 raw = s[i];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          v[8 * i + 2 * jj] = bf16_lo(w[jj]);
          v[8 * i + 2 * jj + 1] = bf16_hi(w[jj]);
          amax = fmaxf(amax, fmaxf(fabsf(v[8 * i + 2 * jj]), fabsf(v[8 * i + 2 * jj + 1])));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
    }
    float inv;
    const uint32_t eb = mxfp8_scale(amax, &inv);
    uint4* d = reinterpret_cast<uint4*>(xq + (size_t)r * Kp + k0);
    d[0] = make_uint4(e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv), e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                      e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv), e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
    d[1] = make_uint4(e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv), e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv),
                      e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv), e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv));
    sfx[((size_t)(blk >> 2) * max_tiles + tile) * SF_ATOM + sf_atom_offset(rin, blk & 3)] = (uint8_t)eb;
  }
}

// Decode (a handful of tokens): routing and quantisation in one launch.  One CTA per token: warp 0 picks the top-k experts while
// all threads round the token's row to MXFP8; the row is then written once per (token, slot) pair, each pair being its own
// one-row tile of the grouped GEMM (pair mode of mx_mxf4_gemm).
__global__ void __launch_bounds__(128) moe_route_quant_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int E, int Kt, int renorm,
                                                              int* __restrict__ topk_idx, float* __restrict__ topk_w, int w_copies, const __nv_bfloat16* __restrict__ x,
                                                              int ldx, int K, int KB, int max_tiles, uint8_t* __restrict__ xq, uint8_t* __restrict__ sfx) {
  pdl_prologue();
  const int t = blockIdx.x;
  if ((threadIdx.x >> 5) == 0) route_token_warp(logits, bias, t, E, Kt, renorm, topk_idx, topk_w, w_copies);
  const int Kp = KB * XT_K;
  for (int blk = threadIdx.x; blk < KB * 4; blk += blockDim.x) {
    const int k0 = blk * 32;
    float v[32];
    float amax = 0.f;
    if (k0 < K) {
      const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)t * ldx + k0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 raw = s[i];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          v[8 * i + 2 * jj] = bf16_lo(w[jj]);
          v[8 * i + 2 * jj + 1] = bf16_hi(w[jj]);
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
    for (int k = 0; k < Kt; ++k) {
      const size_t r = (size_t)t * Kt + k;            // pair = tile r, row 0 of its atom
      uint4* d = reinterpret_cast<uint4*>(xq + r * Kp + k0);
      d[0] = lo;
      d[1] = hi;
      sfx[((size_t)(blk >> 2) * max_tiles + r) * SF_ATOM + sf_atom_offset(0, blk & 3)] = (uint8_t)eb;
    }
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn2 encoder2() {
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    fn = (EncodeTiledFn2)f;
  }
  return fn;
}
// e4m3 activations [rows][inner] (one byte per element), boxes of 128 bytes x box_rows, 128-byte swizzle
static int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint64_t row_stride, uint32_t box_rows) {
  EncodeTiledFn2 enc = encoder2();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {inner, rows};
  cuuint64_t gstr[1] = {row_stride};
  cuuint32_t box[2] = {XT_K, box_rows}, es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
// packed E2M1 tiles: rows of 128 elements (64 bytes), expanded by TMA to 128 one-byte containers per row
static int make_tmap_fp4(CUtensorMap* out, const void* base, uint64_t rows) {
  EncodeTiledFn2 enc = encoder2();
  if (!enc) return -1;
  cuuint64_t gdim[2] = {XT_K, rows};
  cuuint64_t gstr[1] = {XT_K / 2};
  cuuint32_t box[2] = {XT_K, XT_N}, es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
}  // namespace mx

using namespace mx;

// Quantise activation rows to MXFP8 for mx_mxf4_gemm.
//   x [*, ldx] bf16; destination row r reads source row (src_index ? src_index[r] : r) / x_div; negative index = skip
//   row_limit: optional device int[2], rows >= row_limit[1] are skipped (the packer's live row count)
//   xq [rows][KB*128] e4m3, sfx [KB][max_tiles][512] scale atoms; rows_per_tile 128 (padded expert segments) or 1 (pair mode)
MX_HOST_API int mx_moe_quant(const void* x, int ldx, const int* src_index, int x_div, const int* row_limit, int rows, int K, int max_tiles,
                             int rows_per_tile, void* xq, void* sfx, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (K % 32 || ldx % 8 || x_div < 1 || (rows_per_tile != 1 && rows_per_tile != 128)) return -101;
  const int KB = (K + XT_K - 1) / XT_K;
  launch_pdl(moe_quant_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)x, ldx, src_index, x_div, row_limit, K, KB, max_tiles,
             rows_per_tile, (uint8_t*)xq, (uint8_t*)sfx);
  return (int)cudaGetLastError();
}

// Router top-k (see mx_moe_route) and MXFP8 quantisation of T token rows in pair mode: xq [T*Kt][KB*128], sfx [KB][max_tiles][512]
// with max_tiles >= T*Kt; pair t*Kt+k is tile t*Kt+k.  topk_w is [T][w_copies][Kt]: the weights repeated (one per partial row when
// the down projection that follows splits K).
MX_HOST_API int mx_moe_route_quant(const float* logits, const float* bias, int T, int E, int Kt, int renorm, int* topk_idx, float* topk_w, int w_copies,
                                   const void* x, int ldx, int K, int max_tiles, void* xq, void* sfx, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 1024 || Kt > 32 || Kt > E || K % 32 || ldx % 8 || max_tiles < T * Kt) return -120;
  const int KB = (K + XT_K - 1) / XT_K;
  launch_pdl(moe_route_quant_kernel, dim3(T), dim3(128), 0, st, logits, bias, E, Kt, renorm, topk_idx, topk_w, w_copies < 1 ? 1 : w_copies, (const __nv_bfloat16*)x, ldx, K, KB,
             max_tiles, (uint8_t*)xq, (uint8_t*)sfx);
  return (int)cudaGetLastError();
}

// Expert projection over token tiles, weights from a tiled MXFP4 bank of n_experts experts ([E][FB][KB][192][64] codes, [E][FB][KB][2][512] scales).
//   dual = 0: out[row][f] = sum_k xq[row][k] * W_e[f][k] + bias0[e][f]                       -> bf16 `out` [x_rows][ldo]
//   dual = 1: the bank interleaves 96 gate rows and 96 up rows per tile; act(gate + bias0, up + bias1) is written as MXFP8:
//             `oq` [x_rows][oq_ld] e4m3 (oq_ld = N rounded up to 128) + scale atoms `osf` [oq_ld / 128][max_tiles][512]
//   xq [x_rows][KB*128] e4m3 with scale atoms sfx [KB][max_tiles][512]
//   tile_expert[max_tiles] (global ids, bank starts at e_lo), tile_valid nullable (then every tile has default_valid live rows),
//   num_tiles_dev nullable; N = output features (of gate and of up each when dual), a multiple of 32 when dual
MX_HOST_API int mx_mxf4_gemm(const void* w, const void* sfw, int dual, int n_experts, const void* xq, const void* sfx, int x_rows, int N, int K,
                             const int* tile_expert, const int* tile_valid, int default_valid, const int* num_tiles_dev, int max_tiles,
                             int row_stride, int e_lo, const float* bias0, const float* bias1, void* out, int ldo, void* oq, void* osf, int oq_ld,
                             int act, float act_alpha, float act_limit, int ksplit, cudaStream_t st) {
  if (max_tiles <= 0 || x_rows <= 0) return 0;
  if (ksplit < 1 || (dual && ksplit != 1)) return -104;
  if (K % 32 || (row_stride != 1 && row_stride != 128)) return -101;
  if (dual && (act == 0 || N % 32 || oq_ld % 128 || oq_ld < N || !oq || !osf)) return -102;
  if (!dual && !out) return -103;
  Mxf4Params p;
  p.N = N; p.K = K; p.dual = dual;
  p.FB = dual ? (N + XT_HALF - 1) / XT_HALF : (N + XT_N - 1) / XT_N;
  p.KB = (K + XT_K - 1) / XT_K;
  p.KBS = (p.KB + ksplit - 1) / ksplit;
  p.KS = (p.KB + p.KBS - 1) / p.KBS;             // every range owns at least one k-block
  p.split_rows = x_rows;
  p.max_tiles = max_tiles; p.row_stride = row_stride; p.e_lo = e_lo; p.n_experts = n_experts;
  p.num_tiles_dev = num_tiles_dev; p.tile_expert = tile_expert; p.tile_valid = tile_valid; p.default_valid = default_valid;
  p.sfw = (const uint8_t*)sfw; p.sfx = (const uint8_t*)sfx;
  p.bias0 = bias0; p.bias1 = bias1;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.oq = (uint8_t*)oq; p.osf = (uint8_t*)osf; p.oq_ld = oq_ld;
  p.act = act; p.act_alpha = act_alpha; p.act_limit = act_limit;
  p.status = status_word();
  CUtensorMap tw, tx16, tx32, tx64, tx128;
  int r = make_tmap_fp4(&tw, w, (uint64_t)n_experts * p.FB * p.KB * XT_N);
  if (r) return r;
  const uint64_t Kp = (uint64_t)p.KB * XT_K;
  if ((r = make_tmap_u8(&tx16, xq, Kp, x_rows, Kp, 16))) return r;
  if ((r = make_tmap_u8(&tx32, xq, Kp, x_rows, Kp, 32))) return r;
  if ((r = make_tmap_u8(&tx64, xq, Kp, x_rows, Kp, 64))) return r;
  if ((r = make_tmap_u8(&tx128, xq, Kp, x_rows, Kp, 128))) return r;
  const long long items = (long long)max_tiles * p.FB * p.KS;
  const int grid = items < sm_count() ? (int)items : sm_count();
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(mxf4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, XLayout::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured.mark();
  }
  launch_pdl(mxf4_gemm_kernel, dim3(grid), dim3(192), XLayout::TOTAL, st, tw, tx16, tx32, tx64, tx128, p);
  return (int)cudaGetLastError();
}
