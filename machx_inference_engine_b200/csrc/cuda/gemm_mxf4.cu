// Block-scaled MXFP4 grouped GEMM for sm_100a: the expert projections of gpt-oss on the 5th-generation
// tensor cores with nothing decoded on the ALUs.
//
//   * Weights stay packed E2M1 (4 bit) + e8m0 scale per 32 in global memory, repacked once at load time
//     into 128x128 tiles (ops/weights.py: to_mxf4_tiles).  TMA (16U4_ALIGN16B tensor map) expands a tile
//     into the padded 8-bit containers that `tcgen05.mma.kind::mxf8f6f4.block_scale` reads; the scale
//     factors travel as 512-byte atoms (bulk copy -> shared memory -> `tcgen05.cp` -> TMEM).
//   * Activations are MXFP8 (e4m3 + e8m0 per 32), produced by moe_quant_kernel below from the bf16
//     hidden rows while they are gathered into expert order.
//   * Operands are swapped: the 128 weight rows of a tile are the M side of the instruction and the
//     tokens of one expert are its N side (16..96 per instruction, chosen per work item at run time
//     through the instruction descriptor).  An expert with 3 rows costs a 16-column instruction, not a
//     128-row tile, and one launch serves prefill (hundreds of rows per expert) and decode (one row).
//   * gate and up are two weight banks multiplied into two accumulators of the same TMEM lanes, so the
//     gated activation needs no cross-lane traffic in the epilogue.
//   * The kernel is bound by the weight stream: one elected thread issues TMA for a ring of stages,
//     one thread issues tcgen05.cp / tcgen05.mma, four warps drain double-buffered accumulators.
//
// Reference parity: replaces the per-expert dequant + oneDNN GEMM chain of src/model/gptoss_tp.cpp:685-765
// and the MXFP4 GEMV family of src/ops/gemv_mxfp4.cpp:94-323 for the expert projections.
#include "common.cuh"
#include "host_util.h"

#include <cuda_fp8.h>
#include <mutex>

namespace mx {

constexpr int XT_M = 128;        // weight rows per tile (instruction M)
constexpr int XT_K = 128;        // elements of K per stage (4 instructions of K = 32)
constexpr int XT_N = 96;         // token columns per work item (instruction N <= 96)
constexpr int SF_ATOM = 512;     // bytes of one scale-factor atom: 128 rows x 4 k-blocks

// scale-factor atom: row r (0..127), k-block q (0..3) -> byte (r % 32) * 16 + (r / 32) * 4 + q
__host__ __device__ constexpr int sf_atom_offset(int r, int q) { return (r & 31) * 16 + (r >> 5) * 4 + q; }

struct Mxf4Params {
  int N, K;                       // output features per expert, logical K
  int NB, KB;                     // 128-row feature blocks, 128-element k blocks
  int max_tiles;                  // host bound on token tiles; scale atoms of the activations are [KB][max_tiles][512]
  int row_stride;                 // first row of token tile j is j * row_stride (128: padded expert segments, 1: one pair per tile)
  int e_lo, n_experts;            // tile_expert holds global expert ids; the banks hold experts [e_lo, e_lo + n_experts), other tiles are skipped
  const int* num_tiles_dev;       // live tile count (device), nullable
  const int* tile_expert;         // [max_tiles]
  const int* tile_valid;          // [max_tiles] live rows of each tile (1..128), nullable = default_valid
  int default_valid;
  const uint8_t* sfa0;            // weight scale atoms [E][NB][KB][512] (gate, or the only bank)
  const uint8_t* sfa1;            // up bank (dual only)
  const uint8_t* sfb;             // activation scale atoms
  const float* bias0;             // [E][N] nullable
  const float* bias1;
  __nv_bfloat16* out;             // [rows][ldo]
  int ldo;
  int act;                        // dual only: 1 SwiGLU, 2 clamped SwiGLU
  float act_alpha, act_limit;
  int* status;
};

template <bool DUAL>
struct XLayout {
  static constexpr int A_BYTES = XT_M * XT_K;                 // 16 KiB: 128 rows x 128 one-byte containers
  static constexpr int B_BYTES = XT_N * XT_K;                 // 12 KiB
  static constexpr int A0 = 0;
  static constexpr int A1 = A_BYTES;
  static constexpr int B = DUAL ? 2 * A_BYTES : A_BYTES;
  static constexpr int SF = B + B_BYTES;                      // SFA0, SFA1, SFB, pad: 4 x 512
  static constexpr int STAGE = SF + 2048;
  static constexpr int STAGES = DUAL ? 4 : 7;
  static constexpr int BAR_OFFSET = STAGES * STAGE;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;       // barriers + alignment slack
  static_assert(STAGE % 1024 == 0, "stage tiles must stay 1024-byte aligned");
  static_assert(TOTAL <= 232448, "shared memory plan exceeds 227 KB");
};

// kind::mxf8f6f4 instruction descriptor: A = E2M1 (code 5), B = E4M3 (code 0), ue8m0 scales, K-major operands.  The scale-factor
// ids (which of the four bytes of a scale column the instruction uses) are added per k-step: kk * MXF4_IDESC_KSTEP.
__device__ __forceinline__ uint32_t mxf4_idesc(int n) {
  return (5u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(XT_M >> 4) << 24);
}
constexpr uint32_t MXF4_IDESC_KSTEP = (1u << 4) | (1u << 29);

// The loops of the two single-thread roles are written for instruction count: one thread issues every copy or every MMA of an
// SM, and with 16..96-column instructions the tensor pipe finishes an instruction faster than a thread that rebuilds its
// descriptors can issue the next one (measured: 8 instructions per stage took 0.74 us with descriptors rebuilt per instruction).
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

__device__ __forceinline__ float mxf4_act(int act, float g, float u, float alpha, float limit) {
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
  }
  return g / (1.f + __expf(-g)) * u;
}

// work item t -> (token tile j, part h, feature block fb); returns the number of token columns to compute (<= 0: nothing to do).
// Part 0 covers rows 0..95 of the 128-row tile.  Part 1 exists when the tile has more than 96 live rows: it computes rows
// 64.. (the scale-factor address of an instruction moves in steps of two TMEM columns = 64 rows) and stores rows 96.. only.
constexpr int XT_PART1_ROW = 64, XT_PART1_SKIP = XT_N - XT_PART1_ROW;
__device__ __forceinline__ int item_decode(const Mxf4Params& p, int t, int& j, int& h, int& fb) {
  fb = t % p.NB;
  const int jh = t / p.NB;
  h = jh & 1;
  j = jh >> 1;
  const int e = p.tile_expert[j] - p.e_lo;
  if (e < 0 || e >= p.n_experts) return 0;
  const int valid = p.tile_valid ? p.tile_valid[j] : p.default_valid;
  if (h == 0) return min(valid, XT_N);
  return valid > XT_N ? valid - XT_PART1_ROW : 0;
}

template <bool DUAL>
__global__ void __launch_bounds__(192, 1)
mxf4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w0, const __grid_constant__ CUtensorMap tmap_w1,
                 const __grid_constant__ CUtensorMap tmap_x16, const __grid_constant__ CUtensorMap tmap_x32,
                 const __grid_constant__ CUtensorMap tmap_x64, const __grid_constant__ CUtensorMap tmap_x96, const Mxf4Params p) {
  using L = XLayout<DUAL>;
  constexpr int S = L::STAGES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ACC_COLS = 2 * XT_N;     // one accumulator buffer: gate columns, then up columns
  constexpr uint32_t SF_COL = 2 * ACC_COLS;   // scale factors: two buffers of 16 columns behind the accumulators
  static_assert(SF_COL + 32 <= TMEM_COLS, "TMEM plan");
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
  const int total = m_tiles * 2 * p.NB;

  if (warp == 0) {
    // ------------------------------------------------ producer: TMA tiles + bulk copies of the scale atoms
    if (lane == 0) {
      prefetch_tmap(&tmap_w0);
      if (DUAL) prefetch_tmap(&tmap_w1);
      prefetch_tmap(&tmap_x96);
      uint32_t s = 0, ph = 1, st = smem_base, fbar = bar_full, ebar = bar_empty;     // ring cursor (ph: parity to wait for on `empty`)
      const size_t sfb_step = (size_t)p.max_tiles * SF_ATOM;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int j, h, fb;
        const int nv = item_decode(p, t, j, h, fb);
        if (nv <= 0) continue;
        const int box = nv <= 16 ? 16 : (nv <= 32 ? 32 : (nv <= 64 ? 64 : 96));
        const CUtensorMap* tx = box == 16 ? &tmap_x16 : (box == 32 ? &tmap_x32 : (box == 64 ? &tmap_x64 : &tmap_x96));
        const long long wt = ((long long)(p.tile_expert[j] - p.e_lo) * p.NB + fb) * p.KB;   // first weight tile / scale atom of this slab
        const int row0 = j * p.row_stride + XT_PART1_ROW * h;
        // a packed-4-bit TMA load counts its packed bytes on the barrier (half of what it writes to shared memory)
        const uint32_t bytes = (DUAL ? 2 : 1) * (L::A_BYTES / 2 + SF_ATOM) + box * XT_K + SF_ATOM;
        int wy = (int)(wt * XT_M), kx = 0;
        const uint8_t* sa0 = p.sfa0 + wt * SF_ATOM;
        const uint8_t* sa1 = DUAL ? p.sfa1 + wt * SF_ATOM : nullptr;
        const uint8_t* sb = p.sfb + (size_t)j * SF_ATOM;
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!(ok = mbar_wait(ebar, ph, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
          mbar_expect_tx(fbar, bytes);
          tma_load_2d(st + L::A0, &tmap_w0, fbar, 0, wy);
          if (DUAL) tma_load_2d(st + L::A1, &tmap_w1, fbar, 0, wy);
          tma_load_2d(st + L::B, tx, fbar, kx, row0);
          bulk_load(st + L::SF, sa0, SF_ATOM, fbar);
          if (DUAL) bulk_load(st + L::SF + SF_ATOM, sa1, SF_ATOM, fbar);
          bulk_load(st + L::SF + 2 * SF_ATOM, sb, SF_ATOM, fbar);
          wy += XT_M; kx += XT_K; sa0 += SF_ATOM; sa1 += SF_ATOM; sb += sfb_step;
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
        int j, h, fb;
        const int nv = item_decode(p, t, j, h, fb);
        if (nv <= 0) continue;
        const uint32_t idesc = mxf4_idesc((nv + 15) & ~15);
        const uint32_t acc = item_n & 1, acc_ph = (item_n >> 1) & 1;
        ++item_n;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * ACC_COLS, d1 = d0 + XT_N;
        const uint32_t sfb_off = 8 + 2 * h;                             // rows 64.. of the tile sit in columns 2, 3 of the atom
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!(ok = mbar_wait(fbar, ph, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          tc_fence_after();
          const uint32_t sf = tmem_base + SF_COL + sfsel;               // alternate scale buffers between consecutive stages
          sfsel ^= 16;
          tmem_cp_sf(sf, st + L::SF);
          if (DUAL) tmem_cp_sf(sf + 4, st + L::SF + SF_ATOM);
          tmem_cp_sf(sf + 8, st + L::SF + 2 * SF_ATOM);
          const uint32_t a0 = desc_lo(st + L::A0), a1 = desc_lo(st + L::A1), b = desc_lo(st + L::B);
          const uint32_t sfb = sf + sfb_off;
          umma_mxf4<false>(d0, a0, b, idesc, sf, sfb, (uint32_t)kb);
          if (DUAL) umma_mxf4<false>(d1, a1, b, idesc, sf + 4, sfb, (uint32_t)kb);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) {      // 32 elements = 32 bytes per k-step: +2 in the descriptor's 16-byte units
            umma_mxf4<true>(d0, a0 + 2 * kk, b + 2 * kk, idesc + kk * MXF4_IDESC_KSTEP, sf, sfb);
            if (DUAL) umma_mxf4<true>(d1, a1 + 2 * kk, b + 2 * kk, idesc + kk * MXF4_IDESC_KSTEP, sf + 4, sfb);
          }
          umma_commit(ebar);
          st += L::STAGE; fbar += 8; ebar += 8;
          if (++s == S) { s = 0; ph ^= 1; st = smem_base; fbar = bar_full; ebar = bar_empty; }
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);
      }
    }
  } else {
    // ------------------------------------------------ epilogue: lane = weight row (output feature), column = token
    const int q = warp & 3;
    uint32_t item_n = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int j, h, fb;
      const int nv = item_decode(p, t, j, h, fb);
      if (nv <= 0) continue;
      const uint32_t acc = item_n & 1, acc_ph = (item_n >> 1) & 1;
      ++item_n;
      if (!(ok = mbar_wait(bar_tfull + 8 * acc, acc_ph, p.status, ERR_MBAR_TIMEOUT_EPILOGUE, abort_flag, 64))) break;
      tc_fence_after();
      const int e = p.tile_expert[j] - p.e_lo;
      const int f = fb * XT_M + q * 32 + lane;
      const bool f_ok = f < p.N;
      const float b0 = (p.bias0 && f_ok) ? p.bias0[(size_t)e * p.N + f] : 0.f;
      const float b1 = (DUAL && p.bias1 && f_ok) ? p.bias1[(size_t)e * p.N + f] : 0.f;
      __nv_bfloat16* out = p.out + (size_t)(j * p.row_stride + XT_PART1_ROW * h) * p.ldo + f;
      const uint32_t tl = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
#pragma unroll 1
      for (int c0 = h ? XT_PART1_SKIP : 0; c0 < nv; c0 += 32) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(tl + c0, g);
        if (DUAL) tmem_ld_32x32(tl + XT_N + c0, u);
        tmem_ld_wait();
        if (f_ok) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c0 + c < nv) {
              float v = __uint_as_float(g[c]) + b0;
              if (DUAL) v = mxf4_act(p.act, v, __uint_as_float(u[c]) + b1, p.act_alpha, p.act_limit);
              out[(size_t)(c0 + c) * p.ldo] = __float2bfloat16(v);
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
// One CTA per destination row r: source row = src_index ? src_index[r] : r, divided by x_div (pair mode: K pairs share a token row);
// rows whose index is negative (tile padding) are skipped; with `identity` the index only masks and the source row is r itself.  Thread i owns the 32-element block i of the row: amax -> e8m0 scale
// (the smallest power of two that keeps the block inside e4m3's range) -> 32 e4m3 bytes; the scale byte lands in the row's
// slot of the tile's scale atom.  Blocks between K and the padded KB * 128 are written as zeros with a unit scale.
__global__ void __launch_bounds__(128) moe_quant_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ src_index, int identity, int x_div,
                                                        const int* __restrict__ row_limit, int K, int KB, int max_tiles, int rows_per_tile,
                                                        uint8_t* __restrict__ xq, uint8_t* __restrict__ sfb) {
  pdl_prologue();
  const int r = blockIdx.x;
  if (row_limit && r >= row_limit[1]) return;
  int src = r;
  if (src_index) { src = src_index[r]; if (src < 0) return; if (identity) src = r; }
  src /= x_div;
  const int Kp = KB * XT_K;
  const int tile = r / rows_per_tile, rin = r - tile * rows_per_tile;
  for (int blk = threadIdx.x; blk < KB * 4; blk += blockDim.x) {
    const int k0 = blk * 32;
    uint4 raw[4];
    float amax = 0.f;
    const bool live = k0 < K;           // K is a multiple of 32
    if (live) {
      const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)src * ldx + k0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        raw[i] = s[i];
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(w[jj])), fabsf(bf16_hi(w[jj]))));
      }
    }
    uint32_t eb = 127;
    float inv = 1.f;
    if (live && amax > 0.f) {
      int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 8;           // floor(log2 amax) - 8, biased
      ex = max(1, min(ex, 253));
      if (amax * __uint_as_float((uint32_t)(254 - ex) << 23) > 448.f) ex = min(ex + 1, 253);
      eb = (uint32_t)ex;
      inv = __uint_as_float((uint32_t)(254 - ex) << 23);
    }
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        uint32_t packed = 0;
        if (live) {
          const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(bf16_lo(w[2 * jj]) * inv, bf16_hi(w[2 * jj]) * inv), __NV_SATFINITE, __NV_E4M3);
          const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(bf16_lo(w[2 * jj + 1]) * inv, bf16_hi(w[2 * jj + 1]) * inv), __NV_SATFINITE, __NV_E4M3);
          packed = (uint32_t)lo | ((uint32_t)hi << 16);
        }
        o[2 * i + jj] = packed;
      }
    }
    uint4* d = reinterpret_cast<uint4*>(xq + (size_t)r * Kp + k0);
    d[0] = make_uint4(o[0], o[1], o[2], o[3]);
    d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    sfb[((size_t)(blk >> 2) * max_tiles + tile) * SF_ATOM + sf_atom_offset(rin, blk & 3)] = (uint8_t)eb;
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
  cuuint32_t box[2] = {XT_K, XT_M}, es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
}  // namespace mx

using namespace mx;

// Quantise activation rows to MXFP8 for mx_mxf4_gemm.
//   x [*, ldx] bf16; destination row r reads source row (src_index ? src_index[r] : r) / x_div; negative index = skip;
//   identity != 0: src_index only masks, the source row is r
//   row_limit: optional device int[2], rows >= row_limit[1] are skipped (the packer's live row count)
//   xq [rows][KB*128] e4m3, sfb [KB][max_tiles][512] scale atoms; rows_per_tile 128 (padded expert segments) or 1 (pair mode)
MX_HOST_API int mx_moe_quant(const void* x, int ldx, const int* src_index, int identity, int x_div, const int* row_limit, int rows, int K, int max_tiles,
                             int rows_per_tile, void* xq, void* sfb, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (K % 32 || ldx % 8 || x_div < 1 || (rows_per_tile != 1 && rows_per_tile != 128)) return -101;
  const int KB = (K + XT_K - 1) / XT_K;
  launch_pdl(moe_quant_kernel, dim3(rows), dim3(128), 0, st, (const __nv_bfloat16*)x, ldx, src_index, identity, x_div, row_limit, K, KB, max_tiles,
             rows_per_tile, (uint8_t*)xq, (uint8_t*)sfb);
  return (int)cudaGetLastError();
}

// out[row][f] = sum_k xq[row][k] * W_e[f][k]   (+ bias, dual: act(gate, up)) for every live row of every token tile.
//   w0/sfa0 (+ w1/sfa1 when dual): tiled MXFP4 banks of n_experts experts [E][NB][KB][128][64] / [E][NB][KB][512]
//   xq [x_rows][KB*128] e4m3 with scale atoms sfb [KB][max_tiles][512]
//   tile_expert[max_tiles] (global ids, bank starts at e_lo), tile_valid nullable (then every tile has default_valid live rows),
//   num_tiles_dev nullable
//   out bf16 [x_rows][ldo]
MX_HOST_API int mx_mxf4_gemm(const void* w0, const void* sfa0, const void* w1, const void* sfa1, int n_experts, const void* xq, const void* sfb,
                             int x_rows, int N, int K, const int* tile_expert, const int* tile_valid, int default_valid, const int* num_tiles_dev, int max_tiles,
                             int row_stride, int e_lo, const float* bias0, const float* bias1, void* out, int ldo, int act, float act_alpha,
                             float act_limit, cudaStream_t st) {
  if (max_tiles <= 0 || x_rows <= 0) return 0;
  const bool dual = w1 != nullptr;
  if (K % 32 || (dual && act == 0) || (row_stride != 1 && row_stride != 128)) return -101;
  Mxf4Params p;
  p.N = N; p.K = K;
  p.NB = (N + XT_M - 1) / XT_M;
  p.KB = (K + XT_K - 1) / XT_K;
  p.max_tiles = max_tiles; p.row_stride = row_stride; p.e_lo = e_lo; p.n_experts = n_experts;
  p.num_tiles_dev = num_tiles_dev; p.tile_expert = tile_expert; p.tile_valid = tile_valid; p.default_valid = default_valid;
  p.sfa0 = (const uint8_t*)sfa0; p.sfa1 = (const uint8_t*)sfa1; p.sfb = (const uint8_t*)sfb;
  p.bias0 = bias0; p.bias1 = bias1;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.act = act; p.act_alpha = act_alpha; p.act_limit = act_limit;
  p.status = status_word();
  CUtensorMap tw0, tw1, tx16, tx32, tx64, tx96;
  const uint64_t wrows = (uint64_t)n_experts * p.NB * p.KB * XT_M;
  int r = make_tmap_fp4(&tw0, w0, wrows);
  if (r) return r;
  if (dual) { r = make_tmap_fp4(&tw1, w1, wrows); if (r) return r; } else tw1 = tw0;
  const uint64_t Kp = (uint64_t)p.KB * XT_K;
  if ((r = make_tmap_u8(&tx16, xq, Kp, x_rows, Kp, 16))) return r;
  if ((r = make_tmap_u8(&tx32, xq, Kp, x_rows, Kp, 32))) return r;
  if ((r = make_tmap_u8(&tx64, xq, Kp, x_rows, Kp, 64))) return r;
  if ((r = make_tmap_u8(&tx96, xq, Kp, x_rows, Kp, 96))) return r;
  const int items = max_tiles * 2 * p.NB;
  const int grid = items < sm_count() ? items : sm_count();
  static std::mutex mu;
  static bool configured[64][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!configured[dev & 63][dual]) {
      cudaError_t e = dual ? cudaFuncSetAttribute(mxf4_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, XLayout<true>::TOTAL)
                           : cudaFuncSetAttribute(mxf4_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, XLayout<false>::TOTAL);
      if (e != cudaSuccess) return (int)e;
      configured[dev & 63][dual] = true;
    }
  }
  if (dual) launch_pdl(mxf4_gemm_kernel<true>, dim3(grid), dim3(192), XLayout<true>::TOTAL, st, tw0, tw1, tx16, tx32, tx64, tx96, p);
  else launch_pdl(mxf4_gemm_kernel<false>, dim3(grid), dim3(192), XLayout<false>::TOTAL, st, tw0, tw1, tx16, tx32, tx64, tx96, p);
  return (int)cudaGetLastError();
}
