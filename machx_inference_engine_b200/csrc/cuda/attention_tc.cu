// Prefill FlashAttention on the sm_100a tensor cores (head_dim 64 or 128, paged KV, causal,
// sliding window with whole-tile skipping, attention sinks, GQA).
//
// One CTA owns 128 query tokens of one query head.  Per 128-key tile (= one KV page):
//   warp 0  : TMA loads of the K and V pages (two-stage ring) and, once, of the Q tile
//   warp 1  : tcgen05.mma  S = Q K^T  (fp32, 128 x 128 in TMEM)  and  O_tile = P V  (128 x hd in TMEM)
//   warps 2-5 (one thread per query row): read S from TMEM, mask, online softmax, write P (bf16)
//             into a 128-byte-swizzled shared tile for the PV MMA, then fold O_tile into the
//             running output kept in registers (rescaled by exp(m_old - m_new)).
// S(j+1) is issued right after PV(j), so the next score tile is computed while the softmax threads
// accumulate O(j); with head_dim 64 two CTAs share an SM (192 TMEM columns, ~100 KB shared each).
// The per-head sink joins the denominator once, at the end.  Every wait is bounded.
//
// Reference parity: src/ops/attention.cpp:2456-2735 (fa2_tile_wide_impl<HD,Bc,REGDOT,SG,SINK>: causal
// and window masks per key, whole-tile skip outside the window, sink folded at row end).
#include "common.cuh"
#include "host_util.h"

namespace mx {

constexpr int FA_BQ = 128;     // query rows per CTA
constexpr int FA_BKV = 128;    // keys per tile = KV page size

struct FaParams {
  const int* block_table;  // [B][max_blocks]
  const int* seq_lens;     // [B]
  const int* cu_q;         // [B+1]
  const float* sinks;      // [n_q] or null
  __nv_bfloat16* out;      // [Tq][n_q][hd]
  int n_q, n_kv, max_blocks, max_q_tiles, window;
  float scale;
  int* status;
};

template <int HD>
struct FaSmem {
  static constexpr int ATOMS = HD / 64;                 // 64-column (128-byte) swizzle atoms per row
  static constexpr int Q_BYTES = FA_BQ * HD * 2;
  static constexpr int KV_BYTES = FA_BKV * HD * 2;
  static constexpr int KS = 2;                          // K pages in flight
  static constexpr int VS = HD == 64 ? 1 : 2;           // V pages in flight (one keeps head_dim 64 at two CTAs per SM)
  static constexpr int P_BYTES = FA_BQ * FA_BKV * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + KS * KV_BYTES;
  static constexpr int P_OFF = V_OFF + VS * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(192, HD == 64 ? 2 : 1)
fa_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using L = FaSmem<HD>;
  constexpr uint32_t TMEM_COLS = 256;       // S: 128 columns, O tile: HD columns
  constexpr float LOG2E = 1.4426950408889634f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  // barriers: q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full, s_empty, p_full, o_full, o_empty
  const uint32_t b_qfull = smem_u32(bars), b_kfull = b_qfull + 8, b_vfull = b_kfull + 16, b_kempty = b_vfull + 16, b_vempty = b_kempty + 16;
  const uint32_t b_sfull = b_vempty + 16, b_sempty = b_sfull + 8, b_pfull = b_sempty + 8, b_ofull = b_pfull + 8, b_oempty = b_ofull + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  constexpr int KS = L::KS, VS = L::VS;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / p.max_q_tiles, qt = blockIdx.x % p.max_q_tiles;
  const int head = blockIdx.y;
  const int kvh = head / (p.n_q / p.n_kv);
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int t0 = qt * FA_BQ;
  if (t0 >= q_len) return;                       // whole CTA leaves before any barrier / TMEM use
  const int seq_len = p.seq_lens[b];
  const int pos0 = seq_len - q_len + t0;         // absolute position of query row 0 of this tile
  const int rows = min(FA_BQ, q_len - t0);
  const int kv_hi = min(seq_len, pos0 + rows);   // exclusive
  const int kv_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int tile_lo = kv_lo / FA_BKV, tile_hi = (kv_hi + FA_BKV - 1) / FA_BKV;
  const int n_tiles = tile_hi - tile_lo;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(b_kfull + 8 * s, 1); mbar_init(b_vfull + 8 * s, 1); mbar_init(b_kempty + 8 * s, 1); mbar_init(b_vempty + 8 * s, 1); }
    mbar_init(b_sfull, 1); mbar_init(b_sempty, 4); mbar_init(b_pfull, 4); mbar_init(b_ofull, 1); mbar_init(b_oempty, 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_expect_tx(b_qfull, L::Q_BYTES);
#pragma unroll
      for (int a = 0; a < L::ATOMS; ++a)
        tma_load_3d(sbase + L::Q_OFF + a * (FA_BQ * 128), &tmap_q, b_qfull, a * 64, head, q_begin + t0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t sk = j % KS, phk = (j / KS) & 1, sv = j % VS, phv = (j / VS) & 1;
        const int blk = p.block_table[(size_t)b * p.max_blocks + tile_lo + j];
        if (!(ok = mbar_wait(b_kempty + 8 * sk, phk ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
        mbar_expect_tx(b_kfull + 8 * sk, L::KV_BYTES);
#pragma unroll
        for (int a = 0; a < L::ATOMS; ++a)
          tma_load_4d(sbase + L::K_OFF + sk * L::KV_BYTES + a * (FA_BKV * 128), &tmap_k, b_kfull + 8 * sk, a * 64, 0, kvh, blk);
        if (!(ok = mbar_wait(b_vempty + 8 * sv, phv ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
        mbar_expect_tx(b_vfull + 8 * sv, L::KV_BYTES);
#pragma unroll
        for (int a = 0; a < L::ATOMS; ++a)
          tma_load_4d(sbase + L::V_OFF + sv * L::KV_BYTES + a * (FA_BKV * 128), &tmap_v, b_vfull + 8 * sv, a * 64, 0, kvh, blk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BQ, FA_BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(FA_BQ, HD, 0, 1);      // B = V is MN-major (head_dim contiguous)
      bool ok = mbar_wait(b_qfull, 0, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag);
      auto issue_s = [&](int j) {
        const uint32_t s = j % KS;
        const uint32_t qa = sbase + L::Q_OFF, ka = sbase + L::K_OFF + s * L::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (FA_BQ * 128) + (kk & 3) * 32;
          umma_bf16(tmem_s, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(ka + off), idesc_s, kk != 0);
        }
        umma_commit(b_sfull);
        umma_commit(b_kempty + 8 * s);
      };
      if (ok && n_tiles > 0) {
        ok = mbar_wait(b_kfull, 0, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag);
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t s = j % VS, ph = (j / VS) & 1;
        if (!(ok = mbar_wait(b_pfull, j & 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        if (!(ok = mbar_wait(b_vfull + 8 * s, ph, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        if (j > 0 && !(ok = mbar_wait(b_oempty, (j - 1) & 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        tc_fence_after();
        const uint32_t pa = sbase + L::P_OFF, va = sbase + L::V_OFF + s * L::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < FA_BKV / 16; ++kk) {
          const uint64_t ad = umma_desc_k_sw128(pa + (kk >> 2) * (FA_BQ * 128) + (kk & 3) * 32);
          const uint64_t bd = umma_desc_mn_sw128(va + kk * 2048, FA_BKV * 128, 1024);
          umma_bf16(tmem_o, ad, bd, idesc_o, kk != 0);
        }
        umma_commit(b_ofull);
        umma_commit(b_vempty + 8 * s);
        if (j + 1 < n_tiles) {
          const uint32_t s1 = (j + 1) % KS, ph1 = ((j + 1) / KS) & 1;
          if (!(ok = mbar_wait(b_kfull + 8 * s1, ph1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          if (!(ok = mbar_wait(b_sempty, j & 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
          tc_fence_after();
          issue_s(j + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------ softmax + output accumulation, one thread per query row
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;                  // row inside the tile == TMEM lane
    const int qpos = pos0 + r;
    const bool row_ok = r < rows;
    const float c = p.scale * LOG2E;
    float m = -1e30f, l = 0.f;                     // running max (in scaled-score * log2e units) and sum
    float acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) acc[i] = 0.f;
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!(ok = mbar_wait(b_sfull, j & 1, p.status, ERR_MBAR_TIMEOUT_SOFTMAX, abort_flag))) break;
      tc_fence_after();
      const int key0 = (tile_lo + j) * FA_BKV;
      // a tile needs per-key masking only at the diagonal, at the window edge and at the sequence end
      const bool need_mask = (key0 + FA_BKV - 1 > pos0) || (p.window > 0 && key0 <= pos0 + FA_BQ - 1 - p.window + 0) || (key0 + FA_BKV > seq_len);
      float tmax = -1e30f;
#pragma unroll 1
      for (int cb = 0; cb < FA_BKV; cb += 32) {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_s + lane_addr + cb, sv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(sv[i]) * c;
          if (need_mask) {
            const int kpos = key0 + cb + i;
            const bool keep = kpos <= qpos && kpos < seq_len && (p.window <= 0 || kpos > qpos - p.window);
            v = keep ? v : -1e30f;
          }
          tmax = fmaxf(tmax, v);
        }
      }
      const float m_new = fmaxf(m, tmax);
      const float alpha = exp2f(m - m_new);
      float psum = 0.f;
#pragma unroll 1
      for (int cb = 0; cb < FA_BKV; cb += 32) {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_s + lane_addr + cb, sv);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float v0 = __uint_as_float(sv[i]) * c, v1 = __uint_as_float(sv[i + 1]) * c;
          if (need_mask) {
            const int k0 = key0 + cb + i, k1 = k0 + 1;
            const bool keep0 = k0 <= qpos && k0 < seq_len && (p.window <= 0 || k0 > qpos - p.window);
            const bool keep1 = k1 <= qpos && k1 < seq_len && (p.window <= 0 || k1 > qpos - p.window);
            v0 = keep0 ? v0 : -INFINITY;
            v1 = keep1 ? v1 : -INFINITY;
          }
          const float p0 = exp2f(v0 - m_new), p1 = exp2f(v1 - m_new);
          // the PV product uses the bf16-rounded probabilities, so the denominator sums the same values
          const uint32_t w = pack_bf16(p0, p1);
          psum += bf16_lo(w) + bf16_hi(w);
          pk[i >> 1] = w;
        }
        // 32 keys = 64 bytes = 4 chunks of this row, in atom (cb / 64), chunks (cb % 64) / 8 ..
        uint8_t* prow = smem + L::P_OFF + (cb >> 6) * (FA_BQ * 128);
        const int ch0 = (cb & 63) >> 3;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(prow + sw128_offset(r, ch0 + ch)) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      }
      l = l * alpha + psum;
      m = m_new;
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { mbar_arrive(b_pfull); mbar_arrive(b_sempty); }
      // fold the PV tile into the running output
      if (!(ok = mbar_wait(b_ofull, j & 1, p.status, ERR_MBAR_TIMEOUT_SOFTMAX, abort_flag))) break;
      tc_fence_after();
#pragma unroll
      for (int cb = 0; cb < HD; cb += 32) {
        uint32_t ov[32];
        tmem_ld_32x32(tmem_o + lane_addr + cb, ov);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[cb + i] = fmaf(acc[cb + i], alpha, __uint_as_float(ov[i]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(b_oempty);
    }
    if (ok && row_ok) {
      if (p.sinks) l += exp2f(p.sinks[head] * LOG2E - m);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(q_begin + t0 + r) * p.n_q + head) * HD;
#pragma unroll
      for (int i = 0; i < HD; i += 8)
        *reinterpret_cast<uint4*>(orow + i) = make_uint4(pack_bf16(acc[i] * inv, acc[i + 1] * inv), pack_bf16(acc[i + 2] * inv, acc[i + 3] * inv),
                                                         pack_bf16(acc[i + 4] * inv, acc[i + 5] * inv), pack_bf16(acc[i + 6] * inv, acc[i + 7] * inv));
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int HD>
static int launch_fa(const void* q, const void* k_cache, const void* v_cache, const FaParams& p, int B, int Tq, int n_blocks, cudaStream_t st) {
  using L = FaSmem<HD>;
  CUtensorMap tq, tk, tv;
  {
    uint64_t dims[3] = {(uint64_t)HD, (uint64_t)p.n_q, (uint64_t)Tq};
    uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)HD * 2 * p.n_q};
    uint32_t box[3] = {64, 1, FA_BQ};
    int r = make_tmap_bf16(&tq, q, 3, dims, strides, box, 1);
    if (r) return r;
  }
  {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)FA_BKV, (uint64_t)p.n_kv, (uint64_t)n_blocks};
    uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)HD * 2 * FA_BKV, (uint64_t)HD * 2 * FA_BKV * p.n_kv};
    uint32_t box[4] = {64, FA_BKV, 1, 1};
    int r = make_tmap_bf16(&tk, k_cache, 4, dims, strides, box, 1);
    if (r) return r;
    r = make_tmap_bf16(&tv, v_cache, 4, dims, strides, box, 1);
    if (r) return r;
  }
  auto kern = fa_prefill_kernel<HD>;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured.mark();
  }
  dim3 grid(B * p.max_q_tiles, p.n_q);
  kern<<<grid, 192, L::TOTAL, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace mx

using namespace mx;

// Tensor-core prefill attention.  Requirements: head_dim 64 or 128, KV page size 128, no soft-cap.
// n_blocks is the number of pages in the cache tensors (their leading dimension).
MX_HOST_API int mx_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens,
                                        const int* cu_q, const float* sinks, void* out, int B, int Tq, int max_q_len, int n_q, int n_kv,
                                        int hd, int max_blocks, int n_blocks, int block_size, int window, float scale, cudaStream_t st) {
  if (B <= 0 || Tq <= 0) return 0;
  if (block_size != FA_BKV) return -110;
  if (n_q % n_kv) return -111;
  FaParams p;
  p.block_table = block_table; p.seq_lens = seq_lens; p.cu_q = cu_q; p.sinks = sinks; p.out = (__nv_bfloat16*)out;
  p.n_q = n_q; p.n_kv = n_kv; p.max_blocks = max_blocks; p.window = window; p.scale = scale;
  p.max_q_tiles = (max_q_len + FA_BQ - 1) / FA_BQ;
  p.status = status_word();
  if (hd == 64) return launch_fa<64>(q, k_cache, v_cache, p, B, Tq, n_blocks, st);
  if (hd == 128) return launch_fa<128>(q, k_cache, v_cache, p, B, Tq, n_blocks, st);
  return -112;
}
