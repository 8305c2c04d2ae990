// Prefill FlashAttention on the sm_100a tensor cores: head_dim 64, 128 or 256, paged KV, causal, sliding window with
// whole-tile skipping, attention sinks, logit soft-cap, GQA.
//
// One CTA owns 128 query tokens of one query head and walks the key tiles of its range (128 keys per tile, 64 for
// head_dim 256 so that two K and two V tiles still fit in shared memory):
//   warp 0  : TMA loads of the K and V tiles (two-stage rings) and, once, of the Q tile
//   warp 1  : tcgen05.mma  S(j) = Q K_j^T  into one of two S buffers in TMEM, so that S(j+1) is computed while the softmax
//             threads work on S(j);  O += P_j V_j  accumulates in TMEM over all tiles
//   warps 2-5 (one thread per query row = TMEM lane): read S, mask, online softmax, write P (bf16) into a 128-byte-swizzled
//             shared tile for the PV MMA.  The output row is NOT kept in registers: O stays in TMEM and is rescaled in place
//             (tcgen05.ld / tcgen05.st) only when the running maximum has grown by more than 2^8 since the last rescale;
//             until then P is formed against the old reference maximum (it stays far inside bf16's range) and O and the
//             denominator remain consistent.  That removes the per-tile fold of O and is what lets head_dim 256 fit.
// The per-head sink joins the denominator once, at the end.  Every wait is bounded.
//
// Reference parity: src/ops/attention.cpp:2456-2815 (fa2_tile_wide_impl<HD,Bc,REGDOT,SG,SINK> for HD 64..512 and its
// dispatcher: causal and window masks per key, whole-tile skip outside the window, sink folded at row end); the soft-cap
// of src/model/gemma4.cpp's attention is applied to the scores here.
#include "common.cuh"
#include "host_util.h"

namespace mx {

constexpr int FA_BQ = 128;     // query rows per CTA
constexpr int FA_PAGE = 128;   // KV page size

struct FaParams {
  const int* block_table;  // [B][max_blocks]
  const int* seq_lens;     // [B]
  const int* cu_q;         // [B+1]
  const float* sinks;      // [n_q] or null
  __nv_bfloat16* out;      // [Tq][n_q][hd]
  int n_q, n_kv, max_blocks, max_q_tiles, window;
  float scale, softcap;
  int* status;
};

template <int HD>
struct FaCfg {
  static constexpr int BKV = HD <= 128 ? 128 : 64;            // keys per tile
  static constexpr int NS = 2;                                 // S buffers in TMEM
  static constexpr int CTAS = 1;                               // one CTA per SM: its softmax threads keep a whole S row in registers
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr int ATOMS = HD / 64;                        // 64-column (128-byte) swizzle atoms per row of Q / K / V
  static constexpr int Q_BYTES = FA_BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int KS = 2, VS = 2;                         // tiles in flight
  static constexpr int P_BYTES = FA_BQ * BKV * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + KS * KV_BYTES;
  static constexpr int P_OFF = V_OFF + VS * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
  static_assert(TOTAL <= 232448, "shared memory plan exceeds 227 KB");
  static_assert(NS * BKV + HD <= (int)TMEM_COLS, "TMEM plan");
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD, bool CAP>
__global__ void __launch_bounds__(192, FaCfg<HD>::CTAS)
fa_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  using L = FaCfg<HD>;
  constexpr int BKV = L::BKV, NS = L::NS, KS = L::KS, VS = L::VS;
  constexpr float LOG2E = 1.4426950408889634f;
  constexpr float RESCALE_STEP = 8.f;            // in log2 units: O is rescaled when the maximum has grown by a factor of 256
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  // barriers: q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_empty[2], p_full, pv_done
  const uint32_t b_qfull = smem_u32(bars), b_kfull = b_qfull + 8, b_vfull = b_kfull + 16, b_kempty = b_vfull + 16, b_vempty = b_kempty + 16;
  const uint32_t b_sfull = b_vempty + 16, b_sempty = b_sfull + 16, b_pfull = b_sempty + 16, b_pvdone = b_pfull + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
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
  const int tile_lo = kv_lo / BKV, tile_hi = (kv_hi + BKV - 1) / BKV;
  const int n_tiles = tile_hi - tile_lo;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_kfull + 8 * s, 1); mbar_init(b_vfull + 8 * s, 1); mbar_init(b_kempty + 8 * s, 1); mbar_init(b_vempty + 8 * s, 1);
      mbar_init(b_sfull + 8 * s, 1); mbar_init(b_sempty + 8 * s, 4);
    }
    mbar_init(b_pfull, 4); mbar_init(b_pvdone, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), L::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + NS * BKV;

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
        const int key0 = (tile_lo + j) * BKV;
        const int blk = p.block_table[(size_t)b * p.max_blocks + key0 / FA_PAGE];
        const int krow = key0 % FA_PAGE;
        if (!(ok = mbar_wait(b_kempty + 8 * sk, phk ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
        mbar_expect_tx(b_kfull + 8 * sk, L::KV_BYTES);
#pragma unroll
        for (int a = 0; a < L::ATOMS; ++a)
          tma_load_4d(sbase + L::K_OFF + sk * L::KV_BYTES + a * (BKV * 128), &tmap_k, b_kfull + 8 * sk, a * 64, krow, kvh, blk);
        if (!(ok = mbar_wait(b_vempty + 8 * sv, phv ^ 1, p.status, ERR_MBAR_TIMEOUT_PRODUCER, abort_flag))) break;
        mbar_expect_tx(b_vfull + 8 * sv, L::KV_BYTES);
#pragma unroll
        for (int a = 0; a < L::ATOMS; ++a)
          tma_load_4d(sbase + L::V_OFF + sv * L::KV_BYTES + a * (BKV * 128), &tmap_v, b_vfull + 8 * sv, a * 64, krow, kvh, blk);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(FA_BQ, HD, 0, 1);      // B = V is MN-major (head_dim contiguous)
      bool ok = mbar_wait(b_qfull, 0, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag);
      // S(j) = Q K_j^T into S buffer j % NS (waits for K_j and for the softmax threads to have released that buffer)
      auto issue_s = [&](int j) -> bool {
        const uint32_t sk = j % KS, phk = (j / KS) & 1, sb = j % NS, phs = (j / NS) & 1;
        if (!mbar_wait(b_kfull + 8 * sk, phk, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag)) return false;
        if (!mbar_wait(b_sempty + 8 * sb, phs ^ 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = sbase + L::Q_OFF, ka = sbase + L::K_OFF + sk * L::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ad = umma_desc_k_sw128(qa + (kk >> 2) * (FA_BQ * 128) + (kk & 3) * 32);
          const uint64_t bd = umma_desc_k_sw128(ka + (kk >> 2) * (BKV * 128) + (kk & 3) * 32);
          umma_bf16(tmem_base + sb * BKV, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(b_sfull + 8 * sb);
        umma_commit(b_kempty + 8 * sk);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (NS == 2 && j + 1 < n_tiles && !(ok = issue_s(j + 1))) break;       // the next score tile runs while softmax(j) works
        const uint32_t sv = j % VS, phv = (j / VS) & 1;
        if (!(ok = mbar_wait(b_pfull, j & 1, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        if (!(ok = mbar_wait(b_vfull + 8 * sv, phv, p.status, ERR_MBAR_TIMEOUT_MMA, abort_flag))) break;
        tc_fence_after();
        const uint32_t pa = sbase + L::P_OFF, va = sbase + L::V_OFF + sv * L::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t ad = umma_desc_k_sw128(pa + (kk >> 2) * (FA_BQ * 128) + (kk & 3) * 32);
          const uint64_t bd = umma_desc_mn_sw128(va + kk * 2048, BKV * 128, 1024);
          umma_bf16(tmem_o, ad, bd, idesc_o, (j | kk) != 0);
        }
        umma_commit(b_pvdone);
        umma_commit(b_vempty + 8 * sv);
        if (NS == 1 && j + 1 < n_tiles && !(ok = issue_s(j + 1))) break;
      }
    }
  } else {
    // ------------------------------------------------ softmax, one thread per query row
    // Per score: one max, one fused multiply-add, one ex2, half a pack and one add.  The whole S row of the tile sits in
    // registers, so the S buffer goes back to the MMA thread before the exponentials start.
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;                  // row inside the tile == TMEM lane
    const int qpos = pos0 + r;
    const bool row_ok = r < rows;
    const float c = CAP ? 1.f : p.scale * LOG2E;   // factor from the stored score to log2 units
    const float cap_c = p.softcap * LOG2E, inv_cap = CAP ? p.scale / p.softcap : 0.f;
    float m = -1e30f, l = 0.f;                     // reference maximum (log2 units) and running denominator
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t sb = j % NS, phs = (j / NS) & 1;
      if (!(ok = mbar_wait(b_sfull + 8 * sb, phs, p.status, ERR_MBAR_TIMEOUT_SOFTMAX, abort_flag))) break;
      tc_fence_after();
      const uint32_t ts = tmem_base + lane_addr + sb * BKV;
      float sv[BKV];
#pragma unroll
      for (int cb = 0; cb < BKV; cb += 32) tmem_ld_32x32(ts + cb, *reinterpret_cast<uint32_t(*)[32]>(&sv[cb]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(b_sempty + 8 * sb);
      const int key0 = (tile_lo + j) * BKV;
      if (CAP) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) sv[i] = cap_c * tanh_fast(sv[i] * inv_cap);
      }
      // a tile needs per-key masking only at the diagonal, at the window edge and at the sequence end
      if ((key0 + BKV - 1 > pos0) || (p.window > 0 && key0 <= pos0 + FA_BQ - 1 - p.window) || (key0 + BKV > seq_len)) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kpos = key0 + i;
          const bool keep = kpos <= qpos && kpos < seq_len && (p.window <= 0 || kpos > qpos - p.window);
          sv[i] = keep ? sv[i] : -INFINITY;
        }
      }
      float tmax = sv[0];
#pragma unroll
      for (int i = 1; i < BKV; ++i) tmax = fmaxf(tmax, sv[i]);
      tmax *= c;                                   // c > 0
      // P(j) overwrites the shared tile PV(j-1) reads, and a rescale touches the accumulator PV(j-1) writes: both wait for it
      if (j > 0 && !(ok = mbar_wait(b_pvdone, (j - 1) & 1, p.status, ERR_MBAR_TIMEOUT_SOFTMAX, abort_flag))) break;
      // tcgen05.ld / tcgen05.st are warp-wide instructions: the decision to rescale is taken per warp, and a row whose own
      // maximum has not grown simply rescales by 1
      const bool grow = tmax > m + RESCALE_STEP || j == 0;
      const float m_new = grow ? fmaxf(m, tmax) : m;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        const float alpha = ex2_fast(m - m_new);
        l *= alpha;
        tc_fence_after();
#pragma unroll 1
        for (int cb = 0; cb < HD; cb += 32) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_o + lane_addr + cb, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st_32x32(tmem_o + lane_addr + cb, ov);
        }
        tmem_st_wait();
      }
      m = m_new;
      float psum = 0.f;
      const float neg_m = -m;
#pragma unroll
      for (int cb = 0; cb < BKV; cb += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2_fast(fmaf(sv[cb + i], c, neg_m)), p1 = ex2_fast(fmaf(sv[cb + i + 1], c, neg_m));
          psum += p0 + p1;
          pk[i >> 1] = pack_bf16(p0, p1);
        }
        // 32 keys = 64 bytes = 4 chunks of this row, in atom (cb / 64), chunks (cb % 64) / 8 ..
        uint8_t* prow = smem + L::P_OFF + (cb >> 6) * (FA_BQ * 128);
        const int ch0 = (cb & 63) >> 3;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(prow + sw128_offset(r, ch0 + ch)) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      }
      l += psum;
      tc_fence_before();            // a rescale's TMEM stores, before the MMA thread is told to accumulate into O again
      fence_proxy_async();          // the P tile, written through the generic proxy, before the MMA reads it
      __syncwarp();
      if (lane == 0) mbar_arrive(b_pfull);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(b_pvdone, (n_tiles - 1) & 1, p.status, ERR_MBAR_TIMEOUT_SOFTMAX, abort_flag);
    if (ok) {
      tc_fence_after();
      if (p.sinks) l += ex2_fast(p.sinks[head] * LOG2E - m);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + ((size_t)(q_begin + t0 + r) * p.n_q + head) * HD;
#pragma unroll 1
      for (int cb = 0; cb < HD; cb += 32) {
        uint32_t ov[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_o + lane_addr + cb, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(orow + cb + i) =
                make_uint4(pack_bf16(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv), pack_bf16(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv),
                           pack_bf16(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv), pack_bf16(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv));
        }
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

template <int HD, bool CAP>
static int launch_fa(const void* q, const void* k_cache, const void* v_cache, const FaParams& p, int B, int Tq, int n_blocks, cudaStream_t st) {
  using L = FaCfg<HD>;
  CUtensorMap tq, tk, tv;
  {
    uint64_t dims[3] = {(uint64_t)HD, (uint64_t)p.n_q, (uint64_t)Tq};
    uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)HD * 2 * p.n_q};
    uint32_t box[3] = {64, 1, FA_BQ};
    int r = make_tmap_bf16(&tq, q, 3, dims, strides, box, 1);
    if (r) return r;
  }
  {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)FA_PAGE, (uint64_t)p.n_kv, (uint64_t)n_blocks};
    uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)HD * 2 * FA_PAGE, (uint64_t)HD * 2 * FA_PAGE * p.n_kv};
    uint32_t box[4] = {64, (uint32_t)L::BKV, 1, 1};
    int r = make_tmap_bf16(&tk, k_cache, 4, dims, strides, box, 1);
    if (r) return r;
    r = make_tmap_bf16(&tv, v_cache, 4, dims, strides, box, 1);
    if (r) return r;
  }
  auto kern = fa_prefill_kernel<HD, CAP>;
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

// Tensor-core prefill attention.  Requirements: head_dim 64, 128 or 256, KV page size 128.  softcap > 0 applies
// cap * tanh(score / cap) to the scaled scores.  n_blocks is the number of pages in the cache tensors (their leading dimension).
MX_HOST_API int mx_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens,
                                        const int* cu_q, const float* sinks, void* out, int B, int Tq, int max_q_len, int n_q, int n_kv,
                                        int hd, int max_blocks, int n_blocks, int block_size, int window, float scale, float softcap,
                                        cudaStream_t st) {
  if (B <= 0 || Tq <= 0) return 0;
  if (block_size != FA_PAGE) return -110;
  if (n_q % n_kv) return -111;
  FaParams p;
  p.block_table = block_table; p.seq_lens = seq_lens; p.cu_q = cu_q; p.sinks = sinks; p.out = (__nv_bfloat16*)out;
  p.n_q = n_q; p.n_kv = n_kv; p.max_blocks = max_blocks; p.window = window; p.scale = scale; p.softcap = softcap;
  p.max_q_tiles = (max_q_len + FA_BQ - 1) / FA_BQ;
  p.status = status_word();
  const bool cap = softcap > 0.f;
  if (hd == 64) return cap ? launch_fa<64, true>(q, k_cache, v_cache, p, B, Tq, n_blocks, st) : launch_fa<64, false>(q, k_cache, v_cache, p, B, Tq, n_blocks, st);
  if (hd == 128) return cap ? launch_fa<128, true>(q, k_cache, v_cache, p, B, Tq, n_blocks, st) : launch_fa<128, false>(q, k_cache, v_cache, p, B, Tq, n_blocks, st);
  if (hd == 256) return cap ? launch_fa<256, true>(q, k_cache, v_cache, p, B, Tq, n_blocks, st) : launch_fa<256, false>(q, k_cache, v_cache, p, B, Tq, n_blocks, st);
  return -112;
}
