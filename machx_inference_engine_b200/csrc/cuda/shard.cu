// Row-sharded residual stream for prefill under tensor / expert parallelism.
//
// Each rank owns T / W token rows of the residual.  Between the layers' GEMMs only two kinds of traffic cross NVLink,
// all of it plain peer stores into a workspace that every rank has mapped (CUDA IPC), signalled with release / acquire
// flags at system scope and consumed by kernels that wait with a time limit:
//
//   gather    shard_norm_kernel adds the reduced partials to its rows, normalises them and stores the bf16 rows into the
//             gather buffer of EVERY rank; the column-parallel GEMM that follows (gemm_tcgen05.cu, `gathered` mode) waits
//             per row chunk for the owner's flag and starts on the chunks that have arrived: all-gather -> GEMM.
//   scatter   the row-parallel GEMM's epilogue stores each output row only into its owner's inbox (comm.cuh, rs_rows);
//             the owner's next shard_norm_kernel sums the W partials: GEMM -> reduce-scatter.
//   dispatch  expert parallelism: each rank routes only its own rows.  moe_dispatch_plan_kernel exchanges per-expert counts
//             (every rank learns the whole W x E matrix, so every placement below is computed locally and is the same on every
//             run), moe_dispatch_send_kernel quantises a row to MXFP8 once and stores it into the packed expert segments of
//             the ranks that own its top-k experts, moe_return_kernel sends each expert output row back to the rank that owns
//             the token, and moe_combine_wait_kernel forms the weighted sum in slot order.
//
// Buffers are reused layer after layer without acknowledgements: a rank can only write a buffer of layer l + 1 after it has
// consumed what all ranks produced in layer l, and each of those was produced after its producer had finished reading that
// buffer in layer l (see the per-kernel notes).  Only plain loads and stores touch peer memory.
//
// Reference parity: replaces the replicated-activation scheme of src/model/dense_tp.cpp:361,402,416 (broadcast + two all-reduces
// per layer) and the replicated packing of include/ie/qwen3moe_tp.hpp:19-37 / src/model/qwen3moe_tp.cpp:653,662.
#include "comm.cuh"
#include "host_util.h"

#include <cuda_fp8.h>
#include <cstring>

namespace mx {

enum : int { FL_GATHER = 0, FL_COUNT = 1, FL_SEND = 2, FL_RET = 3, FL_KINDS = 4 };

struct ShardWs {
  uint8_t* base[kMaxPeers];   // workspace of every rank (index = rank)
  int world, my_rank;
  long long off_gather;       // bf16 [2][t_max][H]
  long long gather_stride;    // bytes of one gather buffer
  long long off_cnt;          // int32 [W][E]: row s is written by rank s
  long long off_xq;           // u8 [p_max][Kp]: MXFP8 rows received for this rank's experts
  long long off_sf;           // u8 [p_max][sf_ld]: their scale bytes, one row each
  long long off_meta;         // int32 [p_max]: (source rank << 24) | slot of the source's return buffer
  long long off_ret;          // bf16 [r_max * K][H]: expert outputs returned to the token owner
  long long off_flags;        // int32 [FL_KINDS][kMaxPeers]
  int* seq;                   // device int[FL_KINDS], local: last published sequence number per flag kind
  int* ticket;                // device int[FL_KINDS], local: CTA arrival counters
  int wait_cycles_log2;       // waits give up after 2^this SM cycles
};

__device__ __forceinline__ int* ws_flags(const ShardWs& ws, int rank, int kind) {
  return reinterpret_cast<int*>(ws.base[rank] + ws.off_flags) + kind * kMaxPeers;
}

// One thread waits until flag `f` reached `seq`; false (and the status word set) when the limit ran out.
__device__ __forceinline__ bool wait_flag(const int* f, int seq, int limit_log2, int* status) {
  if (ld_acquire_sys(f) - seq >= 0) return true;
  const long long t0 = clock64(), limit = 1ll << limit_log2;
  for (;;) {
    if (ld_acquire_sys(f) - seq >= 0) return true;
    __nanosleep(64);
    if (clock64() - t0 > limit) { atomicCAS(status, 0, ERR_PEER_FLAG_TIMEOUT); return false; }
  }
}
// The CTA waits for the flags of all ranks (one thread per rank polls).
__device__ __forceinline__ bool wait_all(const ShardWs& ws, int kind, int seq, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < ws.world) {
    if (!wait_flag(ws_flags(ws, ws.my_rank, kind) + threadIdx.x, seq, ws.wait_cycles_log2, status)) s_fail = 1;
  }
  __syncthreads();
  return s_fail == 0;
}
// Every thread of every CTA calls this after its last peer store of flag kind `kind`; the last CTA publishes `next` to all ranks.
__device__ __forceinline__ void publish(const ShardWs& ws, int kind, int next) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd((unsigned*)ws.ticket + kind, 1u);
    if (prev == total - 1) {
      ws.ticket[kind] = 0;
      __threadfence_system();
      for (int r = 0; r < ws.world; ++r) st_release_sys(ws_flags(ws, r, kind) + ws.my_rank, next);
      ws.seq[kind] = next;
    }
  }
}

// ------------------------------------------------------------------------------------------ residual add + RMSNorm on a shard
struct ShardNormArgs {
  float* x;                   // [R][H] fp32 residual rows of this rank (updated in place)
  int H;
  const float* w;
  float eps;
  int one_plus_w;
  float delta_scale;
  int mode;                   // 0 no delta, 1 local fp32 delta [R][H], 2 local bf16 delta, 3 partials in the reduce-scatter inbox
  const void* delta;
  const float* dbias;         // bias of the row-parallel layer whose partials are summed (added once)
  const uint8_t* inbox;       // mode 3: this rank's inbox (comm.cuh layout)
  long long slot_bytes;
  const int* inbox_seq;
  int inbox_bf16;
  int row0;                   // absolute row of local row 0
  __nv_bfloat16* out_local;   // [R][H] bf16, nullable
  int gather;                 // 1: also store the normalised rows into gather buffer `gbuf` of every rank
  int gbuf;
  int* status;
};

__global__ void __launch_bounds__(256) shard_norm_kernel(const ShardNormArgs a, const ShardWs ws) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int H = a.H;
  const int gnext = a.gather ? ws.seq[FL_GATHER] + 1 : 0;
  bool ok = true;
  const uint8_t* pbase = nullptr;
  if (a.mode == 3) {
    const int s = *a.inbox_seq;
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < ws.world) {
      const int* flags = reinterpret_cast<const int*>(a.inbox + 2ll * ws.world * a.slot_bytes);
      if (!wait_flag(flags + threadIdx.x, s, ws.wait_cycles_log2, a.status)) s_ok = 0;
    }
    __syncthreads();
    ok = s_ok != 0;
    pbase = a.inbox + (long long)(s & 1) * ws.world * a.slot_bytes;
  }
  float* xr = a.x + (size_t)t * H;
  __shared__ float red[8];
  float ss = 0.f;
  if (ok) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + i);
      if (a.mode) {
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.mode == 1) {
          d = *reinterpret_cast<const float4*>((const float*)a.delta + (size_t)t * H + i);
        } else if (a.mode == 2) {
          const uint2 dv = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)a.delta + (size_t)t * H + i);
          d = make_float4(bf16_lo(dv.x), bf16_hi(dv.x), bf16_lo(dv.y), bf16_hi(dv.y));
        } else {
          for (int r = 0; r < ws.world; ++r) {       // rank order: the same sum on every run
            const uint8_t* slot = pbase + r * a.slot_bytes;
            float4 p;
            if (a.inbox_bf16) {
              const uint2 dv = __ldcg(reinterpret_cast<const uint2*>((const __nv_bfloat16*)slot + (size_t)(a.row0 + t) * H + i));
              p = make_float4(bf16_lo(dv.x), bf16_hi(dv.x), bf16_lo(dv.y), bf16_hi(dv.y));
            } else {
              p = __ldcg(reinterpret_cast<const float4*>((const float*)slot + (size_t)(a.row0 + t) * H + i));
            }
            d.x += p.x; d.y += p.y; d.z += p.z; d.w += p.w;
          }
        }
        if (a.dbias) { d.x += a.dbias[i]; d.y += a.dbias[i + 1]; d.z += a.dbias[i + 2]; d.w += a.dbias[i + 3]; }
        v.x += d.x * a.delta_scale; v.y += d.y * a.delta_scale; v.z += d.z * a.delta_scale; v.w += d.w * a.delta_scale;
        *reinterpret_cast<float4*>(xr + i) = v;
      }
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / H + a.eps);
  }
  __syncthreads();
  const float inv = red[0];
  if (ok && (a.out_local || a.gather)) {
    const long long goff = ws.off_gather + (long long)a.gbuf * ws.gather_stride + ((long long)(a.row0 + t) * H) * 2;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      float4 g = *reinterpret_cast<const float4*>(a.w + i);
      if (a.one_plus_w) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
      const uint2 o = make_uint2(pack_bf16(v.x * inv * g.x, v.y * inv * g.y), pack_bf16(v.z * inv * g.z, v.w * inv * g.w));
      if (a.out_local) *reinterpret_cast<uint2*>(a.out_local + (size_t)t * H + i) = o;
      if (a.gather)
        for (int d = 0; d < ws.world; ++d) *reinterpret_cast<uint2*>(ws.base[d] + goff + (long long)i * 2) = o;
    }
  }
  if (a.gather) publish(ws, FL_GATHER, gnext);
}

// ------------------------------------------------------------------------------------------ expert dispatch: plan
// One CTA.  Pairs are (token, slot) of this rank's rows in row-major order; expert e lives on rank e / e_per_rank.
// Outputs (local): pair_pos[n] = row of the pair inside the owner's packed buffer; for this rank's own experts the tile
// table of the grouped GEMM: tile_expert[], tile_valid[], num_tiles[0] = live 128-row tiles, num_tiles[1] = packed rows.
// Shared memory: int cnt_all[W][E], int hist[nwarps][E], int seg[E], int base[E].
constexpr int PLAN_BATCH = 8;

__global__ void __launch_bounds__(1024) moe_dispatch_plan_kernel(const int* __restrict__ topk_idx, int n, int E, int e_per_rank, const ShardWs ws,
                                                                int* __restrict__ pair_pos, int* __restrict__ tile_expert, int* __restrict__ tile_valid,
                                                                int* __restrict__ num_tiles, int max_tiles, int* status) {
  pdl_prologue();
  extern __shared__ int s_mem[];
  const int W = ws.world, me = ws.my_rank;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int* s_all = s_mem;                    // [W][E]
  int* s_hist = s_all + W * E;           // [nwarps][E]
  int* s_seg = s_hist + nwarps * E;      // [E] first packed row of the expert on its owner
  int* s_base = s_seg + E;               // [E] first packed row of MY pairs of the expert
  __shared__ int s_fail;
  const int next = ws.seq[FL_COUNT] + 1;
  const int chunk = ((n + nwarps - 1) / nwarps + 31) & ~31;
  const int c0 = warp * chunk, c1 = min(n, c0 + chunk);
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) s_hist[i] = 0;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  // (the kernel is a chain of short phases: a warp fetches its pairs eight steps at a time, so a pass costs one trip to memory)
  for (int b0 = c0; b0 < c1; b0 += 32 * PLAN_BATCH) {
    int ev[PLAN_BATCH];
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) {
      const int i = b0 + 32 * u + lane;
      ev[u] = i < c1 ? topk_idx[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u)
      if (ev[u] >= 0) atomicAdd(&s_hist[warp * E + ev[u]], 1);
  }
  __syncthreads();
  // per expert: warp histograms -> exclusive cursors; my count goes to every rank's matrix row `me`
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) { const int c = s_hist[w * E + e]; s_hist[w * E + e] = run; run += c; }
    for (int d = 0; d < W; ++d) reinterpret_cast<int*>(ws.base[d] + ws.off_cnt)[me * E + e] = run;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) for (int d = 0; d < W; ++d) st_release_sys(ws_flags(ws, d, FL_COUNT) + me, next);
  if (threadIdx.x < W && !wait_flag(ws_flags(ws, me, FL_COUNT) + threadIdx.x, next, ws.wait_cycles_log2, status)) s_fail = 1;
  __syncthreads();
  if (s_fail) return;
  const int* cnt = reinterpret_cast<const int*>(ws.base[me] + ws.off_cnt);
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) s_all[i] = __ldcg(cnt + i);
  __syncthreads();
  // segment starts on every owner (padded to 128-row tiles), then my base inside each segment
  if (threadIdx.x < W) {
    const int d = threadIdx.x;
    int off = 0;
    for (int e = d * e_per_rank; e < min(E, (d + 1) * e_per_rank); ++e) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_all[s * E + e];
      s_seg[e] = off;
      off += (tot + 127) & ~127;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int b = s_seg[e];
    for (int s = 0; s < me; ++s) b += s_all[s * E + e];
    s_base[e] = b;
  }
  // tile table of my own experts: every expert writes its own entries (its first tile is its segment start / 128)
  {
    const int e_first = me * e_per_rank, e_last = min(E, (me + 1) * e_per_rank) - 1;
    const int e = e_first + threadIdx.x;
    if (e <= e_last) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_all[s * E + e];
      const int t0 = s_seg[e] >> 7;
      for (int r = 0, k = 0; r < tot && t0 + k < max_tiles; r += 128, ++k) {
        tile_expert[t0 + k] = e;
        tile_valid[t0 + k] = min(128, tot - r);
      }
      if (e == e_last) {
        const int rows = s_seg[e] + ((tot + 127) & ~127);
        num_tiles[0] = min(rows >> 7, max_tiles);
        num_tiles[1] = rows;
        ws.seq[FL_COUNT] = next;
      }
    }
  }
  __syncthreads();
  // stable placement: pairs of one expert keep their pair order
  for (int b0 = c0; b0 < c1; b0 += 32 * PLAN_BATCH) {
    int ev[PLAN_BATCH];
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) {
      const int i = b0 + 32 * u + lane;
      ev[u] = i < c1 ? topk_idx[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < PLAN_BATCH; ++u) {
      if (b0 + 32 * u >= c1) break;          // warp-uniform
      const int i = b0 + 32 * u + lane;
      const int e = ev[u];
      const unsigned m = __match_any_sync(0xffffffffu, e >= 0 ? e : E + lane);
      int cur = 0;
      if (e >= 0) cur = s_hist[warp * E + e];
      __syncwarp();
      if (e >= 0) {
        pair_pos[i] = s_base[e] + cur + __popc(m & ((1u << lane) - 1));
        if (lane == 31 - __clz(m)) s_hist[warp * E + e] = cur + __popc(m);
      }
      __syncwarp();
    }
  }
}

// ------------------------------------------------------------------------------------------ expert dispatch: quantise + send
__device__ __forceinline__ uint32_t shard_mxfp8_scale(float amax, float* inv) {
  if (!(amax > 0.f)) { *inv = 1.f; return 127u; }
  int ex = (int)((__float_as_uint(amax) >> 23) & 0xFF) - 8;
  ex = max(1, min(ex, 253));
  if (amax * __uint_as_float((uint32_t)(254 - ex) << 23) > 448.f) ex = min(ex + 1, 253);
  *inv = __uint_as_float((uint32_t)(254 - ex) << 23);
  return (uint32_t)ex;
}
__device__ __forceinline__ uint32_t shard_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// One CTA per token row: the row is rounded to MXFP8 once (the rule of moe_quant_kernel) into shared memory and then stored
// into the packed buffer of each of the K ranks that own one of its experts, with its scale bytes and its return address.
// Shared memory: Kp + sf_ld bytes.
__global__ void __launch_bounds__(128) moe_dispatch_send_kernel(const __nv_bfloat16* __restrict__ h, int H, int Kp, int sf_ld, const int* __restrict__ topk_idx,
                                                                const int* __restrict__ pair_pos, int K, int e_per_rank, const ShardWs ws) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t s_row[];
  uint8_t* s_sf = s_row + Kp;
  const int t = blockIdx.x;
  const int next = ws.seq[FL_SEND] + 1;
  for (int blk = threadIdx.x; blk < Kp / 32; blk += blockDim.x) {
    const int k0 = blk * 32;
    float v[32];
    float amax = 0.f;
    if (k0 < H) {
      const uint4* s = reinterpret_cast<const uint4*>(h + (size_t)t * H + k0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 raw = s[i];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[8 * i + 2 * j] = bf16_lo(w[j]);
          v[8 * i + 2 * j + 1] = bf16_hi(w[j]);
          amax = fmaxf(amax, fmaxf(fabsf(v[8 * i + 2 * j]), fabsf(v[8 * i + 2 * j + 1])));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
    }
    float inv;
    const uint32_t eb = shard_mxfp8_scale(amax, &inv);
    uint4* d = reinterpret_cast<uint4*>(s_row + k0);
    d[0] = make_uint4(shard_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv), shard_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv),
                      shard_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv), shard_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv));
    d[1] = make_uint4(shard_e4m3x4(v[16] * inv, v[17] * inv, v[18] * inv, v[19] * inv), shard_e4m3x4(v[20] * inv, v[21] * inv, v[22] * inv, v[23] * inv),
                      shard_e4m3x4(v[24] * inv, v[25] * inv, v[26] * inv, v[27] * inv), shard_e4m3x4(v[28] * inv, v[29] * inv, v[30] * inv, v[31] * inv));
    s_sf[blk] = (uint8_t)eb;
  }
  for (int i = Kp / 32 + threadIdx.x; i < sf_ld; i += blockDim.x) s_sf[i] = 127;
  __syncthreads();
  for (int k = 0; k < K; ++k) {
    const int i = t * K + k;
    const int d = topk_idx[i] / e_per_rank;
    const long long pos = pair_pos[i];
    uint4* xq = reinterpret_cast<uint4*>(ws.base[d] + ws.off_xq + pos * Kp);
    for (int j = threadIdx.x; j < Kp / 16; j += blockDim.x) xq[j] = reinterpret_cast<const uint4*>(s_row)[j];
    uint4* sf = reinterpret_cast<uint4*>(ws.base[d] + ws.off_sf + pos * sf_ld);
    if (threadIdx.x < sf_ld / 16) sf[threadIdx.x] = reinterpret_cast<const uint4*>(s_sf)[threadIdx.x];
    if (threadIdx.x == 0) reinterpret_cast<int*>(ws.base[d] + ws.off_meta)[pos] = (ws.my_rank << 24) | i;
  }
  publish(ws, FL_SEND, next);
}

// Receiver: once every rank's rows have arrived, the scale bytes of packed row p move into the 512-byte atoms the GEMM reads
// (row p = tile p / 128, row p % 128 of its atom; k-block q of stage kb at byte (r % 32) * 16 + (r / 32) * 4 + q).
__global__ void __launch_bounds__(128) moe_recv_finalize_kernel(const ShardWs ws, const int* __restrict__ num_tiles, int sf_ld, int n_blk, int max_tiles,
                                                                uint8_t* __restrict__ sfx, int* status) {
  pdl_prologue();
  if (!wait_all(ws, FL_SEND, ws.seq[FL_SEND], status)) return;
  const int rows = num_tiles[1];
  const uint8_t* sf = ws.base[ws.my_rank] + ws.off_sf;
  for (int p = blockIdx.x; p < rows; p += gridDim.x) {
    const int tile = p >> 7, r = p & 127;
    for (int blk = threadIdx.x; blk < n_blk; blk += blockDim.x)
      sfx[((size_t)(blk >> 2) * max_tiles + tile) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (blk & 3)] = __ldcg(sf + (size_t)p * sf_ld + blk);
  }
}

// Expert outputs go back to the rank that owns the token: packed row p -> slot meta[p] of the source's return buffer.
__global__ void __launch_bounds__(128) moe_return_kernel(const __nv_bfloat16* __restrict__ y, int H, const int* __restrict__ num_tiles,
                                                         const int* __restrict__ tile_valid, const ShardWs ws) {
  pdl_prologue();
  const int next = ws.seq[FL_RET] + 1;
  const int rows = num_tiles[1];
  const int* meta = reinterpret_cast<const int*>(ws.base[ws.my_rank] + ws.off_meta);
  for (int p = blockIdx.x; p < rows; p += gridDim.x) {
    if ((p & 127) >= tile_valid[p >> 7]) continue;
    const int m = __ldcg(meta + p);
    const int src = (m >> 24) & 0xFF, slot = m & 0xFFFFFF;
    const uint4* s = reinterpret_cast<const uint4*>(y + (size_t)p * H);
    uint4* d = reinterpret_cast<uint4*>(ws.base[src] + ws.off_ret + (long long)slot * H * 2);
    for (int j = threadIdx.x; j < H / 8; j += blockDim.x) d[j] = s[j];
  }
  publish(ws, FL_RET, next);
}

// delta[t][:] = sum_k w[t][k] * ret[t * K + k][:]   (slot order: the same sum on every run)
__global__ void __launch_bounds__(256) moe_combine_wait_kernel(const ShardWs ws, const float* __restrict__ w, float* __restrict__ out, int H, int K,
                                                               int* status) {
  pdl_prologue();
  if (!wait_all(ws, FL_RET, ws.seq[FL_RET], status)) return;
  const int t = blockIdx.x;
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(ws.base[ws.my_rank] + ws.off_ret);
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < K; ++k) {
      const uint2 v = __ldcg(reinterpret_cast<const uint2*>(ret + (size_t)(t * K + k) * H + i));
      const float ww = w[(size_t)t * K + k];
      a.x = fmaf(ww, bf16_lo(v.x), a.x); a.y = fmaf(ww, bf16_hi(v.x), a.y);
      a.z = fmaf(ww, bf16_lo(v.y), a.z); a.w = fmaf(ww, bf16_hi(v.y), a.w);
    }
    *reinterpret_cast<float4*>(out + (size_t)t * H + i) = a;
  }
}

}  // namespace mx

using namespace mx;

// Host-side description of the workspace, filled by parallel/sharded.py (offsets in bytes from each rank's base).
struct MxShardWs {
  void* base[8];
  int world, my_rank;
  long long off_gather, gather_stride, off_cnt, off_xq, off_sf, off_meta, off_ret, off_flags;
  int* seq;
  int* ticket;
  int wait_cycles_log2;
};
static ShardWs to_ws(const MxShardWs* h) {
  ShardWs ws;
  memset(&ws, 0, sizeof ws);
  for (int r = 0; r < h->world && r < kMaxPeers; ++r) ws.base[r] = (uint8_t*)h->base[r];
  ws.world = h->world; ws.my_rank = h->my_rank;
  ws.off_gather = h->off_gather; ws.gather_stride = h->gather_stride; ws.off_cnt = h->off_cnt; ws.off_xq = h->off_xq; ws.off_sf = h->off_sf;
  ws.off_meta = h->off_meta; ws.off_ret = h->off_ret; ws.off_flags = h->off_flags;
  ws.seq = h->seq; ws.ticket = h->ticket;
  ws.wait_cycles_log2 = h->wait_cycles_log2 > 0 ? h->wait_cycles_log2 : 31;
  return ws;
}

MX_HOST_API int mx_shard_ws_struct_bytes() { return (int)sizeof(MxShardWs); }

// x [R][H] fp32 (+= delta), normalised rows to out_local and / or gather buffer gbuf of every rank at absolute rows row0...
// mode: 0 none, 1 fp32 delta, 2 bf16 delta, 3 reduce-scatter inbox (inbox, slot_bytes, inbox_seq, inbox_bf16)
MX_HOST_API int mx_shard_norm(const MxShardWs* hws, float* x, int R, int H, const float* w, float eps, int one_plus_w, float delta_scale, int mode,
                              const void* delta, const float* dbias, const void* inbox, long long slot_bytes, const int* inbox_seq, int inbox_bf16,
                              int row0, void* out_local, int gather, int gbuf, cudaStream_t st) {
  if (R <= 0) return 0;
  if (H % 4) return -107;
  ShardNormArgs a;
  a.x = x; a.H = H; a.w = w; a.eps = eps; a.one_plus_w = one_plus_w; a.delta_scale = delta_scale; a.mode = mode; a.delta = delta; a.dbias = dbias;
  a.inbox = (const uint8_t*)inbox; a.slot_bytes = slot_bytes; a.inbox_seq = inbox_seq; a.inbox_bf16 = inbox_bf16; a.row0 = row0;
  a.out_local = (__nv_bfloat16*)out_local; a.gather = gather; a.gbuf = gbuf; a.status = status_word();
  launch_pdl(shard_norm_kernel, dim3(R), dim3(256), 0, st, a, to_ws(hws));
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_dispatch_plan(const MxShardWs* hws, const int* topk_idx, int n_pairs, int E, int e_per_rank, int* pair_pos, int* tile_expert,
                                     int* tile_valid, int* num_tiles, int max_tiles, cudaStream_t st) {
  if (E > 1024 || hws->world > kMaxPeers) return -120;
  const int smem = (hws->world * E + 32 * E + 2 * E) * (int)sizeof(int);
  static DeviceOnce attr;
  if (attr.pending()) {
    cudaError_t e = cudaFuncSetAttribute(moe_dispatch_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (8 + 32 + 2) * 1024 * (int)sizeof(int));
    if (e != cudaSuccess) return (int)e;
    attr.mark();
  }
  launch_pdl(moe_dispatch_plan_kernel, dim3(1), dim3(1024), smem, st, topk_idx, n_pairs, E, e_per_rank, to_ws(hws), pair_pos, tile_expert, tile_valid,
             num_tiles, max_tiles, status_word());
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_dispatch_send(const MxShardWs* hws, const void* h, int R, int H, int Kp, int sf_ld, const int* topk_idx, const int* pair_pos, int K,
                                     int e_per_rank, cudaStream_t st) {
  if (R <= 0) return 0;
  if (H % 32 || Kp % 128 || Kp < H || sf_ld % 16 || sf_ld < Kp / 32) return -101;
  launch_pdl(moe_dispatch_send_kernel, dim3(R), dim3(128), (size_t)(Kp + sf_ld), st, (const __nv_bfloat16*)h, H, Kp, sf_ld, topk_idx, pair_pos, K,
             e_per_rank, to_ws(hws));
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_recv_finalize(const MxShardWs* hws, const int* num_tiles, int sf_ld, int n_blk, int max_tiles, void* sfx, cudaStream_t st) {
  const int grid = max_tiles * 128 < 4 * sm_count() ? max_tiles * 128 : 4 * sm_count();
  launch_pdl(moe_recv_finalize_kernel, dim3(grid < 1 ? 1 : grid), dim3(128), 0, st, to_ws(hws), num_tiles, sf_ld, n_blk, max_tiles, (uint8_t*)sfx, status_word());
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_return(const MxShardWs* hws, const void* y, int H, const int* num_tiles, const int* tile_valid, int max_tiles, cudaStream_t st) {
  if (H % 8) return -101;
  const int grid = max_tiles * 128 < 8 * sm_count() ? max_tiles * 128 : 8 * sm_count();
  launch_pdl(moe_return_kernel, dim3(grid < 1 ? 1 : grid), dim3(128), 0, st, (const __nv_bfloat16*)y, H, num_tiles, tile_valid, to_ws(hws));
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_combine_wait(const MxShardWs* hws, const float* w, float* out, int R, int H, int K, cudaStream_t st) {
  if (R <= 0) return 0;
  if (H % 4) return -107;
  launch_pdl(moe_combine_wait_kernel, dim3(R), dim3(256), 0, st, to_ws(hws), w, out, H, K, status_word());
  return (int)cudaGetLastError();
}
