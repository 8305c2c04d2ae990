// Paged attention on CUDA cores: split-KV flash-decode, small-T verify, and the general
// varlen causal kernel (sliding window, attention sinks, GQA sharing, logit soft-cap).
//
// One CTA owns (query tile, kv head, kv split).  Each 64-key K/V tile is staged in shared
// memory once and shared by every (query token, query head) pair of the group; a warp runs
// the online softmax for its pairs with one key per lane, so there is no per-key reduction.
// Every split writes an un-normalised partial (acc, m, l); the CTA of a (query tile, kv head)
// group that finishes last (an atomic ticket per group, reset by its last taker) merges the
// splits and folds the per-head sink into the denominator exactly once, so that decode is one
// launch.  Splits that would get no key tile exit at once and are not counted.  The separate
// combine kernel remains for batches with more groups than there are tickets.
//
// KV cache layout: [block][kv_head][block_size][head_dim] bf16, block_size a multiple of 64.  An int8 cache has the
// same layout with one byte per element plus an fp32 scale per (block, kv head, token) row (value = q * scale); the
// staging loop widens it to bf16, so the math below is shared.  kv_dequant_pages_kernel expands the pages of a prefill
// batch into a bf16 scratch cache for the tensor-core prefill kernel.
//
// Reference parity: src/ops/attention.cpp:229-454 (naive / gpt-oss window + sink),
// :685-1036 (split-K flash decode, sink folded in combine), :2456-2714 (wide tile prefill with
// causal + window masks and whole-tile skipping).
#include "common.cuh"
#include "host_util.h"
#include "mx_noalloc.h"

#include <cstdio>

namespace mx {

constexpr int ATT_WARPS = 8;
constexpr int ATT_TILE = 64;

struct AttnParams {
  const __nv_bfloat16* q;      // [Tq][n_q][hd]
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const float* k_scale;        // non-null: the caches hold int8 and these are the per-row scales [block][kv_head][block_size]
  const float* v_scale;
  const int* block_table;      // [B][max_blocks]
  const int* seq_lens;         // [B] kv length including this step's tokens
  const int* cu_q;             // [B+1]
  float* o_part;               // [splits][Tq][n_q][hd]
  float* ml_part;              // [splits][Tq][n_q][2]
  int* tickets;                // non-null: one counter per (batch entry, query tile, kv head) group; the last split merges
  const float* sinks;          // [n_q] or null (used by the merging CTA)
  __nv_bfloat16* out;          // [Tq][n_q][hd] (written by the merging CTA)
  int B, n_q, n_kv, max_blocks, block_size;
  int q_tile;                  // query tokens per CTA
  int max_q_tiles;             // per sequence
  int n_splits;
  int Tq;
  int window;                  // 0 = full causal
  float scale, softcap;
};

// bytes `first`, `first + 1` of w as signed 8-bit integers, times scale, packed as two bf16
__device__ __forceinline__ uint32_t s8x2_to_bf16x2(uint32_t w, int first, float scale) {
  const float a = (float)(int8_t)(w >> (8 * first)) * scale, b = (float)(int8_t)(w >> (8 * first + 8)) * scale;
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Pages of an int8 cache expanded to bf16: dst page (b * nb + j) = page block_table[b][j] of the source, for every page
// that holds keys of sequence b.  One CTA per (j, b, kv head).
__global__ void __launch_bounds__(256) kv_dequant_pages_kernel(const int8_t* __restrict__ k8, const int8_t* __restrict__ v8,
                                                               const float* __restrict__ ks, const float* __restrict__ vs,
                                                               const int* __restrict__ block_table, const int* __restrict__ seq_lens,
                                                               __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int n_kv,
                                                               int block_size, int hd, int max_blocks, int nb) {
  pdl_prologue();
  const int j = blockIdx.x, b = blockIdx.y, kvh = blockIdx.z;
  if ((long long)j * block_size >= seq_lens[b]) return;
  const int blk = block_table[(size_t)b * max_blocks + j];
  const size_t src = ((size_t)blk * n_kv + kvh) * block_size, dst = (((size_t)b * nb + j) * n_kv + kvh) * block_size;
  const int per_row = hd / 8;
  for (int i = threadIdx.x; i < block_size * per_row; i += blockDim.x) {
    const int r = i / per_row, c = (i % per_row) * 8;
    const uint2 kq = *reinterpret_cast<const uint2*>(k8 + (src + r) * hd + c);
    const uint2 vq = *reinterpret_cast<const uint2*>(v8 + (src + r) * hd + c);
    const float sk_ = ks[src + r], sv_ = vs[src + r];
    uint4 ko, vo;
    ko.x = s8x2_to_bf16x2(kq.x, 0, sk_); ko.y = s8x2_to_bf16x2(kq.x, 2, sk_); ko.z = s8x2_to_bf16x2(kq.y, 0, sk_); ko.w = s8x2_to_bf16x2(kq.y, 2, sk_);
    vo.x = s8x2_to_bf16x2(vq.x, 0, sv_); vo.y = s8x2_to_bf16x2(vq.x, 2, sv_); vo.z = s8x2_to_bf16x2(vq.y, 0, sv_); vo.w = s8x2_to_bf16x2(vq.y, 2, sv_);
    *reinterpret_cast<uint4*>(dk + (dst + r) * hd + c) = ko;
    *reinterpret_cast<uint4*>(dv + (dst + r) * hd + c) = vo;
  }
}

template <int HD, int PPW>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_partial_kernel(const AttnParams p) {
  pdl_prologue();
  constexpr int PAIRS = ATT_WARPS * PPW;
  constexpr int KSTR = HD + 2;   // padded K row (elements): conflict-free one-key-per-lane reads
  extern __shared__ uint8_t smem_raw[];
  float* sq = reinterpret_cast<float*>(smem_raw);                                  // [PAIRS][HD]
  __nv_bfloat16* sk = reinterpret_cast<__nv_bfloat16*>(sq + PAIRS * HD);           // [64][KSTR]
  __nv_bfloat16* sv = sk + ATT_TILE * KSTR;                                        // [64][HD]

  const int b = blockIdx.x / p.max_q_tiles, qt = blockIdx.x % p.max_q_tiles;
  const int kvh = blockIdx.y, split = blockIdx.z;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int t0 = qt * p.q_tile;
  if (t0 >= q_len) return;
  const int nt = min(p.q_tile, q_len - t0);
  const int seq_len = p.seq_lens[b];
  const int pos0 = seq_len - q_len + t0;          // absolute position of the tile's first query
  const int gqa = p.n_q / p.n_kv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // kv range needed by this query tile, in whole 64-key tiles, then this split's share
  const int kv_hi = min(seq_len, pos0 + nt);
  const int kv_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int tile_lo = kv_lo / ATT_TILE, tile_hi = (kv_hi + ATT_TILE - 1) / ATT_TILE;
  const int n_tiles = tile_hi - tile_lo;
  const int per = (n_tiles + p.n_splits - 1) / p.n_splits;
  const int my_lo = tile_lo + split * per, my_hi = min(tile_hi, my_lo + per);
  // splits that own at least one key tile (n_tiles >= 1: a query always sees its own position's tile)
  const int eff = p.tickets ? (n_tiles + per - 1) / per : p.n_splits;
  if (split >= eff) return;

  const int total_pairs = nt * gqa;
  for (int round0 = 0; round0 < total_pairs; round0 += PAIRS) {
    __syncthreads();
    // stage the queries of this round as fp32, pre-scaled
    for (int i = threadIdx.x; i < PAIRS * HD; i += blockDim.x) {
      const int pr = round0 + i / HD, d = i % HD;
      float v = 0.f;
      if (pr < total_pairs) {
        const int tq = pr / gqa, hq = kvh * gqa + pr % gqa;
        v = __bfloat162float(p.q[((size_t)(q_begin + t0 + tq) * p.n_q + hq) * HD + d]) * p.scale;
      }
      sq[i] = v;
    }
    float m[PPW], l[PPW], acc[PPW][HD / 32];
#pragma unroll
    for (int i = 0; i < PPW; ++i) {
      m[i] = -1e30f; l[i] = 0.f;
#pragma unroll
      for (int j = 0; j < HD / 32; ++j) acc[i][j] = 0.f;
    }
    for (int tile = my_lo; tile < my_hi; ++tile) {
      __syncthreads();
      const int key0 = tile * ATT_TILE;
      const int blk = p.block_table[(size_t)b * p.max_blocks + key0 / p.block_size];
      const size_t base = (((size_t)blk * p.n_kv + kvh) * p.block_size + key0 % p.block_size) * HD;
      if (p.k_scale) {
        const int8_t* k8 = reinterpret_cast<const int8_t*>(p.k_cache);
        const int8_t* v8 = reinterpret_cast<const int8_t*>(p.v_cache);
        const size_t srow = ((size_t)blk * p.n_kv + kvh) * p.block_size + key0 % p.block_size;
        for (int i = threadIdx.x; i < ATT_TILE * HD / 8; i += blockDim.x) {
          const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
          const uint2 kq = *reinterpret_cast<const uint2*>(k8 + base + (size_t)r * HD + c);
          const uint2 vq = *reinterpret_cast<const uint2*>(v8 + base + (size_t)r * HD + c);
          const float ks = p.k_scale[srow + r], vs = p.v_scale[srow + r];
          uint32_t* kd = reinterpret_cast<uint32_t*>(sk + r * KSTR + c);
          kd[0] = s8x2_to_bf16x2(kq.x, 0, ks); kd[1] = s8x2_to_bf16x2(kq.x, 2, ks);
          kd[2] = s8x2_to_bf16x2(kq.y, 0, ks); kd[3] = s8x2_to_bf16x2(kq.y, 2, ks);
          uint4 vv;
          vv.x = s8x2_to_bf16x2(vq.x, 0, vs); vv.y = s8x2_to_bf16x2(vq.x, 2, vs);
          vv.z = s8x2_to_bf16x2(vq.y, 0, vs); vv.w = s8x2_to_bf16x2(vq.y, 2, vs);
          *reinterpret_cast<uint4*>(sv + r * HD + c) = vv;
        }
      } else {
        for (int i = threadIdx.x; i < ATT_TILE * HD / 8; i += blockDim.x) {
          const int r = i / (HD / 8), c = (i % (HD / 8)) * 8;
          const uint4 kv4 = *reinterpret_cast<const uint4*>(p.k_cache + base + (size_t)r * HD + c);
          uint32_t* kd = reinterpret_cast<uint32_t*>(sk + r * KSTR + c);
          kd[0] = kv4.x; kd[1] = kv4.y; kd[2] = kv4.z; kd[3] = kv4.w;
          *reinterpret_cast<uint4*>(sv + r * HD + c) = *reinterpret_cast<const uint4*>(p.v_cache + base + (size_t)r * HD + c);
        }
      }
      __syncthreads();
      // Scores of the warp's PPW pairs against the tile's 64 keys (a lane owns keys lane and lane + 32).  One pass over the key
      // row serves all pairs: a key element is read from shared memory once and multiplied into PPW dot products.
      if (round0 + warp * PPW >= total_pairs) continue;          // this warp has no live pair (barriers sit at the loop top)
      float p0[PPW], p1[PPW];
      {
        float sc[PPW][2];
        {
          // both keys of the lane in one pass: a query element read from shared memory feeds two dot products
          const uint32_t* kr0 = reinterpret_cast<const uint32_t*>(sk + lane * KSTR);
          const uint32_t* kr1 = reinterpret_cast<const uint32_t*>(sk + (lane + 32) * KSTR);
          const float* qv = sq + warp * PPW * HD;
          float d0[PPW], d1[PPW];
#pragma unroll
          for (int pi = 0; pi < PPW; ++pi) d0[pi] = d1[pi] = 0.f;
#pragma unroll 8
          for (int c = 0; c < HD / 2; ++c) {
            const uint32_t ka = kr0[c], kb = kr1[c];
            const float a0 = bf16_lo(ka), a1 = bf16_hi(ka), b0 = bf16_lo(kb), b1 = bf16_hi(kb);
#pragma unroll
            for (int pi = 0; pi < PPW; ++pi) {
              const float2 qq = *reinterpret_cast<const float2*>(qv + pi * HD + 2 * c);
              d0[pi] = fmaf(qq.x, a0, d0[pi]); d0[pi] = fmaf(qq.y, a1, d0[pi]);
              d1[pi] = fmaf(qq.x, b0, d1[pi]); d1[pi] = fmaf(qq.y, b1, d1[pi]);
            }
          }
#pragma unroll
          for (int pi = 0; pi < PPW; ++pi) {
            const int pr = round0 + warp * PPW + pi;
            const int qpos = pos0 + pr / gqa;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int kpos = key0 + lane + 32 * half;
              float dd = half ? d1[pi] : d0[pi];
              if (p.softcap > 0.f) dd = p.softcap * tanhf(dd / p.softcap);
              const bool ok = pr < total_pairs && kpos < seq_len && kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
              sc[pi][half] = ok ? dd : -INFINITY;
            }
          }
        }
#pragma unroll
        for (int pi = 0; pi < PPW; ++pi) {
          const float tmax = warp_max(fmaxf(sc[pi][0], sc[pi][1]));
          const float m_new = fmaxf(m[pi], tmax);
          const float corr = __expf(m[pi] - m_new);
          p0[pi] = __expf(sc[pi][0] - m_new);
          p1[pi] = __expf(sc[pi][1] - m_new);
          l[pi] = l[pi] * corr + warp_sum(p0[pi] + p1[pi]);
          m[pi] = m_new;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) acc[pi][c] *= corr;
        }
      }
      // P V: a value element is read once per key and feeds all PPW pairs
#pragma unroll 2
      for (int j = 0; j < ATT_TILE; ++j) {
        const __nv_bfloat16* vr = sv + j * HD;
        float vv[HD / 32];
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) vv[c] = __bfloat162float(vr[lane + 32 * c]);
#pragma unroll
        for (int pi = 0; pi < PPW; ++pi) {
          const float pj = __shfl_sync(0xffffffffu, j < 32 ? p0[pi] : p1[pi], j & 31);
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) acc[pi][c] = fmaf(pj, vv[c], acc[pi][c]);
        }
      }
    }
    // write partials
#pragma unroll
    for (int pi = 0; pi < PPW; ++pi) {
      const int pr = round0 + warp * PPW + pi;
      if (pr >= total_pairs) continue;
      const int tq = pr / gqa, hq = kvh * gqa + pr % gqa;
      const size_t row = ((size_t)split * p.Tq + (q_begin + t0 + tq)) * p.n_q + hq;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) p.o_part[row * HD + lane + 32 * c] = acc[pi][c];
      if (lane == 0) { p.ml_part[row * 2] = m[pi]; p.ml_part[row * 2 + 1] = l[pi]; }
    }
  }
  if (!p.tickets) return;
  // ---- the group's last CTA merges the splits
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* tk = p.tickets + (size_t)blockIdx.x * p.n_kv + kvh;
    const int prev = atomicAdd(tk, 1);
    s_last = prev == eff - 1;
    if (s_last) *tk = 0;                 // every counted split has arrived: the counter is ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const size_t sstride = (size_t)p.Tq * p.n_q;
  for (int pr = warp; pr < total_pairs; pr += ATT_WARPS) {
    const int tq = pr / gqa, hq = kvh * gqa + pr % gqa;
    const size_t r = (size_t)(q_begin + t0 + tq) * p.n_q + hq;
    float M = p.sinks ? p.sinks[hq] : -1e30f;
    for (int s = lane; s < eff; s += 32) M = fmaxf(M, __ldcg(p.ml_part + (s * sstride + r) * 2));
    M = warp_max(M);
    float L = 0.f;
    for (int s = lane; s < eff; s += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.ml_part + (s * sstride + r) * 2));
      L += ml.y * __expf(ml.x - M);
    }
    L = warp_sum(L) + (p.sinks ? __expf(p.sinks[hq] - M) : 0.f);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float acc[HD / 32];
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) acc[c] = 0.f;
    for (int s0 = 0; s0 < eff; s0 += 32) {
      const float sc_l = s0 + lane < eff ? __expf(__ldcg(p.ml_part + ((s0 + lane) * sstride + r) * 2) - M) : 0.f;
      const int cnt = min(32, eff - s0);
#pragma unroll 4
      for (int j = 0; j < cnt; ++j) {
        const float sc = __shfl_sync(0xffffffffu, sc_l, j);
        const float* op = p.o_part + ((s0 + j) * sstride + r) * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) acc[c] = fmaf(__ldcg(op + lane + 32 * c), sc, acc[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) p.out[r * HD + lane + 32 * c] = __float2bfloat16(acc[c] * inv);
  }
}

// out[t][h][:] = sum_s acc_s e^{m_s - M} / (sum_s l_s e^{m_s - M} + e^{sink_h - M})
__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                                           const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out, int Tq, int n_q,
                                                           int hd, int n_splits) {
  pdl_prologue();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= Tq * n_q) return;
  const int h = r % n_q;
  float M = sinks ? sinks[h] : -1e30f;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml_part[((size_t)s * Tq * n_q + r) * 2]);
  float L = sinks ? __expf(sinks[h] - M) : 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float* ml = ml_part + ((size_t)s * Tq * n_q + r) * 2;
    L += ml[1] * __expf(ml[0] - M);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = lane; d < hd; d += 32) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const size_t row = (size_t)s * Tq * n_q + r;
      a += o_part[row * hd + d] * __expf(ml_part[row * 2] - M);
    }
    out[(size_t)r * hd + d] = __float2bfloat16(a * inv);
  }
}

// Tickets of the fused merge: zero at load, and every launch leaves its counters at zero again.  Consecutive launches rotate
// through the slots, so that two launches that overlap (programmatic dependent launch lets the next kernel's CTAs start while
// this one drains) never count on the same words.
constexpr int ATT_TICKET_SLOTS = 8, ATT_TICKETS_PER_SLOT = 2048;
static __device__ int g_attn_tickets[ATT_TICKET_SLOTS * ATT_TICKETS_PER_SLOT];

template <int HD, int PPW>
static int launch_partial(const AttnParams& p, cudaStream_t st) {
  constexpr int PAIRS = ATT_WARPS * PPW;
  const size_t smem = (size_t)PAIRS * HD * 4 + (size_t)ATT_TILE * (HD + 2) * 2 + (size_t)ATT_TILE * HD * 2;
  auto kern = attn_partial_kernel<HD, PPW>;
  static DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured.mark();
  }
  dim3 grid(p.B * p.max_q_tiles, p.n_kv, p.n_splits);
  launch_pdl(kern, dim3(grid), dim3(ATT_WARPS * 32), smem, st, p);
  return (int)cudaGetLastError();
}

}  // namespace mx

using namespace mx;

// pairs per warp (1 for decode-sized work, 4 when there are many query tokens), query tokens per CTA, query tiles per sequence
static void att_tiling(int max_q_len, int gqa, int& ppw, int& q_tile, int& max_q_tiles) {
  ppw = (max_q_len * gqa > ATT_WARPS * 2) ? 4 : (max_q_len * gqa > ATT_WARPS ? 2 : 1);
  const int pairs = ATT_WARPS * ppw;
  q_tile = pairs / gqa > 0 ? pairs / gqa : 1;
  if (q_tile > max_q_len) q_tile = max_q_len;
  max_q_tiles = (max_q_len + q_tile - 1) / q_tile;
}

// Kernels one attention call launches: 1 when the split merge runs inside the partial kernel, 2 with the separate combine.
MX_HOST_API int mx_attention_launches(int B, int max_q_len, int n_q, int n_kv) {
  int ppw, q_tile, max_q_tiles;
  att_tiling(max_q_len, n_q / (n_kv > 0 ? n_kv : 1), ppw, q_tile, max_q_tiles);
  return (long long)B * max_q_tiles * n_kv <= ATT_TICKETS_PER_SLOT ? 1 : 2;
}

// Scratch: o_part needs n_splits*Tq*n_q*hd floats, ml_part n_splits*Tq*n_q*2 floats.
// max_q_len is the longest query segment of the batch (host knows it from cu_q).
static int attention_impl(const void* q, const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                          const int* block_table, const int* seq_lens, const int* cu_q, const float* sinks, void* out, float* o_part,
                          float* ml_part, int B, int Tq, int max_q_len, int n_q, int n_kv, int hd, int max_blocks, int block_size, int window,
                          float scale, float softcap, int n_splits, cudaStream_t st) {
  if (B <= 0 || Tq <= 0) return 0;
  if (block_size % ATT_TILE) return -110;
  if (n_q % n_kv) return -111;
  const int gqa = n_q / n_kv;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.k_scale = k_scale; p.v_scale = k_scale ? v_scale : nullptr;
  p.block_table = block_table; p.seq_lens = seq_lens; p.cu_q = cu_q; p.o_part = o_part; p.ml_part = ml_part;
  p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.max_blocks = max_blocks; p.block_size = block_size;
  p.n_splits = n_splits < 1 ? 1 : n_splits; p.Tq = Tq; p.window = window; p.scale = scale; p.softcap = softcap;
  int ppw;
  att_tiling(max_q_len, gqa, ppw, p.q_tile, p.max_q_tiles);
  p.tickets = nullptr; p.sinks = sinks; p.out = (__nv_bfloat16*)out;
  const long long groups = (long long)B * p.max_q_tiles * n_kv;
  if (groups <= ATT_TICKETS_PER_SLOT) {
    static int* base[64] = {nullptr};
    static unsigned turn[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!base[dev]) {
      void* a = nullptr;
      if (cudaGetSymbolAddress(&a, g_attn_tickets) != cudaSuccess) return -115;
      base[dev] = (int*)a;
    }
    p.tickets = base[dev] + (size_t)(turn[dev]++ % ATT_TICKET_SLOTS) * ATT_TICKETS_PER_SLOT;
  }
  int rc;
#define MX_ATT(HD_)                                                        \
  (ppw == 4 ? launch_partial<HD_, 4>(p, st) : ppw == 2 ? launch_partial<HD_, 2>(p, st) : launch_partial<HD_, 1>(p, st))
  switch (hd) {
    case 64: rc = MX_ATT(64); break;
    case 128: rc = MX_ATT(128); break;
    case 256: rc = MX_ATT(256); break;
    case 512: rc = MX_ATT(512); break;      // Gemma-4 global layers
    default: return -112;
  }
#undef MX_ATT
  if (rc || p.tickets) return rc;
  launch_pdl(attn_combine_kernel, dim3((Tq * n_q + 3) / 4), dim3(128), 0, st, o_part, ml_part, sinks, (__nv_bfloat16*)out, Tq, n_q, hd, p.n_splits);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens,
                             const int* cu_q, const float* sinks, void* out, float* o_part, float* ml_part, int B, int Tq, int max_q_len,
                             int n_q, int n_kv, int hd, int max_blocks, int block_size, int window, float scale, float softcap,
                             int n_splits, cudaStream_t st) {
  return attention_impl(q, k_cache, v_cache, nullptr, nullptr, block_table, seq_lens, cu_q, sinks, out, o_part, ml_part, B, Tq, max_q_len, n_q,
                        n_kv, hd, max_blocks, block_size, window, scale, softcap, n_splits, st);
}

// The same over an int8 cache with per-row scales (see the layout note at the top of this file).
MX_HOST_API int mx_attention_kv8(const void* q, const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                                 const int* block_table, const int* seq_lens, const int* cu_q, const float* sinks, void* out, float* o_part,
                                 float* ml_part, int B, int Tq, int max_q_len, int n_q, int n_kv, int hd, int max_blocks, int block_size,
                                 int window, float scale, float softcap, int n_splits, cudaStream_t st) {
  if (!k_scale || !v_scale) return -113;
  return attention_impl(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, cu_q, sinks, out, o_part, ml_part, B, Tq, max_q_len, n_q,
                        n_kv, hd, max_blocks, block_size, window, scale, softcap, n_splits, st);
}

// dst_k / dst_v: bf16 [B * nb][n_kv][block_size][hd]; page (b, j) is filled when j * block_size < seq_lens[b].
MX_HOST_API int mx_kv_dequant_pages(const void* k8, const void* v8, const float* k_scale, const float* v_scale, const int* block_table,
                                    const int* seq_lens, void* dst_k, void* dst_v, int B, int n_kv, int block_size, int hd, int max_blocks,
                                    int nb, cudaStream_t st) {
  if (B <= 0 || nb <= 0) return 0;
  if (hd % 8) return -114;
  launch_pdl(kv_dequant_pages_kernel, dim3(nb, B, n_kv), dim3(256), 0, st, (const int8_t*)k8, (const int8_t*)v8, k_scale, v_scale, block_table,
             seq_lens, (__nv_bfloat16*)dst_k, (__nv_bfloat16*)dst_v, n_kv, block_size, hd, max_blocks, nb);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (see mx_noalloc.h): the split-KV partials live in this fixed device array.
// In host code the array's name is only a handle for cudaGetSymbolAddress; the kernels are given the
// device address that call returns.
static __device__ __align__(256) float g_noalloc_scratch[MX_NOALLOC_SCRATCH_FLOATS];

namespace {
float* g_noalloc_ptr[64] = {nullptr};        // per device, resolved on first use
thread_local char g_noalloc_err[256] = "";
}  // namespace

MX_HOST_API const char* mx_attention_noalloc_error(void) { return g_noalloc_err; }

MX_HOST_API int mx_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens,
                                     const int* cu_q, const float* sinks, void* out, int B, int Tq, int max_q_len, int n_q, int n_kv, int hd,
                                     int max_blocks, int block_size, int window, float scale, float softcap, int n_splits,
                                     cudaStream_t stream) {
  g_noalloc_err[0] = 0;
  if (B <= 0 || Tq <= 0) return 0;
  const int splits = n_splits < 1 ? 1 : n_splits;
  const unsigned long long need = (unsigned long long)splits * Tq * n_q * (unsigned long long)(hd + 2);
  if (need > MX_NOALLOC_SCRATCH_FLOATS) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err,
             "mx_attention_noalloc: needs %llu scratch floats (n_splits %d x Tq %d x n_q %d x (head_dim %d + 2)) but the built-in scratch holds %u; "
             "use fewer splits / tokens or call mx_attention with caller-provided scratch",
             need, splits, Tq, n_q, hd, (unsigned)MX_NOALLOC_SCRATCH_FLOATS);
    return MX_NOALLOC_E_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err, "mx_attention_noalloc: cannot identify the current device (%s)", cudaGetErrorString(e));
    return MX_NOALLOC_E_SYMBOL;
  }
  if (!g_noalloc_ptr[dev]) {
    // once per device, with that device current: turn the symbol into a device address
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      snprintf(g_noalloc_err, sizeof g_noalloc_err, "mx_attention_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
      return MX_NOALLOC_E_SYMBOL;
    }
    g_noalloc_ptr[dev] = ptr;
  }
  float* o_part = g_noalloc_ptr[dev];
  float* ml_part = o_part + (size_t)splits * Tq * n_q * hd;
  return mx_attention(q, k_cache, v_cache, block_table, seq_lens, cu_q, sinks, out, o_part, ml_part, B, Tq, max_q_len, n_q, n_kv, hd, max_blocks,
                      block_size, window, scale, softcap, splits, stream);
}
