// Mixture-of-experts routing and token packing, entirely on the device (no host round trip):
//   route    : top-k over router logits, weights = softmax over the selected logits (equal to
//              softmax-over-all followed by top-k renormalisation) or plain softmax-over-all
//   pack     : stable counting sort of (token, slot) pairs by expert, expert segments padded to
//              128-row tiles; emits per-tile expert ids and the live tile count for the grouped GEMM
//   gather   : activation rows -> expert-sorted packed rows (bf16), pad rows zeroed
//   combine  : y[t] (+)= sum_k w[t,k] * packed_out[pos(t,k)]  (fixed order: deterministic)
// Reference parity: src/ops/moe.cpp:30-80,268-291,371-429, host router src/model/gptoss.cpp:23-47,
// host packer src/model/qwen3moe_pack.cpp:5-31, reduce src/ops/moe_fused.cpp:1937-1961.
#include "common.cuh"
#include "comm.cuh"
#include "host_util.h"
#include "moe_route.cuh"

namespace mx {

constexpr int MOE_TILE = 128;

// one warp per token; E <= 1024
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int K,
                                                        int renorm, int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  pdl_prologue();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  route_token_warp(logits, bias, t, E, K, renorm, topk_idx, topk_w);
}

// Single-CTA packer.  n = T*K pairs.  Outputs:
//   counts[E], seg_start[E+1] (padded starts, multiples of 128), packed_token[P] (-1 = pad),
//   pair_to_packed[n], tile_expert[max_tiles], tile_valid[max_tiles] (optional: live rows per tile), num_tiles[1], packed_rows[1]
// e_lo/e_hi restrict packing to the experts owned by this rank (expert parallelism): pairs routed
// elsewhere get pair_to_packed = -1.
// Stable counting sort in three passes: every warp owns a contiguous chunk of the pair list and histograms it
// (hist[warp][expert] in shared memory), a scan over the warps turns the histograms into per-warp write cursors,
// and each warp walks its chunk again placing 32 pairs per step (rank among equal experts by __match_any_sync).
// Rows of an expert therefore keep increasing pair order and the result does not depend on timing.
// The kernel is a chain of short phases, so every phase is written for latency: a warp fetches its pairs eight steps at a time
// (independent loads), the expert offsets come from a block-wide prefix sum (expert e = thread e), and every expert writes its own
// tile table entries.
constexpr int PACK_BATCH = 8;

__global__ void __launch_bounds__(1024) moe_pack_kernel(const int* __restrict__ topk_idx, int n, int K, int E, int e_lo, int e_hi,
                                                        int* __restrict__ counts, int* __restrict__ seg_start, int* __restrict__ packed_token,
                                                        int* __restrict__ pair_to_packed, int* __restrict__ tile_expert, int* __restrict__ num_tiles,
                                                        int max_rows, int tile, int* __restrict__ tile_valid) {
  pdl_prologue();
  extern __shared__ int s_hist[];            // [nwarps][E]
  __shared__ int s_cnt[1024];
  __shared__ int s_start[1025];
  __shared__ int s_wsum[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int chunk = ((n + nwarps - 1) / nwarps + 31) & ~31;
  const int c0 = warp * chunk, c1 = min(n, c0 + chunk);
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  for (int base = c0; base < c1; base += 32 * PACK_BATCH) {
    int ev[PACK_BATCH];
#pragma unroll
    for (int u = 0; u < PACK_BATCH; ++u) {
      const int i = base + 32 * u + lane;
      ev[u] = i < c1 ? topk_idx[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < PACK_BATCH; ++u)
      if (ev[u] >= e_lo && ev[u] < e_hi) atomicAdd(&s_hist[warp * E + ev[u]], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) {
      const int c = s_hist[w * E + e];
      s_hist[w * E + e] = run;
      run += c;
    }
    s_cnt[e] = run;
  }
  __syncthreads();
  {
    // exclusive prefix sum of the padded segment lengths over the experts (E <= 1024 = one expert per thread)
    // tile = 128: segments padded to whole GEMM tiles and a tile -> expert map; tile = 1: compact segments (GEMV path)
    const int e = threadIdx.x;
    const int cnt = e < E ? s_cnt[e] : 0;
    const int padded = (cnt + tile - 1) / tile * tile;
    int v = padded;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    if (lane == 31) s_wsum[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nwarps ? s_wsum[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += u;
      }
      s_wsum[lane] = w;                      // inclusive over warps
    }
    __syncthreads();
    const int start = v - padded + (warp ? s_wsum[warp - 1] : 0);
    if (e < E) {
      s_start[e] = start;
      seg_start[e] = start;
      counts[e] = cnt;
      if (tile > 1) {
        const int t0 = start / tile;         // every earlier segment is a whole number of tiles
        for (int tix = 0; tix < padded / tile; ++tix) {
          if (tile_valid) tile_valid[t0 + tix] = min(tile, cnt - tix * tile);      // live rows of this tile
          tile_expert[t0 + tix] = e;
        }
      }
    }
    if (threadIdx.x == blockDim.x - 1) {
      const int off = s_wsum[nwarps - 1];
      s_start[E] = off;
      seg_start[E] = off;
      num_tiles[0] = tile > 1 ? off / tile : 0;
      num_tiles[1] = off;
    }
  }
  __syncthreads();
  const int total = s_start[E];
  for (int i = threadIdx.x; i < max_rows; i += blockDim.x) if (i < total) packed_token[i] = -1;
  __syncthreads();
  for (int base0 = c0; base0 < c1; base0 += 32 * PACK_BATCH) {
    int ev[PACK_BATCH];
#pragma unroll
    for (int u = 0; u < PACK_BATCH; ++u) {
      const int i = base0 + 32 * u + lane;
      ev[u] = i < c1 ? topk_idx[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < PACK_BATCH; ++u) {
      const int base = base0 + 32 * u;
      if (base >= c1) break;                 // warp-uniform
      const int i = base + lane;
      const int e = ev[u];
      const bool owned = e >= e_lo && e < e_hi;
      const unsigned m = __match_any_sync(0xffffffffu, owned ? e : E + lane);
      int cur = 0;
      if (owned) cur = s_hist[warp * E + e];
      __syncwarp();
      if (owned) {
        const int dst = s_start[e] + cur + __popc(m & ((1u << lane) - 1));
        packed_token[dst] = i / K;
        pair_to_packed[i] = dst;
        if (lane == 31 - __clz(m)) s_hist[warp * E + e] = cur + __popc(m);      // the highest lane of the group advances the cursor
      } else if (i < c1) {
        pair_to_packed[i] = -1;
      }
      __syncwarp();
    }
  }
}

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  __half2 h = __floats2half2_rn(bf16_lo(v), bf16_hi(v));
  return *reinterpret_cast<uint32_t*>(&h);
}
// to_f16: convert the bf16 rows to fp16 while copying (MXFP4 expert GEMMs run in fp16 x fp16 mode)
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ packed_token, const int* __restrict__ total_rows,
                                  __nv_bfloat16* __restrict__ xp, int H, int to_f16, int zero_pad) {
  pdl_prologue();
  const int r = blockIdx.x;
  if (r >= total_rows[1]) return;
  const int t = packed_token[r];
  uint4* dst = reinterpret_cast<uint4*>(xp + (size_t)r * H);
  if (t < 0) {
    // tile padding: unless asked, the row is left as it is.  The grouped GEMM's output row depends on its own input row only and
    // nothing refers to padding rows afterwards, and at ten experts per token the padding is as many rows as the live ones.
    if (!zero_pad) return;
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
      uint4 v = src[i];
      if (to_f16) { v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y); v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w); }
      dst[i] = v;
    }
  }
}

// out[t][:] = (accumulate ? out : 0) + sum_k w[t,k] * yp[pair_to_packed[t,k]][:]
template <typename OT>
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ pair_to_packed, const float* __restrict__ w,
                                   OT* __restrict__ out, int H, int K, int accumulate) {
  pdl_prologue();
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int k = 0; k < K; ++k) {
      const int pos = pair_to_packed[(size_t)t * K + k];
      if (pos < 0) continue;
      const uint32_t v = *reinterpret_cast<const uint32_t*>(yp + (size_t)pos * H + i);
      const float ww = w[(size_t)t * K + k];
      a0 = fmaf(ww, bf16_lo(v), a0);
      a1 = fmaf(ww, bf16_hi(v), a1);
    }
    if constexpr (sizeof(OT) == 4) {
      float* o = (float*)out + (size_t)t * H + i;
      if (accumulate) { o[0] += a0; o[1] += a1; } else { o[0] = a0; o[1] = a1; }
    } else {
      *reinterpret_cast<uint32_t*>((__nv_bfloat16*)out + (size_t)t * H + i) = pack_bf16(a0, a1);
    }
  }
}

// Combine fused with the expert-parallel all-reduce: the weighted sum of this rank's expert outputs is stored straight into
// slot [my_rank] of every rank's inbox (bf16 or fp32), and the last CTA publishes the sequence number (see comm.cuh).
template <typename OT>
__global__ void moe_combine_push_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ pair_to_packed, const float* __restrict__ w,
                                        int H, int K, PeerOut po) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int next_seq = *po.seq + 1;
  const int d0 = peer_first(po, t), nd = peer_count(po);
  if ((H & 7) == 0) {
    // eight columns per thread: a warp's store instruction covers 512 (bf16) or 1024 (fp32) contiguous bytes of the peer's row
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int pos = pair_to_packed[(size_t)t * K + k];
        if (pos < 0) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(yp + (size_t)pos * H + i);
        const float ww = w[(size_t)t * K + k];
        a[0] = fmaf(ww, bf16_lo(v.x), a[0]); a[1] = fmaf(ww, bf16_hi(v.x), a[1]);
        a[2] = fmaf(ww, bf16_lo(v.y), a[2]); a[3] = fmaf(ww, bf16_hi(v.y), a[3]);
        a[4] = fmaf(ww, bf16_lo(v.z), a[4]); a[5] = fmaf(ww, bf16_hi(v.z), a[5]);
        a[6] = fmaf(ww, bf16_lo(v.w), a[6]); a[7] = fmaf(ww, bf16_hi(v.w), a[7]);
      }
      for (int d = d0; d < d0 + nd; ++d) {
        if constexpr (sizeof(OT) == 4) {
          float* o = reinterpret_cast<float*>(peer_slot(po, d, next_seq)) + (size_t)t * H + i;
          *reinterpret_cast<float4*>(o) = make_float4(a[0], a[1], a[2], a[3]);
          *reinterpret_cast<float4*>(o + 4) = make_float4(a[4], a[5], a[6], a[7]);
        } else {
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_slot(po, d, next_seq)) + (size_t)t * H + i) =
              make_uint4(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]), pack_bf16(a[4], a[5]), pack_bf16(a[6], a[7]));
        }
      }
    }
  } else {
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
      float a0 = 0.f, a1 = 0.f;
      for (int k = 0; k < K; ++k) {
        const int pos = pair_to_packed[(size_t)t * K + k];
        if (pos < 0) continue;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(yp + (size_t)pos * H + i);
        const float ww = w[(size_t)t * K + k];
        a0 = fmaf(ww, bf16_lo(v), a0);
        a1 = fmaf(ww, bf16_hi(v), a1);
      }
      for (int d = d0; d < d0 + nd; ++d) {
        if constexpr (sizeof(OT) == 4) *reinterpret_cast<float2*>(reinterpret_cast<float*>(peer_slot(po, d, next_seq)) + (size_t)t * H + i) = make_float2(a0, a1);
        else *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(peer_slot(po, d, next_seq)) + (size_t)t * H + i) = pack_bf16(a0, a1);
      }
    }
  }
  peer_publish(po, next_seq);
}

PeerOut make_peer_out(const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket);

}  // namespace mx

using namespace mx;

MX_HOST_API int mx_moe_combine_push(const void* yp, const int* pair_to_packed, const float* w, int out_f32, int T, int H, int K,
                                    const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket, int rs_rows,
                                    cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 2) return -101;
  if ((long long)T * H * (out_f32 ? 4 : 2) > slot_bytes) return -140;
  PeerOut po = make_peer_out(inbox, world, my_rank, slot_bytes, seq, ticket);
  po.rs_rows = rs_rows;
  if (out_f32) launch_pdl(moe_combine_push_kernel<float>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)yp, pair_to_packed, w, H, K, po);
  else launch_pdl(moe_combine_push_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)yp, pair_to_packed, w, H, K, po);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_route(const float* logits, const float* bias, int T, int E, int K, int renorm, int* topk_idx, float* topk_w,
                             cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 1024 || K > 32 || K > E) return -120;
  launch_pdl(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, st, logits, bias, T, E, K, renorm, topk_idx, topk_w);
  return (int)cudaGetLastError();
}

// num_tiles must hold 2 ints: [0] live 128-row tiles, [1] packed row count.
MX_HOST_API int mx_moe_pack(const int* topk_idx, int n_pairs, int K, int E, int e_lo, int e_hi, int* counts, int* seg_start,
                            int* packed_token, int* pair_to_packed, int* tile_expert, int* num_tiles, int max_rows, int tile, int* tile_valid,
                            cudaStream_t st) {
  if (E > 1024 || (tile != 1 && tile != MOE_TILE)) return -120;
  const int pack_smem = 32 * E * (int)sizeof(int);
  static DeviceOnce pack_attr;
  if (pack_attr.pending()) {
    cudaError_t e = cudaFuncSetAttribute(moe_pack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024 * (int)sizeof(int));
    if (e != cudaSuccess) return (int)e;
    pack_attr.mark();
  }
  launch_pdl(moe_pack_kernel, dim3(1), dim3(1024), pack_smem, st, topk_idx, n_pairs, K, E, e_lo, e_hi, counts, seg_start, packed_token, pair_to_packed, tile_expert,
                                      num_tiles, max_rows, tile, tile_valid);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_gather(const void* x, const int* packed_token, const int* num_tiles, void* xp, int H, int max_rows, int to_f16,
                              int zero_pad, cudaStream_t st) {
  if (max_rows <= 0) return 0;
  if (H % 8) return -101;
  launch_pdl(moe_gather_kernel, dim3(max_rows), dim3(128), 0, st, (const __nv_bfloat16*)x, packed_token, num_tiles, (__nv_bfloat16*)xp, H, to_f16,
             zero_pad);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_moe_combine(const void* yp, const int* pair_to_packed, const float* w, void* out, int out_f32, int T, int H, int K,
                               int accumulate, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 2) return -101;
  if (out_f32) launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)yp, pair_to_packed, w, (float*)out, H, K, accumulate);
  else launch_pdl(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)yp, pair_to_packed, w, (__nv_bfloat16*)out, H, K, accumulate);
  return (int)cudaGetLastError();
}
