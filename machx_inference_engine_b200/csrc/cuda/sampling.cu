// Batched token sampling: one CTA per request row.
//   argmax            : greedy pick, ties -> lowest id
//   rep_penalty       : in-place penalty on the logits of previously seen ids (unique id list)
//   sample            : temperature, top-k, top-p, min-p in that order, over at most CAP (256)
//                       winners extracted in logit space in descending order (ties -> lowest id),
//                       then one xorshift64* draw walks the winners in descending-probability order
// Reference parity: src/ops/sampling.cpp:37-240 (argmax, rep_penalty, topk_topp with K_CAP
// semantics, tie rule and draw order); batching over requests is new.
#include "common.cuh"
#include "host_util.h"

namespace mx {

constexpr int SAMP_THREADS = 1024;
constexpr int SAMP_CAP = 256;

struct ValIdx { float v; int i; };
__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

__device__ __forceinline__ ValIdx block_argmax(ValIdx x, ValIdx* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ValIdx y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sh[warp] = x;
  __syncthreads();
  if (warp == 0) {
    ValIdx y = lane < (blockDim.x >> 5) ? sh[lane] : ValIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ValIdx z;
      z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
      z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
      y = better(y, z);
    }
    if (lane == 0) sh[0] = y;
  }
  __syncthreads();
  return sh[0];
}

// A row of NaN logits never beats the initial {-inf, 0x7fffffff}: the id that leaves the sampler is always a row index (0 then),
// so that nothing downstream (token history, detokeniser, callbacks) sees an out-of-range id.
__device__ __forceinline__ int valid_id(int i, int V) { return (i < 0 || i >= V) ? 0 : i; }

__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* __restrict__ logits, int V, int ld, int* __restrict__ out) {
  pdl_prologue();
  __shared__ ValIdx sh[32];
  const float* row = logits + (size_t)blockIdx.x * ld;
  ValIdx best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) best = better(best, ValIdx{row[i], i});
  best = block_argmax(best, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = valid_id(best.i, V);
}

// Wide vocabularies: ARGMAX_CHUNKS CTAs per row reduce a slice each into a device scratch slot, and the last CTA of a
// row to finish (ticket counter) reduces the partials.  `better` is a total order, so the result does not depend on
// which CTA comes last.  The scratch is shared by all launches: callers issue argmax on one stream at a time.
constexpr int ARGMAX_CHUNKS = 32;
constexpr int ARGMAX_MAX_ROWS = 1024;
__device__ ValIdx g_argmax_part[ARGMAX_MAX_ROWS * ARGMAX_CHUNKS];
__device__ unsigned g_argmax_ticket[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(SAMP_THREADS) argmax_split_kernel(const float* __restrict__ logits, int V, int ld, int* __restrict__ out) {
  pdl_prologue();
  __shared__ ValIdx sh[32];
  __shared__ bool last;
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS, lo = c * per, hi = min(V, lo + per);
  ValIdx best{-INFINITY, 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) best = better(best, ValIdx{row[i], i});
  best = block_argmax(best, sh);
  if (threadIdx.x == 0) {
    g_argmax_part[r * ARGMAX_CHUNKS + c] = best;
    __threadfence();
    last = atomicAdd(&g_argmax_ticket[r], 1u) == ARGMAX_CHUNKS - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {
    __threadfence();
    ValIdx y = threadIdx.x < ARGMAX_CHUNKS ? g_argmax_part[r * ARGMAX_CHUNKS + threadIdx.x] : ValIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ValIdx z;
      z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
      z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
      y = better(y, z);
    }
    if (threadIdx.x == 0) { out[r] = valid_id(y.i, V); g_argmax_ticket[r] = 0; }
  }
}

// ids: [rows][max_ids] padded with -1; each id must appear at most once per row.
__global__ void rep_penalty_kernel(float* __restrict__ logits, int V, int ld, const int* __restrict__ ids, int max_ids, const float* __restrict__ penalty) {
  pdl_prologue();
  const int r = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_ids) return;
  const float pen = penalty[r];
  if (pen == 1.f) return;
  const int id = ids[(size_t)r * max_ids + i];
  if (id < 0 || id >= V) return;
  float* p = logits + (size_t)r * ld + id;
  const float v = *p;
  *p = v > 0.f ? v / pen : v * pen;
}

struct SampleParams {
  const float* logits; int V, ld;
  const float* temperature;   // [rows] (<=0 -> greedy)
  const int* top_k;           // [rows] (<=0 -> CAP)
  const float* top_p;         // [rows]
  const float* min_p;         // [rows]
  unsigned long long* rng;    // [rows] xorshift state, updated
  int* out;
};

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(const SampleParams p) {
  pdl_prologue();
  __shared__ ValIdx sh[32];
  __shared__ float win_v[SAMP_CAP];
  __shared__ int win_i[SAMP_CAP];
  __shared__ int s_pick;
  const int r = blockIdx.x;
  const float* row = p.logits + (size_t)r * p.ld;
  const float temp = p.temperature[r];
  int k = p.top_k[r];
  if (k <= 0 || k > SAMP_CAP) k = SAMP_CAP;
  if (k > p.V) k = p.V;
  if (temp <= 0.f) k = 1;
  // thread-local best over a strided subset; "taken" entries are tracked by value/index ordering:
  // after a winner (v*, i*) is extracted the owner rescans for the best entry strictly after it.
  ValIdx last{INFINITY, -1};
  ValIdx local{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < p.V; i += blockDim.x) local = better(local, ValIdx{row[i], i});
  for (int n = 0; n < k; ++n) {
    const ValIdx w = block_argmax(local, sh);
    if (threadIdx.x == 0) { win_v[n] = w.v; win_i[n] = w.i; }
    if (w.i >= 0 && w.i < p.V && (w.i % blockDim.x) == threadIdx.x) {
      last = w;
      local = ValIdx{-INFINITY, 0x7fffffff};
      for (int i = threadIdx.x; i < p.V; i += blockDim.x) {
        const ValIdx c{row[i], i};
        // strictly after `last` in (value desc, index asc) order
        if (c.v < last.v || (c.v == last.v && c.i > last.i)) local = better(local, c);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pick = win_i[0];
    if (temp > 0.f && k > 1) {
      const float inv_t = 1.f / temp, vmax = win_v[0];
      float sum = 0.f;
      for (int n = 0; n < k; ++n) { win_v[n] = __expf((win_v[n] - vmax) * inv_t); sum += win_v[n]; }
      // top-p: smallest prefix whose mass reaches top_p;  min-p: keep p_i >= min_p * p_max (p_max = win_v[0]/sum)
      const float tp = p.top_p[r], mp = p.min_p[r];
      int keep = k;
      if (tp > 0.f && tp < 1.f) {
        float c = 0.f;
        for (int n = 0; n < k; ++n) { c += win_v[n] / sum; if (c >= tp) { keep = n + 1; break; } }
      }
      if (mp > 0.f) {
        int n = 1;
        while (n < keep && win_v[n] >= mp * win_v[0]) ++n;
        keep = n;
      }
      float ksum = 0.f;
      for (int n = 0; n < keep; ++n) ksum += win_v[n];
      unsigned long long s = p.rng[r];
      s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
      p.rng[r] = s;
      const unsigned long long z = s * 2685821657736338717ull;
      const float u = (float)(z >> 40) * (1.f / 16777216.f) * ksum;
      float c = 0.f;
      pick = win_i[keep - 1];
      for (int n = 0; n < keep; ++n) { c += win_v[n]; if (u < c) { pick = win_i[n]; break; } }
    }
    s_pick = pick;
    p.out[r] = valid_id(s_pick, p.V);
  }
}

}  // namespace mx

using namespace mx;

MX_HOST_API int mx_argmax(const float* logits, int rows, int V, int ld, int* out, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V >= 32768 && rows <= ARGMAX_MAX_ROWS) launch_pdl(argmax_split_kernel, dim3(dim3(ARGMAX_CHUNKS, rows)), dim3(256), 0, st, logits, V, ld, out);
  else launch_pdl(argmax_kernel, dim3(rows), dim3(SAMP_THREADS), 0, st, logits, V, ld, out);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_rep_penalty(float* logits, int rows, int V, int ld, const int* ids, int max_ids, const float* penalty, cudaStream_t st) {
  if (rows <= 0 || max_ids <= 0) return 0;
  dim3 grid((max_ids + 255) / 256, rows);
  launch_pdl(rep_penalty_kernel, dim3(grid), dim3(256), 0, st, logits, V, ld, ids, max_ids, penalty);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_sample(const float* logits, int rows, int V, int ld, const float* temperature, const int* top_k, const float* top_p,
                          const float* min_p, unsigned long long* rng, int* out, cudaStream_t st) {
  if (rows <= 0) return 0;
  SampleParams p{logits, V, ld, temperature, top_k, top_p, min_p, rng, out};
  launch_pdl(sample_kernel, dim3(rows), dim3(SAMP_THREADS), 0, st, p);
  return (int)cudaGetLastError();
}
