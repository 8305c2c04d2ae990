// Router top-k for one token, executed by one warp: weights = softmax over the selected logits (renorm) or softmax over all.
// Lane k < K ends up holding the k-th selection; E <= 1024, K <= 32.  The logits are read past L1: the caller may be the last CTA
// of the kernel that produced them.
#pragma once
#include "common.cuh"

namespace mx {

__device__ __forceinline__ void route_token_warp(const float* __restrict__ logits, const float* __restrict__ bias, int t, int E, int K, int renorm,
                                                 int* __restrict__ topk_idx, float* __restrict__ topk_w, int w_copies = 1) {
  const int lane = threadIdx.x & 31;
  float v[32];
  const int per = (E + 31) / 32;
  float mx_all = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int e = lane + 32 * i;
    v[i] = (i < per && e < E) ? __ldcg(logits + (size_t)t * E + e) + (bias ? bias[e] : 0.f) : -INFINITY;
    mx_all = fmaxf(mx_all, v[i]);
  }
  mx_all = warp_max(mx_all);
  float denom_all = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) if (i < per) denom_all += __expf(v[i] - mx_all);
  denom_all = warp_sum(denom_all);
  float sel_sum = 0.f;
  float my_w = 0.f; int my_e = 0;    // lane k keeps the k-th selection (K <= 32)
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int e = lane + 32 * i;
      if (i < per && (v[i] > best || (v[i] == best && e < bi))) { best = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    const float pw = __expf(best - mx_all);
    sel_sum += pw;
    if (lane == k) { my_w = pw; my_e = bi; }
#pragma unroll
    for (int i = 0; i < 32; ++i) if (lane + 32 * i == bi) v[i] = -INFINITY;
  }
  if (lane < K) {
    topk_idx[(size_t)t * K + lane] = my_e;
    // w_copies > 1: the weight row is [w_copies][K] (a consumer that sums several partial rows per pair reads one weight per partial)
    const float wv = my_w / (renorm ? sel_sum : denom_all);
    for (int c = 0; c < w_copies; ++c) topk_w[((size_t)t * w_copies + c) * K + lane] = wv;
  }
}

}  // namespace mx
