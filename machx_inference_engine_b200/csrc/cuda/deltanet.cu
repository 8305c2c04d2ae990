// Gated-DeltaNet (linear attention) kernels for the hybrid families (Qwen3-Next, Qwen3.6):
//   conv1d_silu     : depthwise causal convolution with fused SiLU over batched variable-length sequences,
//                     per-sequence streaming state, optional per-position state checkpoints
//   deltanet_scan   : gated delta rule   S <- e^g S ; d = (v - S^T k) beta ; S <- S + k d^T ; o = S^T q
//                     with the q/k L2 normalisation, the g / beta activations and the k-head -> v-head mapping
//                     fused in; one CTA owns 32 of the 128 value columns of one (sequence, v-head) and keeps its
//                     slice of S in registers for the whole sequence (prefill, decode and verify use the same kernel)
//   gated_rmsnorm   : y = w * o / rms(o) * silu(z) per 128-wide head, z read in place from the projection output
// Reference parity: src/ops/conv1d.cpp:28-117, src/ops/deltanet.cpp:41-480 (sequential recurrence with one work-group
// per (batch, v-head) and one state column per lane).  Here the state is split by value columns so a 32-head layer
// fills 128 CTAs, the per-token reductions stay inside 8 lanes, and the state lives transposed ([v][k]) so that
// every thread loads and stores one contiguous 64-byte run.
#include "common.cuh"
#include "host_util.h"

namespace mx {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------ conv1d + SiLU
// x: [T, ld] bf16, conv input in columns [0, C) of the view; w: [C, Kc] fp32, tap j multiplies input t-(Kc-1)+j;
// state: [slots, Kc-1, C] bf16 = the Kc-1 inputs that precede the next token of the sequence in that slot.
__global__ void __launch_bounds__(128) conv1d_silu_kernel(const bf16* __restrict__ x, int ld, int C, int Kc, const float* __restrict__ w,
                                                          bf16* __restrict__ state, const int* __restrict__ slots,
                                                          const int* __restrict__ cu_q, int B, bf16* __restrict__ y,
                                                          bf16* __restrict__ ckpt, int fuse_state) {
  pdl_prologue();
  const int t = blockIdx.y;
  const int c = (blockIdx.x * 128 + threadIdx.x) * 2;
  if (c >= C) return;
  int b = 0;
  while (b + 1 < B && cu_q[b + 1] <= t) ++b;
  const int t_start = cu_q[b];
  const int slot = slots[b];
  float v0[8], v1[8];
  for (int j = 0; j < Kc; ++j) {
    const int src = t - (Kc - 1) + j;
    uint32_t raw;
    if (src >= t_start) raw = *reinterpret_cast<const uint32_t*>(x + (size_t)src * ld + c);
    else raw = *reinterpret_cast<const uint32_t*>(state + ((size_t)slot * (Kc - 1) + (Kc - 1 + src - t_start)) * C + c);
    v0[j] = bf16_lo(raw);
    v1[j] = bf16_hi(raw);
  }
  float a0 = 0.f, a1 = 0.f;
  for (int j = 0; j < Kc; ++j) {
    a0 = fmaf(w[(size_t)c * Kc + j], v0[j], a0);
    a1 = fmaf(w[(size_t)(c + 1) * Kc + j], v1[j], a1);
  }
  a0 = a0 / (1.f + __expf(-a0));
  a1 = a1 / (1.f + __expf(-a1));
  *reinterpret_cast<uint32_t*>(y + (size_t)t * C + c) = pack_bf16(a0, a1);
  if (ckpt)
    for (int p = 0; p + 1 < Kc; ++p) *reinterpret_cast<uint32_t*>(ckpt + ((size_t)t * (Kc - 1) + p) * C + c) = pack_bf16(v0[p + 1], v1[p + 1]);
  if (fuse_state)   // every sequence has exactly one token: this thread owns the channel pair of its slot
    for (int p = 0; p + 1 < Kc; ++p) *reinterpret_cast<uint32_t*>(state + ((size_t)slot * (Kc - 1) + p) * C + c) = pack_bf16(v0[p + 1], v1[p + 1]);
}

// Prefill form: a thread owns four channels and walks a strip of CONV_STRIP tokens with the Kc-tap window in registers, so an
// input element is read about once (plus Kc-1 per strip) instead of Kc times and the taps are loaded once per strip.  Sequence
// starts inside a strip reload the window from the stored state.
constexpr int CONV_STRIP = 16;

template <int KC>
__global__ void __launch_bounds__(128) conv1d_silu_strip_kernel(const bf16* __restrict__ x, int ld, int C, const float* __restrict__ w,
                                                                const bf16* __restrict__ state, const int* __restrict__ slots,
                                                                const int* __restrict__ cu_q, int B, int T, bf16* __restrict__ y,
                                                                bf16* __restrict__ ckpt) {
  pdl_prologue();
  const int c = (blockIdx.x * 128 + threadIdx.x) * 4;
  if (c >= C) return;
  const int t_lo = blockIdx.y * CONV_STRIP, t_hi = min(T, t_lo + CONV_STRIP);
  float wt[KC][4];                         // [tap][channel]
#pragma unroll
  for (int j = 0; j < KC; ++j)
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) wt[j][ch] = w[(size_t)(c + ch) * KC + j];
  float win[KC][4];                        // win[j] = input at t - (KC - 1) + j
  auto unpack = [](const uint2 raw, float (&o)[4]) {
    o[0] = bf16_lo(raw.x); o[1] = bf16_hi(raw.x); o[2] = bf16_lo(raw.y); o[3] = bf16_hi(raw.y);
  };
  uint2 cur[CONV_STRIP];                   // the strip's own inputs, fetched together (one trip to memory)
#pragma unroll
  for (int i = 0; i < CONV_STRIP; ++i)
    cur[i] = t_lo + i < t_hi ? *reinterpret_cast<const uint2*>(x + (size_t)(t_lo + i) * ld + c) : make_uint2(0u, 0u);
  int b = 0;
  while (b + 1 < B && cu_q[b + 1] <= t_lo) ++b;
  int t_start = cu_q[b], t_next = cu_q[b + 1];
  bool fresh = true;                       // the window has to be (re)loaded: first token of the strip or of a sequence
#pragma unroll
  for (int i = 0; i < CONV_STRIP; ++i) {
    const int t = t_lo + i;
    if (t >= t_hi) break;
    while (t >= t_next && b + 1 < B) { ++b; t_start = cu_q[b]; t_next = cu_q[b + 1]; fresh = true; }
    if (fresh) {
      const int slot = slots[b];
#pragma unroll
      for (int j = 0; j < KC - 1; ++j) {
        const int src = t - (KC - 1) + j;
        unpack(src >= t_start ? *reinterpret_cast<const uint2*>(x + (size_t)src * ld + c)
                              : *reinterpret_cast<const uint2*>(state + ((size_t)slot * (KC - 1) + (KC - 1 + src - t_start)) * C + c), win[j]);
      }
      fresh = false;
    }
    unpack(cur[i], win[KC - 1]);
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < KC; ++j)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) a[ch] = fmaf(wt[j][ch], win[j][ch], a[ch]);
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) a[ch] = __fdividef(a[ch], 1.f + __expf(-a[ch]));
    *reinterpret_cast<uint2*>(y + (size_t)t * C + c) = make_uint2(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]));
    if (ckpt)
#pragma unroll
      for (int pp = 0; pp < KC - 1; ++pp)
        *reinterpret_cast<uint2*>(ckpt + ((size_t)t * (KC - 1) + pp) * C + c) =
            make_uint2(pack_bf16(win[pp + 1][0], win[pp + 1][1]), pack_bf16(win[pp + 1][2], win[pp + 1][3]));
#pragma unroll
    for (int j = 0; j < KC - 1; ++j)         // slide
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) win[j][ch] = win[j + 1][ch];
  }
}

// New streaming state after a multi-token step: the last Kc-1 inputs of every sequence.  One thread owns a channel
// pair of a sequence and walks p upwards, so an old entry is read (at p + q_len) before it is overwritten.
__global__ void conv1d_state_kernel(const bf16* __restrict__ x, int ld, int C, int Kc, bf16* __restrict__ state, const int* __restrict__ slots,
                                    const int* __restrict__ cu_q) {
  pdl_prologue();
  const int b = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const int t_start = cu_q[b], t_end = cu_q[b + 1], q_len = t_end - t_start;
  if (q_len <= 0) return;
  bf16* st = state + (size_t)slots[b] * (Kc - 1) * C + c;
  for (int p = 0; p + 1 < Kc; ++p) {
    const int src = t_end - (Kc - 1) + p;
    const uint32_t raw = src >= t_start ? *reinterpret_cast<const uint32_t*>(x + (size_t)src * ld + c)
                                        : *reinterpret_cast<const uint32_t*>(st + (size_t)(p + q_len) * C);
    *reinterpret_cast<uint32_t*>(st + (size_t)p * C) = raw;
  }
}

// ------------------------------------------------------------------ gated delta rule scan
constexpr int DN_D = 128;        // key and value head width
constexpr int DN_VSPLIT = 4;     // CTAs per (sequence, v-head)
constexpr int DN_VC = DN_D / DN_VSPLIT;   // value columns per CTA
constexpr int DN_LANES = 8;      // lanes that share one value column (each keeps DN_KPT key rows of it in registers)
constexpr int DN_KPT = DN_D / DN_LANES;
constexpr int DN_THREADS = DN_VC * DN_LANES;
constexpr int DN_CH = 16;        // tokens staged per chunk
constexpr int DN_KSTR = 20;      // smem stride of one 16-float key slice (padded: the eight slices of a column hit different banks)

struct ScanParams {
  const bf16* qkv; int ld; int q_off, k_off, v_off;     // conv output [T, ld]
  const bf16* ab; int ab_ld;                            // alpha / beta logits, one column per v-head through the index tables
  const int* a_idx; const int* b_idx; const int* k_of_v;
  const float* ssm_a; const float* dt_bias;
  float* state;                                         // [slots, n_v, 128 (v), 128 (k)] fp32
  const int* slots; const int* cu_q;
  float* out;                                           // [T, n_v * 128] fp32
  float* ckpt;                                          // optional [T, n_v, 128 (v), 128 (k)]
  int n_v; float q_scale; float eps;
};

struct ScanStage {     // one chunk of raw inputs held in registers while the previous chunk is being scanned
  uint2 q[2], k[2]; uint32_t v; float a, b;
};

// 8 warps: warp w stages tokens 2w and 2w+1 (lane l holds key elements 4l..4l+3 of q and k)
__device__ __forceinline__ void scan_prefetch(const ScanParams& p, ScanStage& s, int tc, int n, int h, int kh, int vs) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int tok = warp * 2 + r;
    if (tok < n) {
      const bf16* row = p.qkv + (size_t)(tc + tok) * p.ld + kh * DN_D + lane * 4;
      s.q[r] = *reinterpret_cast<const uint2*>(row + p.q_off);
      s.k[r] = *reinterpret_cast<const uint2*>(row + p.k_off);
    }
  }
  {
    const int tok = tid >> 4, c2 = (tid & 15) * 2;
    if (tok < n) s.v = *reinterpret_cast<const uint32_t*>(p.qkv + (size_t)(tc + tok) * p.ld + p.v_off + h * DN_D + vs * DN_VC + c2);
  }
  if (tid < n) {
    s.a = __bfloat162float(p.ab[(size_t)(tc + tid) * p.ab_ld + p.a_idx[h]]);
    s.b = __bfloat162float(p.ab[(size_t)(tc + tid) * p.ab_ld + p.b_idx[h]]);
  }
}

__device__ __forceinline__ int dn_koff(int k) { return (k >> 4) * DN_KSTR + (k & 15); }     // key element -> padded smem offset

__global__ void __launch_bounds__(DN_THREADS) deltanet_scan_kernel(ScanParams p) {
  pdl_prologue();
  const int h = blockIdx.x / DN_VSPLIT, vs = blockIdx.x % DN_VSPLIT, b = blockIdx.y;
  const int t0 = p.cu_q[b], t1 = p.cu_q[b + 1];
  if (t1 <= t0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = tid / DN_LANES, kq = tid % DN_LANES, col = vs * DN_VC + c;
  const int kh = p.k_of_v[h];
  __shared__ __align__(16) float sq[DN_CH][DN_LANES * DN_KSTR];
  __shared__ __align__(16) float sk[DN_CH][DN_LANES * DN_KSTR];
  __shared__ float sv[DN_CH][DN_VC];
  __shared__ float sdecay[DN_CH], sbeta[DN_CH], sqk[DN_CH];

  float S[DN_KPT];
  float* sp = p.state + (((size_t)p.slots[b] * p.n_v + h) * DN_D + col) * DN_D + kq * DN_KPT;
#pragma unroll
  for (int j = 0; j < DN_KPT / 4; ++j) {
    const float4 v = reinterpret_cast<const float4*>(sp)[j];
    S[4 * j] = v.x; S[4 * j + 1] = v.y; S[4 * j + 2] = v.z; S[4 * j + 3] = v.w;
  }
  const float a_h = p.ssm_a[h], dtb = p.dt_bias[h];
  ScanStage st;
  scan_prefetch(p, st, t0, min(DN_CH, t1 - t0), h, kh, vs);
  for (int tc = t0; tc < t1; tc += DN_CH) {
    const int n = min(DN_CH, t1 - tc);
    __syncthreads();                       // the previous chunk's shared tiles are no longer read
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int tok = warp * 2 + r;
      if (tok < n) {                       // warp-uniform
        const float q0 = bf16_lo(st.q[r].x), q1 = bf16_hi(st.q[r].x), q2 = bf16_lo(st.q[r].y), q3 = bf16_hi(st.q[r].y);
        const float k0 = bf16_lo(st.k[r].x), k1 = bf16_hi(st.k[r].x), k2 = bf16_lo(st.k[r].y), k3 = bf16_hi(st.k[r].y);
        const float ssq = warp_sum(q0 * q0 + q1 * q1 + q2 * q2 + q3 * q3);
        const float ssk = warp_sum(k0 * k0 + k1 * k1 + k2 * k2 + k3 * k3);
        const float dqk = warp_sum(q0 * k0 + q1 * k1 + q2 * k2 + q3 * k3);
        const float iq = rsqrtf(ssq + p.eps) * p.q_scale, ik = rsqrtf(ssk + p.eps);
        const int o = dn_koff(lane * 4);
        *reinterpret_cast<float4*>(&sq[tok][o]) = make_float4(q0 * iq, q1 * iq, q2 * iq, q3 * iq);
        *reinterpret_cast<float4*>(&sk[tok][o]) = make_float4(k0 * ik, k1 * ik, k2 * ik, k3 * ik);
        if (lane == 0) sqk[tok] = dqk * iq * ik;
      }
    }
    {
      const int tok = tid >> 4, c2 = (tid & 15) * 2;
      if (tok < n) { sv[tok][c2] = bf16_lo(st.v); sv[tok][c2 + 1] = bf16_hi(st.v); }
    }
    if (tid < n) {
      const float x = st.a + dtb;
      const float sp_ = fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x)));      // softplus
      sdecay[tid] = __expf(a_h * sp_);
      sbeta[tid] = 1.f / (1.f + __expf(-st.b));
    }
    __syncthreads();
    if (tc + DN_CH < t1) scan_prefetch(p, st, tc + DN_CH, min(DN_CH, t1 - tc - DN_CH), h, kh, vs);
    // The recurrence S -> S^T k -> delta -> S is one dependent chain per token: every 16-term dot runs as four
    // independent partial sums, and two warps per scheduler interleave their chains.
    for (int i = 0; i < n; ++i) {
      const float4* kk = reinterpret_cast<const float4*>(&sk[i][kq * DN_KSTR]);
      const float4* qq = reinterpret_cast<const float4*>(&sq[i][kq * DN_KSTR]);
      float4 k4[DN_KPT / 4];
      float ak[4] = {0.f, 0.f, 0.f, 0.f}, aq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < DN_KPT / 4; ++j) {
        k4[j] = kk[j];
        const float4 q4 = qq[j];
        ak[0] = fmaf(S[4 * j], k4[j].x, ak[0]); ak[1] = fmaf(S[4 * j + 1], k4[j].y, ak[1]);
        ak[2] = fmaf(S[4 * j + 2], k4[j].z, ak[2]); ak[3] = fmaf(S[4 * j + 3], k4[j].w, ak[3]);
        aq[0] = fmaf(S[4 * j], q4.x, aq[0]); aq[1] = fmaf(S[4 * j + 1], q4.y, aq[1]);
        aq[2] = fmaf(S[4 * j + 2], q4.z, aq[2]); aq[3] = fmaf(S[4 * j + 3], q4.w, aq[3]);
      }
      float sk_ = (ak[0] + ak[1]) + (ak[2] + ak[3]), sq_ = (aq[0] + aq[1]) + (aq[2] + aq[3]);
#pragma unroll
      for (int m = 1; m < DN_LANES; m <<= 1) {
        sk_ += __shfl_xor_sync(0xffffffffu, sk_, m);
        sq_ += __shfl_xor_sync(0xffffffffu, sq_, m);
      }
      const float decay = sdecay[i];
      const float delta = (sv[i][c] - decay * sk_) * sbeta[i];
#pragma unroll
      for (int j = 0; j < DN_KPT / 4; ++j) {
        S[4 * j] = fmaf(S[4 * j], decay, k4[j].x * delta); S[4 * j + 1] = fmaf(S[4 * j + 1], decay, k4[j].y * delta);
        S[4 * j + 2] = fmaf(S[4 * j + 2], decay, k4[j].z * delta); S[4 * j + 3] = fmaf(S[4 * j + 3], decay, k4[j].w * delta);
      }
      if (kq == 0) p.out[(size_t)(tc + i) * p.n_v * DN_D + h * DN_D + col] = decay * sq_ + delta * sqk[i];
      if (p.ckpt) {
        float* cp = p.ckpt + ((((size_t)(tc + i)) * p.n_v + h) * DN_D + col) * DN_D + kq * DN_KPT;
#pragma unroll
        for (int j = 0; j < DN_KPT / 4; ++j) reinterpret_cast<float4*>(cp)[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < DN_KPT / 4; ++j) reinterpret_cast<float4*>(sp)[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
}

// ------------------------------------------------------------------ gated RMSNorm, z read through a row stride
__global__ void __launch_bounds__(128) gated_rmsnorm_ld_kernel(const float* __restrict__ x, const bf16* __restrict__ z, int z_ld,
                                                               const float* __restrict__ w, bf16* __restrict__ y, int T, int n_h, int hd,
                                                               float eps) {
  pdl_prologue();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= T * n_h) return;
  const int t = r / n_h, h = r % n_h;
  const float* xr = x + (size_t)r * hd;
  const bf16* zr = z + (size_t)t * z_ld + h * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) ss += xr[i] * xr[i];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / hd + eps);
  for (int i = lane; i < hd; i += 32) {
    const float zz = __bfloat162float(zr[i]);
    y[(size_t)r * hd + i] = __float2bfloat16(xr[i] * inv * w[i] * (zz / (1.f + __expf(-zz))));
  }
}

}  // namespace mx

using namespace mx;

MX_HOST_API int mx_conv1d_silu(const void* x, int ld, int C, int Kc, const float* w, void* state, const int* slots, const int* cu_q, int B,
                               int T, int max_q_len, void* y, void* ckpt, cudaStream_t st) {
  if (T <= 0) return 0;
  if (Kc < 2 || Kc > 8 || (C & 1) || (ld & 1)) return -101;
  const int fuse = max_q_len == 1;
  if (!fuse && T >= 4 * CONV_STRIP && (Kc == 4 || Kc == 3) && (C & 3) == 0 && (ld & 3) == 0 && ((uintptr_t)x & 7) == 0 && ((uintptr_t)state & 7) == 0) {
    dim3 grid((C / 4 + 127) / 128, (T + CONV_STRIP - 1) / CONV_STRIP);
    if (Kc == 4)
      launch_pdl(conv1d_silu_strip_kernel<4>, dim3(grid), dim3(128), 0, st, (const bf16*)x, ld, C, w, (const bf16*)state, slots, cu_q, B, T, (bf16*)y, (bf16*)ckpt);
    else
      launch_pdl(conv1d_silu_strip_kernel<3>, dim3(grid), dim3(128), 0, st, (const bf16*)x, ld, C, w, (const bf16*)state, slots, cu_q, B, T, (bf16*)y, (bf16*)ckpt);
  } else {
    dim3 grid((C / 2 + 127) / 128, T);
    launch_pdl(conv1d_silu_kernel, dim3(grid), dim3(128), 0, st, (const bf16*)x, ld, C, Kc, w, (bf16*)state, slots, cu_q, B, (bf16*)y, (bf16*)ckpt, fuse);
  }
  if (!fuse) {
    dim3 g2((C / 2 + 127) / 128, B);
    launch_pdl(conv1d_state_kernel, dim3(g2), dim3(128), 0, st, (const bf16*)x, ld, C, Kc, (bf16*)state, slots, cu_q);
  }
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_deltanet_scan(const void* qkv, int ld, int q_off, int k_off, int v_off, const void* ab, int ab_ld, const int* a_idx,
                                 const int* b_idx, const int* k_of_v, const float* ssm_a, const float* dt_bias, float* state,
                                 const int* slots, const int* cu_q, int B, int n_v, int head_dim, float q_scale, float eps, float* out,
                                 float* ckpt, cudaStream_t st) {
  if (B <= 0 || n_v <= 0) return 0;
  if (head_dim != DN_D || (ld & 3) || (q_off & 3) || (k_off & 3) || (v_off & 3)) return -101;
  ScanParams p;
  p.qkv = (const bf16*)qkv; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.ab = (const bf16*)ab; p.ab_ld = ab_ld; p.a_idx = a_idx; p.b_idx = b_idx; p.k_of_v = k_of_v;
  p.ssm_a = ssm_a; p.dt_bias = dt_bias; p.state = state; p.slots = slots; p.cu_q = cu_q; p.out = out; p.ckpt = ckpt;
  p.n_v = n_v; p.q_scale = q_scale; p.eps = eps;
  launch_pdl(deltanet_scan_kernel, dim3(dim3(n_v * DN_VSPLIT, B)), dim3(DN_THREADS), 0, st, p);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_gated_rmsnorm_ld(const float* x, const void* z, int z_ld, const float* w, void* y, int T, int n_h, int hd, float eps,
                                    cudaStream_t st) {
  if (T <= 0) return 0;
  launch_pdl(gated_rmsnorm_ld_kernel, dim3((T * n_h + 3) / 4), dim3(128), 0, st, x, (const bf16*)z, z_ld, w, (bf16*)y, T, n_h, hd, eps);
  return (int)cudaGetLastError();
}
