// Host plumbing and the stand-alone kernels of the peer-memory all-reduce (see comm.cuh):
//   * CUDA IPC export / import of the inbox allocation
//   * push      : copy an existing local tensor into every rank's inbox (producers that cannot take
//                 the fused epilogue, e.g. the MoE combine output)
//   * reduce    : consumer that materialises sum_r inbox[r] (+bias) as a tensor
//   * rmsnorm_reduce : consumer fused with the residual add and RMSNorm that follows every
//                 row-parallel projection:  x += sum_r inbox[r] (+bias);  out = rmsnorm(x) * w
// The fused producers are the GEMV / GEMM epilogues (gemv.cu, gemm_tcgen05.cu) given a PeerOut.
#include "comm.cuh"
#include "host_util.h"

#include <cstring>

namespace mx {

// How long a consumer waits for its peers' flags, in SM clock cycles (about one second by default); mx_set_wait_limit_cycles
// lowers it for the test that lets a wait run out.
__device__ long long g_wait_limit_cycles = 2000000000ll;

// Bounded wait until every source's flag reached `seq`.  One thread per CTA polls (with a short sleep between polls, so that
// thousands of waiting CTAs do not saturate the path the flag arrives on), the CTA follows.
__device__ __forceinline__ bool wait_all_flags(const int* flags, int world, int seq, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64(), limit = g_wait_limit_cycles;
    for (int r = 0; r < world; ++r) {
      while (ld_acquire_sys(flags + r) - seq < 0) {
        __nanosleep(32);
        if (clock64() - t0 > limit) { atomicCAS(status, 0, ERR_PEER_FLAG_TIMEOUT); ok = 0; break; }
      }
      if (!ok) break;
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

template <typename ST>
__device__ __forceinline__ float4 load4(const ST* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
}

__global__ void push_kernel(const uint4* __restrict__ src, long long n16, PeerOut po) {
  pdl_prologue();
  const int next_seq = *po.seq + 1;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int r = 0; r < po.world; ++r) reinterpret_cast<uint4*>(peer_slot(po, r, next_seq))[i] = v;
  }
  peer_publish(po, next_seq);
}

// Reduce-scatter owner step: this rank sums the W partials of its rows [row0, row1) and stores the reduced rows as bf16
// into every rank's gather region; the last CTA publishes the gather flags.
template <typename ST>
__global__ void __launch_bounds__(256) rs_gather_kernel(const uint8_t* __restrict__ inbox, PeerOut po, const float* __restrict__ bias, int row0,
                                                        int row1, int H, int* status) {
  pdl_prologue();
  const int s = *po.seq;
  const int world = po.world;
  const int* flags = reinterpret_cast<const int*>(inbox + 2ll * world * po.slot_bytes);
  const bool ok = wait_all_flags(flags, world, s, status);
  const uint8_t* base = inbox + (long long)(s & 1) * world * po.slot_bytes;
  const long long goff = gather_offset(world, po.slot_bytes) + (long long)(s & 1) * po.slot_bytes;
  for (int t = row0 + blockIdx.x; t < row1 && ok; t += gridDim.x) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 d = load4<ST>(reinterpret_cast<const ST*>(base + r * po.slot_bytes) + (size_t)t * H + i);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      }
      if (bias) { a.x += bias[i]; a.y += bias[i + 1]; a.z += bias[i + 2]; a.w += bias[i + 3]; }
      const uint2 o = make_uint2(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w));
      for (int d = 0; d < world; ++d) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(po.inbox[d] + goff) + (size_t)t * H + i) = o;
    }
  }
  // publish: same ticket scheme as peer_publish, into the gather flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd((unsigned*)po.ticket, 1u);
    if (prev == total - 1) {
      *po.ticket = 0;
      __threadfence_system();
      for (int r = 0; r < world; ++r) {
        int* gflags = reinterpret_cast<int*>(po.inbox[r] + gather_flags_offset(world, po.slot_bytes));
        st_release_sys(gflags + po.my_rank, s);
      }
    }
  }
}

// out[t][:] = sum_r slot_r[t][:] (+bias).  gathered: the single bf16 tensor of the gather region (bias already added).
template <typename ST>
__global__ void __launch_bounds__(256) reduce_kernel(const uint8_t* __restrict__ inbox, int world, long long slot_bytes, const int* __restrict__ seq,
                                                     const float* __restrict__ bias, float* __restrict__ out, long long n, int H, int* status,
                                                     int gathered) {
  pdl_prologue();
  const int s = *seq;
  const int* flags = reinterpret_cast<const int*>(inbox + (gathered ? gather_flags_offset(world, slot_bytes) : 2ll * world * slot_bytes));
  if (!wait_all_flags(flags, world, s, status)) return;
  const uint8_t* base = gathered ? inbox + gather_offset(world, slot_bytes) + (long long)(s & 1) * slot_bytes
                                 : inbox + (long long)(s & 1) * world * slot_bytes;
  if (gathered) world = 1;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = load4<ST>(reinterpret_cast<const ST*>(base + r * slot_bytes) + i);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    if (bias) { const int c = (int)(i % H); a.x += bias[c]; a.y += bias[c + 1]; a.z += bias[c + 2]; a.w += bias[c + 3]; }
    *reinterpret_cast<float4*>(out + i) = a;
  }
}

// x[t][:] += (sum_r slot_r[t][:] + bias) * delta_scale ;  out = rmsnorm(x) * w
template <typename ST>
__global__ void __launch_bounds__(256) rmsnorm_reduce_kernel(float* __restrict__ x, const uint8_t* __restrict__ inbox, int world, long long slot_bytes,
                                                             const int* __restrict__ seq, const float* __restrict__ dbias, const float* __restrict__ w,
                                                             __nv_bfloat16* __restrict__ out, float eps, int H, int one_plus_w, float delta_scale,
                                                             int* status, int gathered) {
  pdl_prologue();
  const int s = *seq;
  const int* flags = reinterpret_cast<const int*>(inbox + (gathered ? gather_flags_offset(world, slot_bytes) : 2ll * world * slot_bytes));
  if (!wait_all_flags(flags, world, s, status)) return;
  const uint8_t* base = gathered ? inbox + gather_offset(world, slot_bytes) + (long long)(s & 1) * slot_bytes
                                 : inbox + (long long)(s & 1) * world * slot_bytes;
  if (gathered) world = 1;
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * H;
  __shared__ float red[8];
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(xr + i);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 d = load4<ST>(reinterpret_cast<const ST*>(base + r * slot_bytes) + (size_t)t * H + i);
      a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
    }
    if (dbias) { a.x += dbias[i]; a.y += dbias[i + 1]; a.z += dbias[i + 2]; a.w += dbias[i + 3]; }
    v.x += a.x * delta_scale; v.y += a.y * delta_scale; v.z += a.z * delta_scale; v.w += a.w * delta_scale;
    *reinterpret_cast<float4*>(xr + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / H + eps);
  }
  __syncthreads();
  const float inv = red[0];
  if (!out) return;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    float4 g = *reinterpret_cast<const float4*>(w + i);
    if (one_plus_w) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
    uint2 o;
    o.x = pack_bf16(v.x * inv * g.x, v.y * inv * g.y);
    o.y = pack_bf16(v.z * inv * g.z, v.w * inv * g.w);
    *reinterpret_cast<uint2*>(out + (size_t)t * H + i) = o;
  }
}

PeerOut make_peer_out(const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket) {
  PeerOut po;
  memset(&po, 0, sizeof po);
  for (int r = 0; r < world && r < kMaxPeers; ++r) po.inbox[r] = (uint8_t*)inbox[r];
  po.world = world; po.my_rank = my_rank; po.slot_bytes = slot_bytes; po.seq = seq; po.ticket = ticket;
  return po;
}

}  // namespace mx

using namespace mx;

// The inbox is a dedicated cudaMalloc allocation (IPC handles describe whole allocations), zero-filled
// so that flags and sequence numbers start at 0.
// Time limit of the consumers' flag waits on the current device, in SM cycles (default 2e9, about a second).
MX_HOST_API int mx_set_wait_limit_cycles(long long cycles) {
  if (cycles < 1000) return -1;
  return (int)cudaMemcpyToSymbol(g_wait_limit_cycles, &cycles, sizeof cycles);
}

MX_HOST_API void* mx_raw_alloc(long long bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, (size_t)bytes);
  cudaDeviceSynchronize();
  return p;
}
MX_HOST_API int mx_raw_free(void* p) { return (int)cudaFree(p); }

MX_HOST_API int mx_ipc_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
MX_HOST_API int mx_ipc_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
MX_HOST_API int mx_ipc_release(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

// src: n_bytes (multiple of 16) of an existing local tensor -> slot [my_rank] of every inbox
MX_HOST_API int mx_comm_push(const void* src, long long n_bytes, const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq,
                             int* ticket, cudaStream_t st) {
  if (n_bytes % 16 || n_bytes > slot_bytes) return -140;
  PeerOut po = make_peer_out(inbox, world, my_rank, slot_bytes, seq, ticket);
  const long long n16 = n_bytes / 16;
  int grid = (int)((n16 + 255) / 256);
  grid = grid < 1 ? 1 : (grid > 2 * sm_count() ? 2 * sm_count() : grid);
  launch_pdl(push_kernel, dim3(grid), dim3(256), 0, st, (const uint4*)src, n16, po);
  return (int)cudaGetLastError();
}

// slot_is_bf16: element type of the slots.  n = T*H elements (multiple of 4).
MX_HOST_API long long mx_comm_inbox_bytes(int world, long long slot_bytes) { return inbox_total_bytes(world, slot_bytes); }

// Owner step of the reduce-scatter form: rows [row0, row1) of this rank, slots hold bf16 or fp32 partials.
MX_HOST_API int mx_comm_rs_gather(const void* const* inbox, int world, int my_rank, long long slot_bytes, int* seq, int* ticket, int slot_is_bf16,
                                  const float* bias, int row0, int row1, int H, cudaStream_t st) {
  if (H % 4) return -107;
  PeerOut po = make_peer_out(inbox, world, my_rank, slot_bytes, seq, ticket);
  const int rows = row1 - row0;
  const int grid = rows < 1 ? 1 : (rows > 4 * sm_count() ? 4 * sm_count() : rows);
  if (slot_is_bf16) launch_pdl(rs_gather_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const uint8_t*)inbox[my_rank], po, bias, row0, row1, H, status_word());
  else launch_pdl(rs_gather_kernel<float>, dim3(grid), dim3(256), 0, st, (const uint8_t*)inbox[my_rank], po, bias, row0, row1, H, status_word());
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_comm_reduce(const void* my_inbox, int world, long long slot_bytes, const int* seq, int slot_is_bf16, const float* bias, float* out,
                               long long n, int H, int gathered, cudaStream_t st) {
  if (n % 4 || H % 4) return -107;
  int grid = (int)((n / 4 + 255) / 256);
  grid = grid < 1 ? 1 : (grid > 4 * sm_count() ? 4 * sm_count() : grid);
  if (slot_is_bf16) launch_pdl(reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, (const uint8_t*)my_inbox, world, slot_bytes, seq, bias, out, n, H, status_word(), gathered);
  else launch_pdl(reduce_kernel<float>, dim3(grid), dim3(256), 0, st, (const uint8_t*)my_inbox, world, slot_bytes, seq, bias, out, n, H, status_word(), gathered);
  return (int)cudaGetLastError();
}

MX_HOST_API int mx_comm_rmsnorm_reduce(float* x, const void* my_inbox, int world, long long slot_bytes, const int* seq, int slot_is_bf16,
                                       const float* dbias, const float* w, void* out_bf16, float eps, int T, int H, int one_plus_w,
                                       float delta_scale, int gathered, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 4) return -107;
  if (slot_is_bf16)
    launch_pdl(rmsnorm_reduce_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, st, x, (const uint8_t*)my_inbox, world, slot_bytes, seq, dbias, w, (__nv_bfloat16*)out_bf16,
                                                              eps, H, one_plus_w, delta_scale, status_word(), gathered);
  else
    launch_pdl(rmsnorm_reduce_kernel<float>, dim3(T), dim3(256), 0, st, x, (const uint8_t*)my_inbox, world, slot_bytes, seq, dbias, w, (__nv_bfloat16*)out_bf16, eps, H,
                                                    one_plus_w, delta_scale, status_word(), gathered);
  return (int)cudaGetLastError();
}
