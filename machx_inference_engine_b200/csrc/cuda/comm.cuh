// Peer-memory all-reduce that is fused into its producer and its consumer.
//
// Every rank owns an "inbox" in device memory that all peers have mapped (CUDA IPC over NVLink):
//     inbox[parity 0..1][source rank 0..W-1][slot_bytes]      followed by      flags[W] , seq
// A row-parallel GEMM / GEMV (or the MoE combine) does not write its partial result locally: its
// epilogue stores the partial straight into slot [parity][my_rank] of EVERY rank's inbox with plain
// peer stores, and the last CTA of the kernel publishes a sequence number into every rank's flag word
// for this source.  The consumer (the following residual + RMSNorm kernel, or a plain reduce) waits
// until all W flags reach its own sequence number and sums the W slots in rank order, so the result is
// bit-identical on every rank and from run to run.  No separate collective kernel runs and nothing
// goes through NCCL.
//
// Two parities make slot reuse safe without acknowledgements: a rank can only start pushing sequence
// s+2 after it consumed s+1, which needs every peer's push of s+1, which each peer issues only after it
// consumed s.  Sequence numbers live in device memory (one word per rank, bumped by the producer's last
// CTA), so captured CUDA graphs replay correctly.  Every wait is bounded and reports through the
// status word.  Only plain loads and stores touch peer memory: no TMA, no multicast.
//
// Reference parity: replaces DeviceFleet::all_reduce_sum_fp16 (src/core/allocator.cpp:158-193) at the
// call sites dense_tp.cpp:402,416, gptoss_tp.cpp:961,999, qwen3moe_tp.cpp:653,662, qwen35_tp.cpp:750.
#pragma once
#include "common.cuh"

namespace mx {

constexpr int kMaxPeers = 8;

struct PeerOut {
  uint8_t* inbox[kMaxPeers];   // base of every rank's inbox (index = destination rank); null entries unused
  int world;                   // 0 = not a fused-collective launch
  int my_rank;
  long long slot_bytes;
  int* seq;                    // this rank's sequence word (device, local)
  int* ticket;                 // CTA arrival counter (device, local)
  int rs_rows;                 // > 0: reduce-scatter form, row t goes only to rank min(t / rs_rows, world - 1)
};

// Reduce-scatter form (prefill-sized collectives).  Writing every partial to every rank moves (W-1) full [T,H] tensors
// per rank; instead a producer sends each row only to the rank that owns it, the owner sums the W partials of its rows
// and broadcasts the reduced rows (bf16) into every rank's gather region, and the consumer reads that single tensor:
// 2 (W-1)/W [T,H] per rank.  The gather region [2 parities][slot_bytes] and its W flags follow the inbox flags.
__device__ __forceinline__ int peer_first(const PeerOut& po, int row) { return po.rs_rows > 0 ? min(row / po.rs_rows, po.world - 1) : 0; }
__device__ __forceinline__ int peer_count(const PeerOut& po) { return po.rs_rows > 0 ? 1 : po.world; }
__host__ __device__ __forceinline__ long long gather_offset(int world, long long slot_bytes) { return 2ll * world * slot_bytes + 4096; }
__host__ __device__ __forceinline__ long long gather_flags_offset(int world, long long slot_bytes) { return gather_offset(world, slot_bytes) + 2 * slot_bytes; }
__host__ __device__ __forceinline__ long long inbox_total_bytes(int world, long long slot_bytes) { return gather_flags_offset(world, slot_bytes) + 4096; }

__device__ __forceinline__ long long inbox_flags_offset(int world, long long slot_bytes) { return 2ll * world * slot_bytes; }

// Destination of this rank's partial inside rank `dst`'s inbox for the collective that is being produced.
__device__ __forceinline__ uint8_t* peer_slot(const PeerOut& po, int dst, int next_seq) {
  return po.inbox[dst] + ((long long)(next_seq & 1) * po.world + po.my_rank) * po.slot_bytes;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by every thread of every CTA after its last peer store.  The last CTA to arrive bumps the
// sequence word and publishes it to all ranks.
__device__ __forceinline__ void peer_publish(const PeerOut& po, int next_seq) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned prev = atomicAdd((unsigned*)po.ticket, 1u);
    if (prev == total - 1) {
      *po.ticket = 0;
      __threadfence_system();
      for (int r = 0; r < po.world; ++r) {
        int* flags = reinterpret_cast<int*>(po.inbox[r] + inbox_flags_offset(po.world, po.slot_bytes));
        st_release_sys(flags + po.my_rank, next_seq);
      }
      *po.seq = next_seq;
    }
  }
}

}  // namespace mx
