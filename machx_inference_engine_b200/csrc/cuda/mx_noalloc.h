// Allocation-free attention entry point.
//
// This entry point has no counterpart in the reference engine; it exists for hosts that embed this
// library but are not allowed to allocate device memory themselves.
//
// Who needs it: a host runtime that has already handed every byte of HBM to its own pools (weights,
// KV pages, activation arenas) and forbids cudaMalloc / cudaFree after start-up; a latency-critical
// loop that must never take the driver's allocator lock; and callers written against a fixed memory
// budget who audit every allocation.  The regular mx_attention() makes its caller provide two scratch
// buffers for the split-KV partial results (so somebody has to allocate them); mx_attention_noalloc()
// keeps that scratch inside the library, in a file-scope device array of fixed size, and the caller
// passes only inputs and the output.
//
// Contract
//   * Scratch capacity: MX_NOALLOC_SCRATCH_FLOATS floats (8 MiB) per device.  The call needs
//     n_splits * Tq * n_q * (head_dim + 2) floats; a larger request is refused with
//     MX_NOALLOC_E_TOO_LARGE and nothing is launched.  mx_attention_noalloc_error() returns the text.
//   * Every GPU that loads this library carries the 8 MiB array until the process exits, used or not.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress) and caches
//     it.  Make that first call outside of any stream capture; later calls do no set-up work.
//   * No cudaMalloc, cudaFree, or allocating library routine is called, on any path.
//   * All calls on a device share the one array.  The kernels overwrite every scratch element they
//     later read, so stale contents from an earlier call are harmless and nothing has to be cleared;
//     but two calls whose kernels overlap on the GPU (different streams) would race on it.  Serialise
//     them: same stream, or an event between them.
//   * Arguments and numerics are those of mx_attention(): the two entry points run the same kernels.
#pragma once
#include <cuda_runtime.h>

#define MX_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define MX_NOALLOC_E_TOO_LARGE (-130)
#define MX_NOALLOC_E_SYMBOL (-131)

#ifdef __cplusplus
extern "C" {
#endif

int mx_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_table, const int* seq_lens,
                         const int* cu_q, const float* sinks, void* out, int B, int Tq, int max_q_len, int n_q, int n_kv, int hd,
                         int max_blocks, int block_size, int window, float scale, float softcap, int n_splits, cudaStream_t stream);

// Text of the last refusal or set-up failure on the calling thread ("" if none).
const char* mx_attention_noalloc_error(void);

#ifdef __cplusplus
}
#endif
