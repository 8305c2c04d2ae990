// Host-side declarations shared between the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace mx {
// "Has this kernel's attribute been set on the current device yet": function attributes such as the dynamic shared-memory
// limit are per device, so a launcher keeps one latch bit per device ordinal (a process may drive several GPUs).  Two threads
// that race through `pending()` both set the attribute, which is harmless.
struct DeviceOnce {
  std::atomic<unsigned long long> done{0};
  static int ordinal() { int d = 0; cudaGetDevice(&d); return d & 63; }
  bool pending() const { return !((done.load(std::memory_order_acquire) >> ordinal()) & 1ull); }
  void mark() { done.fetch_or(1ull << ordinal(), std::memory_order_release); }
};

int* status_word();
int sm_count();
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, int swizzle128);
int make_tmap_bytes(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t row_stride, uint32_t box_bytes, uint32_t box_rows);
bool pdl_enabled();

// Kernel launch with the programmatic-dependent-launch attribute (see pdl_* in common.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace mx
