// Host-side plumbing shared by the kernel files: the per-device status word and the
// tensor-map (TMA descriptor) encoder obtained from the driver at run time.
#include "common.cuh"
#include "host_util.h"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace mx {

static std::mutex g_mu;
static int* g_status[64] = {nullptr};
static int g_sm_count[64] = {0};

int* status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    cudaMalloc(&g_status[dev], 64);
    cudaMemset(g_status[dev], 0, 64);
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_sm_count[dev]) cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  return g_sm_count[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static EncodeTiledFn encoder() {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return nullptr;
    g_encode = (EncodeTiledFn)fn;
  }
  return g_encode;
}

// bf16 tensor of `rank` dims (dims[0] innermost), byte strides for dims 1.., box in elements.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, int swizzle128) {
  EncodeTiledFn enc = encoder();
  if (!enc) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, b, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Bytes as a 2-D tensor of 8-byte elements: rows of `row_bytes` (a multiple of 8) `row_stride` bytes apart (a multiple of 16), box of
// box_bytes x box_rows, no swizzle: the tile lands in shared memory as box_rows dense rows of box_bytes.
int make_tmap_bytes(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t row_stride, uint32_t box_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return -1;
  if (row_bytes % 8 || box_bytes % 16 || box_bytes / 8 > 256 || box_rows > 256 || row_stride % 16 || ((uintptr_t)base & 15)) return -2;
  cuuint64_t gdim[2] = {row_bytes / 8, rows};
  cuuint64_t gstr[1] = {row_stride};
  cuuint32_t b[2] = {box_bytes / 8, box_rows}, es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), gdim, gstr, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }
}  // namespace mx

// Reads the status word of the current device and clears it.  Synchronises the device.
MX_HOST_API int mx_status_read_and_clear() {
  int* p = mx::status_word();
  int v = 0;
  cudaDeviceSynchronize();
  cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (v) cudaMemset(p, 0, sizeof(int));
  return v;
}

MX_HOST_API int mx_sm_count() { return mx::sm_count(); }

MX_HOST_API const char* mx_cuda_last_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

// Programmatic dependent launch for the decode-chain kernels (default on; measured 4.26 -> 4.02 ms per gpt-oss-120b token);
// off = plain stream order.
MX_HOST_API void mx_set_pdl(int on) { mx::set_pdl(on != 0); }
