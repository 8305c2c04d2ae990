// Host-side declarations shared between the kernel translation units.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace mx {
int* status_word();
int sm_count();
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, int swizzle128);
}  // namespace mx
