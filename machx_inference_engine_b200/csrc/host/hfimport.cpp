// Hugging Face checkpoint ingestion, host side: a memory-mapped safetensors reader and the 4-bit AWQ / GPTQ
// decoders that feed `ie import` (reference parity: src/loaders/safetensors_reader.cpp, src/loaders/awq.cpp).
//
// Decoders write fp32 in [out_features][in_features] order -- the row-major layout a GGUF tensor wants (input dimension
// contiguous) -- so the importer can hand each matrix straight to the block quantisers; rows are split over threads.
//   AWQ  ("gemm" packing): qweight int32 [in, out/8], qzeros int32 [in/G, out/8], scales fp16 [in/G, out];
//        logical column j of a packed word sits at bit 4*{0,4,1,5,2,6,3,7}[j];  w = (q - z) * s
//   GPTQ: qweight int32 [in/8, out] (nibble i%8 along the input axis), qzeros int32 [groups, out/8] (natural order),
//        scales fp16 [groups, out], optional g_idx[in];  w = (q - (z + 1)) * s
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_st_err;

struct StFile {
  int fd = -1; void* base = MAP_FAILED; size_t size = 0; uint64_t header_len = 0;
  ~StFile() { if (base != MAP_FAILED) munmap(base, size); if (fd >= 0) close(fd); }
};

inline float half_to_float(uint16_t h) {
  const uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF;
  uint32_t bits;
  if (e == 0) {
    if (m == 0) bits = s;
    else { int sh = 0; uint32_t mm = m; while (!(mm & 0x400)) { mm <<= 1; ++sh; } bits = s | ((127 - 15 - sh + 1) << 23) | ((mm & 0x3FF) << 13); }
  } else if (e == 31) bits = s | 0x7F800000u | (m << 13);
  else bits = s | ((e - 15 + 127) << 23) | (m << 13);
  float f; memcpy(&f, &bits, 4); return f;
}

template <class F> void parallel_rows(int64_t n, int nthreads, F fn) {
  nthreads = std::max(1, std::min<int>(nthreads, (int)std::min<int64_t>(n, 64)));
  if (nthreads == 1) { fn(0, n); return; }
  std::vector<std::thread> th;
  const int64_t per = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    const int64_t lo = t * per, hi = std::min(n, lo + per);
    if (lo < hi) th.emplace_back([=] { fn(lo, hi); });
  }
  for (auto& t : th) t.join();
}

constexpr int kAwqNibble[8] = {0, 4, 1, 5, 2, 6, 3, 7};

}  // namespace

extern "C" {

const char* mx_st_last_error() { return g_st_err.c_str(); }

void* mx_st_open(const char* path) {
  StFile* f = new StFile();
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) { g_st_err = std::string("safetensors: cannot open ") + path; delete f; return nullptr; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) { g_st_err = std::string("safetensors: file too small: ") + path; delete f; return nullptr; }
  f->size = (size_t)st.st_size;
  f->base = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (f->base == MAP_FAILED) { g_st_err = std::string("safetensors: mmap failed: ") + path; delete f; return nullptr; }
  memcpy(&f->header_len, f->base, 8);                     // unaligned-safe
  if (f->header_len == 0 || f->header_len > f->size - 8 || f->header_len > (1ull << 30)) {
    g_st_err = std::string("safetensors: bad header length in ") + path; delete f; return nullptr;
  }
  return f;
}
const char* mx_st_header(void* h) { return (const char*)((StFile*)h)->base + 8; }
uint64_t mx_st_header_len(void* h) { return ((StFile*)h)->header_len; }
const void* mx_st_data(void* h) { StFile* f = (StFile*)h; return (const char*)f->base + 8 + f->header_len; }
uint64_t mx_st_data_len(void* h) { StFile* f = (StFile*)h; return f->size - 8 - f->header_len; }
void mx_st_close(void* h) { delete (StFile*)h; }

int mx_awq_dequant(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, int64_t in_f, int64_t out_f, int64_t group,
                   float* w_out, int nthreads) {
  if (out_f % 8 || group <= 0 || in_f % group) { g_st_err = "awq: out_features must be a multiple of 8 and in_features of group_size"; return -1; }
  const int64_t pc = out_f / 8;
  parallel_rows(out_f, nthreads, [=](int64_t lo, int64_t hi) {
    for (int64_t o = lo; o < hi; ++o) {
      const int64_t c = o >> 3;
      const int sh = 4 * kAwqNibble[o & 7];
      float* dst = w_out + o * in_f;
      for (int64_t g = 0; g < in_f / group; ++g) {
        uint32_t zw; memcpy(&zw, qzeros + g * pc + c, 4);
        const int z = (zw >> sh) & 0xF;
        uint16_t sb; memcpy(&sb, scales + g * out_f + o, 2);
        const float s = half_to_float(sb);
        for (int64_t i = g * group; i < (g + 1) * group; ++i) {
          uint32_t qw; memcpy(&qw, qweight + i * pc + c, 4);
          dst[i] = float(int((qw >> sh) & 0xF) - z) * s;
        }
      }
    }
  });
  return 0;
}

int mx_gptq_dequant(const int32_t* qweight, const int32_t* qzeros, const uint16_t* scales, const int32_t* g_idx, int64_t in_f, int64_t out_f,
                    int64_t group, float* w_out, int nthreads) {
  if (in_f % 8 || out_f % 8 || group <= 0) { g_st_err = "gptq: in/out features must be multiples of 8"; return -1; }
  const int64_t zc = out_f / 8;
  parallel_rows(out_f, nthreads, [=](int64_t lo, int64_t hi) {
    for (int64_t o = lo; o < hi; ++o) {
      const int osh = int(o & 7) * 4;
      float* dst = w_out + o * in_f;
      for (int64_t i = 0; i < in_f; ++i) {
        int32_t gi = int32_t(i / group);
        if (g_idx) memcpy(&gi, g_idx + i, 4);
        uint32_t qw, zw; uint16_t sb;
        memcpy(&qw, qweight + (i >> 3) * out_f + o, 4);
        memcpy(&zw, qzeros + (int64_t)gi * zc + (o >> 3), 4);
        memcpy(&sb, scales + (int64_t)gi * out_f + o, 2);
        const int q = (qw >> (int(i & 7) * 4)) & 0xF, z = ((zw >> osh) & 0xF) + 1;
        dst[i] = float(q - z) * half_to_float(sb);
      }
    }
  });
  return 0;
}

}  // extern "C"
