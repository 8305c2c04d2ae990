// EXL3 weights on the host: trellis decode and the 128-point Hadamard transform.
//
// An EXL3 linear layer stores, per 16 x 16 tile of the (rotated) weight matrix W_rot[K][N], a cyclic bit stream of
// 256 * bits bits (16 * bits int16 words).  Weight t of a tile (t = 0..255) is the 16-bit window of that stream that ends
// at bit (t + 1) * bits, counted from the most significant bit of 32-bit words formed from consecutive int16 pairs
// (low word first); windows that start before bit 0 wrap to the end of the tile's stream.  The window is hashed
// (multiply-add, mask, xor) into two fp16 bit patterns whose sum, rounded to fp16, is the weight: a procedural codebook
// with roughly Gaussian values.  The 256 weights of a tile come out in the order a 16x8x16 tensor-core fragment holds
// them (lane l, register j -> t = 8 l + j) and are put back to row-major here.  Around the matrix product the layer
// applies y = had128(had128(x * suh) W_rot) * svh with per-feature sign-and-scale vectors and a block-diagonal, normalised
// 128-point Sylvester Hadamard transform.
//
// Reference parity: src/core/exl3_decode.cpp (decode), src/ops/hadamard.cpp:36 (transform), include/ie/exl3.hpp.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "quant.h"

namespace mx {
namespace {

// position (row * 16 + col) inside the tile of weight t: lane l = t / 8 owns rows {2 (l % 4), +1, +8, +9} of columns
// {l / 4, l / 4 + 8}; its eight values run over the four rows of the first column, then of the second
inline int exl3_tile_pos(int t) {
  const int l = t >> 3, j = t & 7;
  const int row = (l & 3) * 2 + (j & 1) + ((j >> 1) & 1) * 8;
  const int col = (l >> 2) + (j >> 2) * 8;
  return row * 16 + col;
}

inline float exl3_code_value(uint32_t code) {
  uint32_t x = code * 89226354u + 64248484u;
  x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
  // both halves have exponents 12..15, so their fp32 sum is exact and one rounding to fp16 follows
  const float s = fp16_to_fp32((uint16_t)(x & 0xffffu)) + fp16_to_fp32((uint16_t)(x >> 16));
  return fp16_to_fp32(fp32_to_fp16(s));
}

}  // namespace
}  // namespace mx

extern "C" {

// out: W_rot as [K][N] (transpose == 0) or [N][K] (transpose != 0), K = 16 tile_k, N = 16 tile_n.
int mx_exl3_decode(const uint16_t* trellis, uint32_t tile_k, uint32_t tile_n, uint32_t bits, float* out, int transpose, int nthreads) {
  using namespace mx;
  if (!trellis || !out || bits < 1 || bits > 8) return 1;
  const uint32_t K = tile_k * 16, N = tile_n * 16;
  const uint32_t nwords = bits * 8;                    // 32-bit words per tile
  const uint32_t nbits = bits * 256;
  // per weight: the two words that hold its window and the shift that brings the window to the low 16 bits
  struct Win { uint16_t w0, w1, shift, pos; };
  Win win[256];
  for (int t = 0; t < 256; ++t) {
    const uint32_t end = ((uint32_t)(t + 1) * bits + nbits) % nbits;        // one past the window's last bit, cyclic
    const uint32_t last = (end + nbits - 1) % nbits, first = (end + nbits - 16) % nbits;
    win[t].w0 = (uint16_t)(first / 32);
    win[t].w1 = (uint16_t)(last / 32);
    win[t].shift = (uint16_t)(31 - last % 32);
    win[t].pos = (uint16_t)exl3_tile_pos(t);
  }
  std::vector<float> lut(65536);
  for (uint32_t c = 0; c < 65536; ++c) lut[c] = exl3_code_value(c);
  auto work = [&](uint32_t k_lo, uint32_t k_hi) {
    std::vector<uint32_t> w(nwords);
    for (uint32_t ki = k_lo; ki < k_hi; ++ki)
      for (uint32_t ni = 0; ni < tile_n; ++ni) {
        const uint16_t* tile = trellis + ((size_t)ki * tile_n + ni) * (16 * bits);
        for (uint32_t j = 0; j < nwords; ++j) w[j] = (uint32_t)tile[2 * j] | ((uint32_t)tile[2 * j + 1] << 16);
        for (int t = 0; t < 256; ++t) {
          const uint64_t pair = ((uint64_t)w[win[t].w0] << 32) | w[win[t].w1];
          // (w0 == w1 when the window lies inside one word: the high copy is shifted out by the mask)
          const uint32_t code = (uint32_t)(pair >> win[t].shift) & 0xffffu;
          const int r = win[t].pos >> 4, c = win[t].pos & 15;
          const size_t k = (size_t)ki * 16 + r, n = (size_t)ni * 16 + c;
          out[transpose ? n * K + k : k * N + n] = lut[code];
        }
      }
  };
  int nt = nthreads > 0 ? nthreads : (int)std::thread::hardware_concurrency();
  if (nt < 1) nt = 1;
  if ((uint32_t)nt > tile_k) nt = (int)tile_k;
  if (nt <= 1) { work(0, tile_k); return 0; }
  std::vector<std::thread> th;
  for (int i = 0; i < nt; ++i) th.emplace_back(work, (uint32_t)((uint64_t)tile_k * i / nt), (uint32_t)((uint64_t)tile_k * (i + 1) / nt));
  for (auto& t : th) t.join();
  return 0;
}

// In place: every aligned run of 128 elements along the last dimension of x[rows][n] becomes its normalised Sylvester Hadamard transform.
int mx_hadamard128(float* x, uint64_t rows, uint64_t n) {
  if (!x || n % 128) return 1;
  const float norm = 0.08838834764831845f;     // 1 / sqrt(128)
  for (uint64_t r = 0; r < rows; ++r)
    for (uint64_t b = 0; b < n; b += 128) {
      float* v = x + r * n + b;
      for (int len = 1; len < 128; len <<= 1)
        for (int i = 0; i < 128; ++i)
          if (!(i & len)) {
            const float a = v[i], c = v[i | len];
            v[i] = a + c;
            v[i | len] = a - c;
          }
      for (int i = 0; i < 128; ++i) v[i] *= norm;
    }
  return 0;
}

}  // extern "C"
