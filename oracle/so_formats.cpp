// TEST INFRASTRUCTURE - CPU oracle, not part of the product library.
//
// GGUF native blocks and their fp32 values (llama.cpp dequantize_row_* semantics, pinned at
// llama.cpp 7ab4ee7 by the reference), restated from the reference's CPU twin
// dev/tests/engine/GgufFormatReference.hpp:326-329 (scale_min_k4), :370-381 (Q4_K),
// :418-432 (Q6_K), :453-458 (Q8_0) and runtime/metal/kernels/common/quant_formats.h:474-487
// (NVFP4), plus the fixture recipe behind the reference's SHA-256 goldens
// (dev/tests/engine/GgufFixtures.hpp:148-165, GgufFormatReference.hpp:196-219,
// dev/tests/engine/gguf_reference_test.mm:21-30).
//
// Parity pin: tests hash so_golden_fixture + so_dequant output against
// tests/golden/weight_goldens.json (copied hashes of dev/tests/fixtures/weight-goldens/goldens.json)
// and, where the reference tree is present, compare bit-for-bit with the reference header itself
// compiled into oracle/_ref (oracle/ref_shim.cpp).
#include "so_common.h"

#include <algorithm>
#include <random>
#include <vector>

namespace so {

enum Fmt : uint32_t { Q4K = 0, Q6K = 4, Q80 = 6, NVFP4 = 37, BF16 = 41, F16 = 42, F32 = 64 };

struct FmtInfo {
  uint32_t block_elements, block_bytes;
};
inline bool fmt_info(uint32_t f, FmtInfo &i) {
  switch (f) {
    case Q4K: i = {256, 144}; return true;
    case Q6K: i = {256, 210}; return true;
    case Q80: i = {32, 34}; return true;
    case NVFP4: i = {256, 148}; return true;
    case BF16: case F16: i = {1, 2}; return true;
    case F32: i = {1, 4}; return true;
  }
  return false;
}

inline void scale_min_k4(const uint8_t *sc, int j, uint8_t &s, uint8_t &m) {
  if (j < 4) {
    s = sc[j] & 63;
    m = sc[j + 4] & 63;
  } else {
    s = uint8_t((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4));
    m = uint8_t((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
  }
}

// E4M3 byte value; bias 7, subnormals below exponent 1 (GgufFormatReference.hpp:72-77).
inline float e4m3(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  const float mag = e ? std::ldexp(1.0f + m / 8.0f, e - 7) : std::ldexp(m / 8.0f, -6);
  return (b & 0x80) ? -mag : mag;
}
// 2 x E2M1 (runtime/metal/abi/QuantTables.h:842).
static const float kFP4Values[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// fp32 values of one native block (block_elements of them).
void block_values(uint32_t f, const uint8_t *blk, float *out) {
  switch (f) {
    case Q4K: {
      uint16_t d16, m16;
      memcpy(&d16, blk, 2);
      memcpy(&m16, blk + 2, 2);
      const float d = h2f(d16), dmin = h2f(m16);
      for (int j = 0; j < 8; ++j) {
        uint8_t sc, mn;
        scale_min_k4(blk + 4, j, sc, mn);
        const uint8_t *q = blk + 16 + (j / 2) * 32;
        const int sh = (j % 2) * 4;
        for (int k = 0; k < 32; ++k) {
          const uint8_t code = (q[k] >> sh) & 15;
          // Left to right in fp32, as the reference writes it; every product is exact, so this is
          // the single rounding of d*sc*code - dmin*mn.
          out[32 * j + k] = d * sc * code - dmin * mn;
        }
      }
      return;
    }
    case Q6K: {
      uint16_t d16;
      memcpy(&d16, blk + 208, 2);
      const float d = h2f(d16);
      const int8_t *scales = reinterpret_cast<const int8_t *>(blk + 192);
      for (int j = 0; j < 8; ++j) {
        const int n = j / 4, r = j % 4;
        const uint8_t *ql = blk + 64 * n, *qh = blk + 128 + 32 * n;
        for (int k = 0; k < 32; ++k) {
          const uint8_t l4 = (ql[k + 32 * (r & 1)] >> (4 * (r >> 1))) & 15, h2 = (qh[k] >> (2 * r)) & 3;
          const int q6 = int(l4 | (h2 << 4)) - 32;
          out[32 * j + k] = d * scales[8 * n + 2 * r + k / 16] * q6;
        }
      }
      return;
    }
    case Q80: {
      uint16_t d16;
      memcpy(&d16, blk, 2);
      const int8_t *qs = reinterpret_cast<const int8_t *>(blk + 2);
      for (int k = 0; k < 32; ++k) out[k] = h2f(d16) * qs[k];
      return;
    }
    case NVFP4: {
      float g;
      memcpy(&g, blk + 16, 4);
      for (int e = 0; e < 256; ++e) {
        const uint8_t code = (blk[20 + e / 2] >> (4 * (e % 2))) & 15;
        // value = T[code] * ((e4m3 / 256) * (128 g)), the kernels' order.
        const float s = (e4m3(blk[e / 16]) * (1.0f / 256.0f)) * (128.0f * g);
        out[e] = kFP4Values[code] * s;
      }
      return;
    }
  }
}

}  // namespace so

using namespace so;

// Bytes of one row of K weights in format f; 0 for an unknown format or a K that is not whole blocks.
SO_API uint64_t so_row_bytes(uint32_t f, uint32_t K) {
  FmtInfo i;
  if (!fmt_info(f, i) || K % i.block_elements) return 0;
  return uint64_t(K / i.block_elements) * i.block_bytes;
}

// fp32 values of `rows` native rows of K weights each.
SO_API int so_dequant(uint32_t f, const uint8_t *native, uint32_t rows, uint32_t K, float *out) {
  FmtInfo i;
  if (!fmt_info(f, i) || K % i.block_elements) return -1;
  const uint64_t rb = so_row_bytes(f, K);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < int64_t(rows); ++r) {
    const uint8_t *row = native + r * rb;
    float *o = out + uint64_t(r) * K;
    if (f == F32) { memcpy(o, row, size_t(K) * 4); continue; }
    if (f == BF16 || f == F16) {
      for (uint32_t k = 0; k < K; ++k) {
        uint16_t u;
        memcpy(&u, row + 2 * k, 2);
        o[k] = f == BF16 ? bf2f(u) : h2f(u);
      }
      continue;
    }
    for (uint32_t b = 0; b < K / i.block_elements; ++b)
      block_values(f, row + uint64_t(b) * i.block_bytes, o + uint64_t(b) * i.block_elements);
  }
  return 0;
}

// The fixture the reference's golden hashes are taken over: every byte of the rows drawn from
// std::mt19937(seed) as (uint8_t)rng(), then per block its half scale(s) replaced by a random
// finite half (redrawn while Inf/NaN); Q4_K draws d then dmin. NVFP4 is not hashed upstream.
SO_API int so_golden_fixture(uint32_t f, uint32_t rows, uint32_t K, uint32_t seed, uint8_t *out) {
  FmtInfo i;
  if (!(f == Q4K || f == Q6K || f == Q80) || !fmt_info(f, i) || K % i.block_elements) return -1;
  std::mt19937 rng(seed);
  const uint64_t bytes = uint64_t(rows) * so_row_bytes(f, K);
  for (uint64_t b = 0; b < bytes; ++b) out[b] = uint8_t(rng());
  const uint32_t off = f == Q6K ? 208 : 0;
  auto finite_half = [&] {
    uint16_t h;
    do h = uint16_t(rng());
    while ((h & 0x7C00) == 0x7C00);
    return h;
  };
  for (uint64_t b = 0; b < bytes / i.block_bytes; ++b) {
    uint8_t *blk = out + b * i.block_bytes;
    const uint16_t d = finite_half();
    memcpy(blk + off, &d, 2);
    if (f == Q4K) {
      const uint16_t m = finite_half();
      memcpy(blk + off + 2, &m, 2);
    }
  }
  return 0;
}
