// Per-element value of a GGUF native row on the device (shared by the dequantization kernel and the
// embedding gather): the single fp32 rounding of each format's defining expression.
#pragma once
#include "sb_internal.h"
#include "sb_ptx.cuh"

namespace sb {

__device__ __forceinline__ float half_bits_to_float(uint32_t b) { return __half2float(__ushort_as_half(uint16_t(b))); }

__device__ __forceinline__ float e4m3_value(uint32_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  const float mag = e ? ldexpf(1.0f + m * 0.125f, e - 7) : ldexpf(m * 0.125f, -6);
  return (b & 0x80) ? -mag : mag;
}

static __constant__ float kFP4Values[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// Value of weight `c` of the native row at `row`.
__device__ __forceinline__ float weight_value(uint32_t format, const uint8_t *row, uint32_t c) {
  float v = 0.0f;
  if (format == SB_FMT_Q4K) {
    const uint8_t *blk = row + (c / 256) * 144;
    const uint32_t e = c % 256, j = e / 32, kk = e % 32;
    const float d = half_bits_to_float(blk[0] | (blk[1] << 8)), dmin = half_bits_to_float(blk[2] | (blk[3] << 8));
    const uint8_t *s = blk + 4;
    uint32_t sc, mn;
    if (j < 4) {
      sc = s[j] & 63;
      mn = s[j + 4] & 63;
    } else {
      sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
      mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
    const uint32_t code = (blk[16 + (j / 2) * 32 + kk] >> ((j % 2) * 4)) & 15;
    v = __fmaf_rn(float(code), d * float(sc), -(dmin * float(mn)));
  } else if (format == SB_FMT_Q6K) {
    const uint8_t *blk = row + (c / 256) * 210;
    const uint32_t e = c % 256, j = e / 32, kk = e % 32, n = j / 4, rr = j % 4;
    const float d = half_bits_to_float(blk[208] | (blk[209] << 8));
    const uint32_t l4 = (blk[64 * n + kk + 32 * (rr & 1)] >> (4 * (rr >> 1))) & 15;
    const uint32_t h2 = (blk[128 + 32 * n + kk] >> (2 * rr)) & 3;
    const int q6 = int(l4 | (h2 << 4)) - 32;
    const int sc = int(int8_t(blk[192 + 8 * n + 2 * rr + kk / 16]));
    v = __fmul_rn(__fmul_rn(d, float(sc)), float(q6));
  } else if (format == SB_FMT_Q80) {
    const uint8_t *blk = row + (c / 32) * 34;
    v = __fmul_rn(half_bits_to_float(blk[0] | (blk[1] << 8)), float(int(int8_t(blk[2 + c % 32]))));
  } else if (format == SB_FMT_NVFP4) {
    const uint8_t *blk = row + (c / 256) * 148;
    const uint32_t e = c % 256;
    const float g = __uint_as_float(blk[16] | (blk[17] << 8) | (blk[18] << 16) | (uint32_t(blk[19]) << 24));
    const uint32_t code = (blk[20 + e / 2] >> (4 * (e % 2))) & 15;
    const float s = __fmul_rn(__fmul_rn(e4m3_value(blk[e / 16]), 1.0f / 256.0f), __fmul_rn(128.0f, g));
    v = __fmul_rn(kFP4Values[code], s);
  }
  return v;
}

}  // namespace sb
