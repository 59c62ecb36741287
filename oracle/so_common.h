// TEST INFRASTRUCTURE - CPU oracle of the DFlash2 verify step. Never linked into the product
// library; only tests, the smoke check and the benchmark's CPU-baseline leg load it.
//
// Scalar helpers shared by the oracle's translation units: bf16 / fp16 conversions (round to
// nearest even, as the reference's kernels and CPU tests convert:
// dev/tests/engine/LinearNumerics.hpp:11-20, dev/tests/engine/GgufFormatReference.hpp:44-45,223-227)
// and the activation functions of runtime/metal/kernels/common/activation.h:8-16.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace so {

inline float bf2f(uint16_t u) {
  const uint32_t v = uint32_t(u) << 16;
  float f;
  memcpy(&f, &v, 4);
  return f;
}
// Nearest, ties to even; NaN keeps a quiet payload.
inline uint16_t f2bf(float f) {
  uint32_t v;
  memcpy(&v, &f, 4);
  if ((v & 0x7f800000u) == 0x7f800000u && (v & 0x007fffffu)) return uint16_t((v >> 16) | 0x40);
  return uint16_t((v + 0x7fffu + ((v >> 16) & 1u)) >> 16);
}
inline float rbf(float f) { return bf2f(f2bf(f)); }
inline float h2f(uint16_t u) {
  _Float16 h;
  memcpy(&h, &u, 2);
  return float(h);
}
inline uint16_t f2h(float f) {
  const _Float16 h = _Float16(f);
  uint16_t u;
  memcpy(&u, &h, 2);
  return u;
}
inline float rh(float f) { return h2f(f2h(f)); }

// e^-x taken as exp2(-x log2 e), as every kernel of the reference evaluates SiLU and the sigmoid.
inline float silu(float x) { return x / (1.0f + exp2f(-1.44269504089f * x)); }
inline float sigmoid(float x) { return 1.0f / (1.0f + exp2f(-1.44269504089f * x)); }

constexpr float kRmsEps = 1e-6f;

}  // namespace so

#define SO_API extern "C" __attribute__((visibility("default")))
