// TEST INFRASTRUCTURE - builds only where the reference tree is present.
//
// C entry points over the reference's own CPU test references, compiled from the headers where
// they lie in the reference tree (dev/tests/engine/GgufFormatReference.hpp,
// dev/tests/engine/Q8PageFormatReference.hpp, dev/tests/engine/PenaltyReference.hpp); no reference source is copied. The result,
// oracle/_ref/libsplash_ref.so, lets the tests compare the oracle's restatement bit for bit
// with the reference's code and lets the fixture script under tests/golden/ emit vectors.
#include "GgufFormatReference.hpp"
#include "Q8PageFormatReference.hpp"
#include "PenaltyReference.hpp"

#include <cstdint>
#include <random>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

using namespace gguf_reference;

// rowValues over `rows` native rows (GgufFormatReference.hpp:643-646).
REF_API int ref_row_values(uint32_t fmt, const uint8_t *native, uint32_t rows, uint32_t K, float *out) {
  if (fmt >= FMT_COUNT) return -1;
  const uint32_t rb = rowBytes(Fmt(fmt), K);
  for (uint32_t r = 0; r < rows; ++r) rowValues(Fmt(fmt), native + size_t(r) * rb, K, out + size_t(r) * K);
  return 0;
}

// The fixture behind the golden hashes, by the recipe of dev/tests/engine/GgufFixtures.hpp:148-165
// for a GGUF block format: makeNative with every half scale a random finite half.
REF_API int ref_fixture(uint32_t fmt, uint32_t rows, uint32_t K, uint32_t seed, uint8_t *out) {
  if (fmt >= FMT_COUNT) return -1;
  std::mt19937 rng(seed);
  const std::vector<uint8_t> v = makeNative(Fmt(fmt), rows, K, rng, [&] {
    uint16_t h;
    do h = static_cast<uint16_t>(rng());
    while ((h & 0x7C00) == 0x7C00);
    return h;
  });
  memcpy(out, v.data(), v.size());
  return 0;
}

// makeNative with the format's realistic scale range (GgufFormatReference.hpp:292-324).
REF_API int ref_realistic(uint32_t fmt, uint32_t rows, uint32_t K, uint32_t seed, uint8_t *out) {
  if (fmt >= FMT_COUNT) return -1;
  std::mt19937 rng(seed);
  const std::vector<uint8_t> v = makeNative(Fmt(fmt), rows, K, rng);
  memcpy(out, v.data(), v.size());
  return 0;
}

REF_API uint32_t ref_row_bytes(uint32_t fmt, uint32_t K) { return fmt < FMT_COUNT ? rowBytes(Fmt(fmt), K) : 0; }

// dot + projectionBound (GgufFormatReference.hpp:711-742) of one bf16-valued input row against one weight row.
REF_API void ref_projection(const float *x, const float *w, uint32_t K, double *value, double *exact, double *staged) {
  const Dot d = dot(x, w, K);
  *value = d.value;
  *exact = projectionBound(d, false);
  *staged = projectionBound(d, true);
}

// The INT8 KV quantizer's scale and code of one value at its row's largest magnitude
// (Q8PageFormatReference.hpp:107-119).
REF_API float ref_kv_scale(float maximum) { return splash::kv::reference_detail::storedScale(maximum); }
REF_API int ref_kv_code(float value, float maximum) { return splash::kv::reference_detail::quantize(value, maximum); }

// The sampling penalties' arithmetic on one logit (PenaltyReference.hpp:28-40).
REF_API float ref_penalty(float value, uint32_t count, int prompt, float repetition, float presence, float frequency) {
  splash::ops::SamplingPenalties p;
  p.repetition = repetition, p.presence = presence, p.frequency = frequency;
  return splash::test::referencePenalty(value, count, prompt != 0, p);
}
