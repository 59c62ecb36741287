// TEST INFRASTRUCTURE - builds only where the reference tree is present.
//
// C entry points over the reference's prompt-lookup index, compiled from its own source where it lies in the reference
// tree (runtime/model/LookupProposals.cpp with runtime/model/LookupProposals.hpp); no reference source is copied. The
// result, oracle/_ref/libsplash_ref_lookup.so, lets the CPU tests hold the library's index against the reference's after
// every token, and lets the script under tests/golden/ write vectors from it.
#include "model/LookupProposals.hpp"

#include <cstdint>
#include <span>

#define REF_API extern "C" __attribute__((visibility("default")))

using splash::model::LookupIndex;

REF_API void *ref_lookup_create() { return new LookupIndex(); }
REF_API void ref_lookup_destroy(void *index) { delete static_cast<LookupIndex *>(index); }
REF_API void ref_lookup_append(void *index, const uint32_t *tokens, uint64_t count) {
  static_cast<LookupIndex *>(index)->append(std::span<const uint32_t>(tokens, size_t(count)));
}
REF_API void ref_lookup_match(void *index, uint32_t *length, uint32_t *end) {
  const LookupIndex::Match m = static_cast<LookupIndex *>(index)->match();
  *length = m.length, *end = m.end;
}
REF_API uint32_t ref_lookup_proposals(void *index, uint32_t count, uint32_t *out) {
  const std::span<const uint32_t> p = static_cast<LookupIndex *>(index)->proposals(count);
  for (size_t i = 0; i < p.size(); ++i) out[i] = p[i];
  return uint32_t(p.size());
}
// Appends the tokens one by one and records the match after each: lengths and ends of `count` words.
REF_API void ref_lookup_trace(const uint32_t *tokens, uint64_t count, uint32_t *lengths, uint32_t *ends) {
  LookupIndex index;
  for (uint64_t i = 0; i < count; ++i) {
    index.append(std::span<const uint32_t>(tokens + i, 1));
    lengths[i] = index.match().length, ends[i] = index.match().end;
  }
}
