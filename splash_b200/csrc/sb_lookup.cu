// C ABI of the prompt-lookup index (include/splash_b200.h, "prompt lookup"): host code, no device needed.
#include <memory>
#include <new>

#include "model/PromptLookup.hpp"
#include "sb_internal.h"

using splash::b200::model::LookupIndex;

extern "C" {

int sb_lookup_create(void **out_index) {
  if (!out_index) return sb::fail(SB_ERR_INVALID, "sb_lookup_create: null pointer");
  LookupIndex *index = new (std::nothrow) LookupIndex();
  if (!index) return sb::fail(SB_ERR_OOM, "sb_lookup_create: out of host memory");
  *out_index = index;
  return SB_OK;
}
int sb_lookup_destroy(void *index) {
  delete static_cast<LookupIndex *>(index);
  return SB_OK;
}
int sb_lookup_append(void *index, const uint32_t *tokens, uint64_t count) {
  if (!index || (count && !tokens)) return sb::fail(SB_ERR_INVALID, "sb_lookup_append: null pointer");
  LookupIndex &l = *static_cast<LookupIndex *>(index);
  if (l.tokens().size() + count >= UINT32_MAX) return sb::fail(SB_ERR_INVALID, "sb_lookup_append: more than 2^32 - 1 tokens");
  try {
    l.append(tokens, size_t(count));
  } catch (const std::bad_alloc &) {
    return sb::fail(SB_ERR_OOM, "sb_lookup_append: out of host memory");
  }
  return SB_OK;
}
int sb_lookup_match(void *index, uint32_t *out_length, uint32_t *out_end) {
  if (!index || !out_length || !out_end) return sb::fail(SB_ERR_INVALID, "sb_lookup_match: null pointer");
  const LookupIndex::Match m = static_cast<LookupIndex *>(index)->match();
  *out_length = m.length, *out_end = m.end;
  return SB_OK;
}
int sb_lookup_proposals(void *index, uint32_t count, uint32_t *out_tokens, uint32_t *out_count) {
  if (!index || !out_count || (count && !out_tokens)) return sb::fail(SB_ERR_INVALID, "sb_lookup_proposals: null pointer");
  const uint32_t *from = nullptr;
  const size_t n = static_cast<LookupIndex *>(index)->proposals(count, &from);
  for (size_t i = 0; i < n; ++i) out_tokens[i] = from[i];
  *out_count = uint32_t(n);
  return SB_OK;
}
int sb_lookup_size(void *index, uint64_t *out_tokens) {
  if (!index || !out_tokens) return sb::fail(SB_ERR_INVALID, "sb_lookup_size: null pointer");
  *out_tokens = static_cast<LookupIndex *>(index)->tokens().size();
  return SB_OK;
}
int sb_lookup_agreement(uint32_t token, uint32_t depth, const uint32_t *candidates, uint64_t count, uint32_t *out_agreement) {
  if (!out_agreement || (count && !candidates)) return sb::fail(SB_ERR_INVALID, "sb_lookup_agreement: null pointer");
  *out_agreement = splash::b200::model::lookupAgreement(token, depth, candidates, size_t(count));
  return SB_OK;
}

}  // extern "C"
