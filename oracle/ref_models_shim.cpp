// TEST INFRASTRUCTURE - builds only where the reference tree is present.
//
// C entry points over the fp64 CPU models that the reference's kernel tests check their kernels
// against:
//   attention   loadKey, loadValue, cpuReference      dev/tests/engine/q8_flash_attention_metal_test.mm
//   GDN         convolutionSilu, normalizedHead,      dev/tests/engine/gdn_decode_metal_test.mm
//               recurrence
//   selection   referenceDistribution (min_p, top_k,  dev/tests/engine/target_sampling_metal_test.mm
//               top_p), startOf, reject,
//               referenceSelection (child tests and the residual draw),
//               referenceBest / referenceArgmax (the greedy order)
//   RMSNorm     normWeight, rmsNorm, roundedOnceToBf16   dev/tests/engine/NormReference.hpp
// Those functions are plain C++ inside Objective-C++ test files. The build recipe (Makefile, target
// `ref`) cuts their text out of the files where they lie in the reference tree into a scratch folder that
// it deletes after the compile, and this file includes the cuts between stand-ins for the tests'
// fixture types (the members the functions read, nothing else). No reference source is committed; the
// result is oracle/_ref/libsplash_ref_models.so, which lets the CPU tests hold the oracle's attention and
// GDN restatements against the reference's own models.
#include "LinearNumerics.hpp"
#include "Q8PageFormatReference.hpp"
#include "metal/abi/ExecutionGeometry.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <array>
#include <limits>
#include <memory>
#include <numeric>
#include <span>
#include <string>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

// ---- attention -------------------------------------------------------------------------------------
namespace attention_model {
using namespace splash::kv;

constexpr uint32_t kQueryStride = kPageTokens;

struct Shape {
  uint32_t kvHeads, queryHeadsPerKvHead;
  uint32_t queryHeads() const { return kvHeads * queryHeadsPerKvHead; }
};
struct Sequence {
  uint32_t row_bound, committed_tokens;
};
struct Contents {
  void *contents;
};
struct TreeRow {
  uint32_t ancestors;
  uint16_t parent, depth;
};
// The cache as the caller holds it: [page][kv head][page token][dimension] codes, [page][kv head][page token]
// fp32 scales (the order of splash_kv_key_element and splash_kv_scale_element inside a page).
struct Pool {
  const int8_t *k, *v;
  const float *ks, *vs;
  uint32_t kvHeads;
  uint64_t valueElement(uint32_t head, uint32_t token, uint32_t dimension) const {
    return splash_kv_key_element(head, token, dimension);
  }
};
struct Case {
  Shape shape;
  Sequence params;
  Contents queries;
  const uint32_t *pageTable;
  const TreeRow *tree;  // null: a chain
  std::unique_ptr<Pool> pool;

  uint32_t token(uint32_t slot) const { return slot; }
  bool attends(uint32_t, uint32_t) const { return true; }
  bool onPath(uint32_t row, uint32_t token) const {
    return !tree || token < params.committed_tokens || ((tree[row].ancestors >> (token - params.committed_tokens)) & 1u);
  }
  // Rows of [row][query head][dimension], for queries and outputs alike.
  uint64_t queryIndex(uint32_t head, uint32_t row, uint32_t dimension) const {
    return (uint64_t{row} * shape.queryHeads() + head) * kHeadDimension + dimension;
  }
  template <typename T> T *slab(uint32_t tensor, uint32_t logicalPage) const {
    const uint64_t page = pageTable[logicalPage];
    const uint64_t scales = uint64_t{pool->kvHeads} * kPageTokens;
    const void *base = nullptr;
    switch (tensor) {
      case SPLASH_KV_KEYS: base = pool->k + page * scales * kHeadDimension; break;
      case SPLASH_KV_VALUES: base = pool->v + page * scales * kHeadDimension; break;
      case SPLASH_KV_KEY_SCALES: base = pool->ks + page * scales; break;
      default: base = pool->vs + page * scales; break;
    }
    return static_cast<T *>(const_cast<void *>(base));
  }
};
// Only the unquantized branch of the model calls these; the entry point below asks for the stored pages.
inline float keyPattern(uint32_t, uint32_t, uint32_t) { return 0.0f; }
inline float valuePattern(uint32_t, uint32_t, uint32_t) { return 0.0f; }

#include "attention_model.inc"
}  // namespace attention_model

REF_API uint32_t ref_attention_page_tokens() { return splash::kv::kPageTokens; }
REF_API uint32_t ref_attention_head_dim() { return splash::kv::kHeadDimension; }

// Rows of one sequence over its stored INT8 pages. queries, out: bf16 [rows][kv_heads * group][head dim];
// tree: 8 bytes a row (ancestors u32, parent u16, depth u16) or null. Returns 0, or -1 for a shape the
// model does not cover.
REF_API int ref_attention(const uint16_t *queries, const int8_t *k, const int8_t *v, const float *k_scales, const float *v_scales,
                          const uint32_t *page_table, uint32_t kv_heads, uint32_t group, uint32_t committed, uint32_t rows,
                          const void *tree, uint16_t *out) {
  using namespace attention_model;
  if (!rows || rows > kQueryStride || !kv_heads || !group) return -1;
  Case c;
  c.shape = {kv_heads, group};
  c.params = {rows, committed};
  c.queries.contents = const_cast<uint16_t *>(queries);
  c.pageTable = page_table;
  c.tree = static_cast<const TreeRow *>(tree);
  c.pool = std::make_unique<Pool>(Pool{k, v, k_scales, v_scales, kv_heads});
  const std::vector<BFloat16Bits> o = cpuReference(c, true);
  std::memcpy(out, o.data(), uint64_t{rows} * c.shape.queryHeads() * kHeadDimension * sizeof(uint16_t));
  return 0;
}

// ---- GDN -------------------------------------------------------------------------------------------
namespace gdn_model {
using namespace splash::test;

constexpr uint32_t kHeadDim = 128;
constexpr uint32_t kTaps = 4, kCarried = kTaps - 1;
constexpr double kQueryScale = 0.0078125, kKeyScale = 0.08838834765;

inline double roundBfloat(double value) { return bf16ToFloat(floatToBf16(static_cast<float>(value))); }
inline double sigmoid(double value) { return 1.0 / (1.0 + std::exp(-value)); }

struct GdnShape {
  uint32_t keyHeads, valueHeads, convolutionDimension, packedWidth;
};
struct Contents {
  const void *p;
  const void *contents() const { return p; }
};
struct StepInputs {
  std::vector<uint16_t> history;  // [kCarried][conv]
  std::vector<uint16_t> packed;   // [rows][packedWidth], the convolution's channels first
};
// One layer's tape of one step: rows of [k of every key head | v of every value head], decays, betas.
struct Fixture {
  GdnShape shape;
  Contents convWeights;
  const uint16_t *kv;
  const float *decay;
  const uint16_t *beta;
  const uint16_t *tapeKv(uint64_t, uint32_t, uint32_t token) const {
    return kv + uint64_t{token} * (shape.convolutionDimension - shape.keyHeads * kHeadDim);
  }
  const float *tapeDecay(uint64_t, uint32_t, uint32_t token) const { return decay + uint64_t{token} * shape.valueHeads; }
  const uint16_t *tapeBeta(uint64_t, uint32_t, uint32_t token) const { return beta + uint64_t{token} * shape.valueHeads; }
};

#include "gdn_model.inc"
}  // namespace gdn_model

// The rows' q (scaled), k (scaled) and v after convolution, SiLU and the heads' RMS norm, as the model has
// them before the kernel's last rounding. history: bf16 [3][conv]; packed: bf16 [rows][packed_width];
// conv_w: bf16 [conv][4]. q, k: f64 [rows][key_heads * 128]; v: f64 [rows][value_heads * 128].
REF_API int ref_gdn_rows(const uint16_t *history, const uint16_t *packed, uint32_t packed_width, const uint16_t *conv_w, uint32_t rows,
                         uint32_t key_heads, uint32_t value_heads, double *q, double *k, double *v) {
  using namespace gdn_model;
  const uint32_t kw = key_heads * kHeadDim, vw = value_heads * kHeadDim, conv = 2 * kw + vw;
  if (packed_width < conv) return -1;
  Fixture f{};
  f.shape = {key_heads, value_heads, conv, packed_width};
  f.convWeights.p = conv_w;
  StepInputs step;
  step.history.assign(history, history + uint64_t{kCarried} * conv);
  step.packed.assign(packed, packed + uint64_t{rows} * packed_width);
  for (uint32_t token = 0; token < rows; ++token) {
    for (uint32_t head = 0; head < key_heads; ++head) {
      const std::vector<double> qr = normalizedHead(f, step, token, head * kHeadDim, kQueryScale);
      const std::vector<double> kr = normalizedHead(f, step, token, kw + head * kHeadDim, kKeyScale);
      std::copy(qr.begin(), qr.end(), q + uint64_t{token} * kw + head * kHeadDim);
      std::copy(kr.begin(), kr.end(), k + uint64_t{token} * kw + head * kHeadDim);
    }
    for (uint32_t channel = 0; channel < vw; ++channel) v[uint64_t{token} * vw + channel] = convolutionSilu(f, step, token, 2 * kw + channel);
  }
  return 0;
}

// The delta rule over `tokens` tape rows from `state` (f32 [value_heads][128][128]) for every value head.
// tape_kv: bf16 [tokens][key_heads * 128 + value_heads * 128]; decay: f32 [tokens][value_heads]; beta: bf16
// likewise. state_out: f64 like state. With history/packed/conv_w given, outputs: f64 [tokens][value_heads * 128]
// holds the recurrent output rows read with the model's own q, and magnitudes (optional, same shape) the sums of
// their terms' magnitudes, which bound the fp32 error of a kernel's rows.
REF_API int ref_gdn_recurrence(const float *state, const uint16_t *tape_kv, const float *decay, const uint16_t *beta, uint32_t tokens,
                               uint32_t key_heads, uint32_t value_heads, const uint16_t *history, const uint16_t *packed,
                               uint32_t packed_width, const uint16_t *conv_w, double *state_out, double *outputs, double *magnitudes) {
  using namespace gdn_model;
  const uint32_t kw = key_heads * kHeadDim, vw = value_heads * kHeadDim, conv = 2 * kw + vw;
  Fixture f{};
  f.shape = {key_heads, value_heads, conv, packed_width ? packed_width : conv};
  f.convWeights.p = conv_w;
  f.kv = tape_kv;
  f.decay = decay;
  f.beta = beta;
  StepInputs step;
  const bool with_rows = outputs && history && packed && conv_w;
  if (with_rows) {
    step.history.assign(history, history + uint64_t{kCarried} * conv);
    step.packed.assign(packed, packed + uint64_t{tokens} * packed_width);
  }
  for (uint32_t head = 0; head < value_heads; ++head) {
    std::vector<double> rows, sizes;
    const std::vector<double> s = recurrence(f, state, 0, 0, head, tokens, with_rows ? &step : nullptr, with_rows ? &rows : nullptr,
                                             with_rows && magnitudes ? &sizes : nullptr);
    std::copy(s.begin(), s.end(), state_out + uint64_t{head} * kHeadDim * kHeadDim);
    if (with_rows)
      for (uint32_t token = 0; token < tokens; ++token) {
        std::copy_n(rows.begin() + uint64_t{token} * kHeadDim, kHeadDim, outputs + uint64_t{token} * vw + head * kHeadDim);
        if (magnitudes) std::copy_n(sizes.begin() + uint64_t{token} * kHeadDim, kHeadDim, magnitudes + uint64_t{token} * vw + head * kHeadDim);
      }
  }
  return 0;
}

// ---- selection -------------------------------------------------------------------------------------
namespace sampling_model {
constexpr uint32_t kCandidates = SPLASH_DRAFT_CANDIDATES, kChildren = 4;

// The members of the reference's policy that its distribution reads.
struct SamplingPolicy {
  uint32_t topK;
  float temperature, topP, minP;
};
// The tokens a lane that ignores end-of-sequence never selects: set by the entry points below before they call the model.
struct StopTokens {
  std::vector<uint32_t> ids;
  bool contains(uint32_t token) const { return std::find(ids.begin(), ids.end(), token) != ids.end(); }
};
static StopTokens kStopTokens;

#include "sampling_model.inc"
}  // namespace sampling_model

REF_API uint32_t ref_sampling_candidates() { return sampling_model::kCandidates; }

// The same selections under an admission: mask (u32 words, a bit a token; NULL: unconstrained) and excluded tokens.
// greedy: the first token of the model's order among the admitted; sampled: referenceDistribution with the admission, then
// the draw of a row without children. token 0xFFFFFFFF: nothing admitted.
REF_API int ref_select_admitted(const float *logits, uint32_t vocab, const uint32_t *mask, const uint32_t *excluded, uint32_t n_excluded,
                                float temperature, float min_p, uint32_t top_k, float top_p, float uniform, uint32_t *token, uint32_t *close,
                                double *ambiguous) {
  using namespace sampling_model;
  kStopTokens.ids.assign(excluded, excluded + n_excluded);
  const Admission admits{mask, n_excluded != 0};
  bool any = false;
  for (uint32_t t = 0; t < vocab && !any; ++t) any = admits(t);
  *close = 0, *ambiguous = 0.0;
  if (!any) {
    *token = 0xffffffffu;
  } else if (!(temperature > 0.0f)) {
    *token = referenceArgmax(logits, vocab, admits);
  } else {
    const Distribution target = referenceDistribution(logits, vocab, SamplingPolicy{top_k, temperature, top_p, min_p}, admits);
    const float none[kChildren] = {};
    const Selection s = referenceSelection(target.probabilities, Children{}, std::span<const float>(none, kChildren), uniform);
    *token = s.token, *close = s.close, *ambiguous = target.ambiguousMass;
  }
  kStopTokens.ids.clear();
  return 0;
}

// The greedy selection of one row: the model's order (value descending, id ascending), its first token.
REF_API uint32_t ref_argmax(const float *logits, uint32_t vocab) { return sampling_model::referenceArgmax(logits, vocab); }
// The row's best `count` tokens in that order.
REF_API uint32_t ref_best(const float *logits, uint32_t vocab, uint32_t count, uint32_t *out) {
  const std::vector<uint32_t> best = sampling_model::referenceBest(logits, vocab, count);
  std::copy(best.begin(), best.end(), out);
  return uint32_t(best.size());
}

// One sampled row. logits: f32 [vocab]; ids, q: the row's 16 candidates and the draft's probabilities of them;
// draws: up to 4 candidate indices in the order drawn, 0xff past them (all 0xff: no children); tests: the 4
// uniforms of the child tests; uniform: the one of the final draw. token: the model's selection; close: 1
// where a comparison lay within 1e-5 of its threshold; ambiguous: the mass of tokens that the policy's cuts could
// keep or drop either way (relative to the kept mass).
REF_API int ref_sample_row(const float *logits, uint32_t vocab, float temperature, float min_p, uint32_t top_k, float top_p,
                           const uint32_t *ids, const float *q, const uint8_t *draws, const float *tests, float uniform,
                           uint32_t *token, uint32_t *close, double *ambiguous, double *probabilities) {
  using namespace sampling_model;
  if (!(temperature > 0.0f) || !vocab) return -1;
  const Distribution target = referenceDistribution(logits, vocab, SamplingPolicy{top_k, temperature, top_p, min_p});
  Children children;
  for (uint32_t i = 0; i < kCandidates; ++i) {
    children.ids[i] = ids ? ids[i] : 0xffffffffu;
    children.q[i] = q ? q[i] : 0.0;
  }
  for (uint32_t c = 0; draws && c < kChildren && draws[c] < kCandidates; ++c) children.draws.push_back(draws[c]);
  const float none[kChildren] = {};
  const Selection s = referenceSelection(target.probabilities, children, std::span<const float>(tests ? tests : none, kChildren), uniform);
  *token = s.token;
  *close = s.close;
  *ambiguous = target.ambiguousMass;
  if (probabilities) std::copy(target.probabilities.begin(), target.probabilities.end(), probabilities);
  return 0;
}

// ---- RMSNorm ---------------------------------------------------------------------------------------
// The header's functions are inline in namespace splash::test behind includes of the Metal backend; their text is cut
// like the models above, between a stand-in for the weights' buffer.
namespace norm_model {
namespace ops {
struct Contents {
  const void *p;
  const void *contents() const { return p; }
};
struct NormWeights {
  Contents buffer;
  bool float32;
};
}  // namespace ops
using splash::test::bf16ToFloat;
using splash::test::ulpBf16;
#include "norm_model.inc"
}  // namespace norm_model

// The fp64 norm of `rows` bf16 rows of `size` values with fp32 weights; `once` (optional, u8 a value) says whether the bf16
// value `got` holds there is the exact one rounded once, by the reference's own test.
REF_API void ref_rmsnorm(const uint16_t *x, uint32_t rows, uint32_t size, const float *weights, double *out, const uint16_t *got, uint8_t *once) {
  const norm_model::ops::NormWeights norm{{weights}, true};
  for (uint32_t r = 0; r < rows; ++r) {
    const std::vector<double> exact = norm_model::rmsNorm(x + size_t(r) * size, norm, size);
    for (uint32_t i = 0; i < size; ++i) {
      out[size_t(r) * size + i] = exact[i];
      if (got && once) once[size_t(r) * size + i] = norm_model::roundedOnceToBf16(got[size_t(r) * size + i], exact[i]);
    }
  }
}
