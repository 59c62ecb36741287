// TEST INFRASTRUCTURE - CPU oracle, not part of the product library.
//
// Glue operators and attention of the verify step, restated from the reference's kernels:
//   RMSNorm            runtime/metal/kernels/shared/normalization.metal:60-94,
//                      runtime/metal/kernels/common/rms_inverse.h:15-30
//   embedding gather   runtime/metal/kernels/shared/embedding.metal:10-18 (out-of-range token -> row 0)
//   RoPE tables        runtime/metal/kernels/shared/rope.metal:50-76, common/target_rope.h:7-16
//   q/k norm + RoPE + INT8 KV store
//                      runtime/metal/kernels/common/attention_qkv_prepare.h:26-91,
//                      runtime/metal/kernels/common/attention_store.h:52-85
//                      (CPU twin dev/tests/engine/Q8PageFormatReference.hpp:107-119)
//   paged attention    runtime/metal/kernels/common/paged_attention_tile.h:178-285,339-471,498-535,
//                      runtime/metal/kernels/common/attention_gate.h:19-45; the fp64 model follows
//                      dev/tests/engine/q8_flash_attention_metal_test.mm:483-536
//   selection          runtime/metal/kernels/decode/sampling.metal:984-989,1896-1991 (greedy),
//                      :44-49,:778-800 (temperature weights, child test, residual draw)
//   acceptance         runtime/metal/kernels/decode/sampling.metal:2044-2083
//   path commit        runtime/metal/kernels/shared/kv_path_commit.metal:21-46
// Parity of the INT8 quantizer is pinned against the reference's own CPU code through oracle/_ref
// (tests/test_oracle_ops.py), and attention against the reference's fp64 model compiled from its
// test file, as is the sampled selection (distribution cuts, child tests, residual draw) against the
// fp64 recursion of the reference's sampling test (oracle/ref_models_shim.cpp,
// tests/test_oracle_ref_models.py), and the greedy order against its referenceBest. Acceptance has neither
// stored vectors nor a host model in the reference ("parity unpinned" for it: invariants only).
#include "so_common.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

SO_API int so_dequant(uint32_t f, const uint8_t *native, uint32_t rows, uint32_t K, float *out);
SO_API uint64_t so_row_bytes(uint32_t f, uint32_t K);

using namespace so;

// y = bf16((x * rsqrt(mean x^2 + 1e-6)) * w); the sum of squares runs in the product's order: lanes
// of 32 over 8-element groups strided by 256, a butterfly over the lanes, then (rows wider than a
// warp's share) the warps in order. Tests compare with a tolerance of one bf16 ulp, the latitude the
// reference's own simd_sum leaves.
SO_API void so_rmsnorm(const uint16_t *x, uint32_t rows, uint32_t width, uint32_t x_stride, const float *w,
                       uint16_t *out, uint32_t out_stride) {
  for (uint32_t r = 0; r < rows; ++r) {
    double ss = 0;
    for (uint32_t c = 0; c < width; ++c) {
      const double v = bf2f(x[size_t(r) * x_stride + c]);
      ss += v * v;
    }
    const float inv = 1.0f / std::sqrt(float(ss / width) + kRmsEps);
    for (uint32_t c = 0; c < width; ++c)
      out[size_t(r) * out_stride + c] = f2bf((bf2f(x[size_t(r) * x_stride + c]) * inv) * w[c]);
  }
}

// Token row gather with dequantization to bf16; a token outside the table reads row 0.
SO_API int so_embed(uint32_t fmt, const uint8_t *table, uint32_t vocab, uint32_t width, const uint32_t *tokens,
                    uint32_t rows, uint16_t *out, uint32_t out_stride) {
  const uint64_t rb = so_row_bytes(fmt, width);
  if (!rb) return -1;
  std::vector<float> v(width);
  for (uint32_t r = 0; r < rows; ++r) {
    const uint32_t t = tokens[r] < vocab ? tokens[r] : 0;
    so_dequant(fmt, table + t * rb, 1, width, v.data());
    for (uint32_t c = 0; c < width; ++c) out[size_t(r) * out_stride + c] = f2bf(v[c]);
  }
  return 0;
}

// cos/sin[row][pair] at position anchor + depth; angle = float(position) * inv_freq[pair], times scale.
SO_API void so_rope_tables(const uint32_t *positions, uint32_t rows, const float *inv_freq, uint32_t pairs, float scale,
                           float *cosine, float *sine) {
  for (uint32_t r = 0; r < rows; ++r)
    for (uint32_t p = 0; p < pairs; ++p) {
      const float angle = float(positions[r]) * inv_freq[p];
      cosine[size_t(r) * pairs + p] = std::cos(angle) * scale;
      sine[size_t(r) * pairs + p] = std::sin(angle) * scale;
    }
}

// INT8 KV row: scale = max|x| / 127 (0 for a zero row), code = clamp(rint(x * 127 / max), -127, 127).
static inline float kv_scale(float m) { return m == 0.0f ? 0.0f : m / 127.0f; }
static inline int8_t kv_code(float v, float m) {
  if (m == 0.0f) return 0;
  long q = long(std::nearbyint(v * 127.0f / m));
  return int8_t(std::clamp<long>(q, -127, 127));
}
SO_API float so_kv_scale(float m) { return kv_scale(m); }
SO_API int so_kv_code(float v, float m) { return kv_code(v, m); }

// One attention layer's cache: pages of `page_tokens` tokens, keys and values token-major
// [page][kv_head][token][dim] int8, scales [page][kv_head][token] fp32 (scale_f16 == 0) or fp16.
struct SoKvLayer {
  int8_t *k, *v;
  void *k_scale, *v_scale;
  uint32_t kv_heads, head_dim, page_tokens, scale_f16;
};
static inline size_t kv_elem(const SoKvLayer &c, uint32_t page, uint32_t head, uint32_t tok) {
  return ((size_t(page) * c.kv_heads + head) * c.page_tokens + tok) * c.head_dim;
}
static inline size_t kv_sc(const SoKvLayer &c, uint32_t page, uint32_t head, uint32_t tok) {
  return (size_t(page) * c.kv_heads + head) * c.page_tokens + tok;
}
static inline float load_scale(const void *p, size_t i, uint32_t f16) {
  return f16 ? h2f(static_cast<const uint16_t *>(p)[i]) : static_cast<const float *>(p)[i];
}
static inline void store_scale(void *p, size_t i, uint32_t f16, float s) {
  if (f16) static_cast<uint16_t *>(p)[i] = f2h(s);
  else static_cast<float *>(p)[i] = s;
}

// Per row of one sequence: per-head RMSNorm of q and k with weights, rotation of pairs (i, i + pairs)
// of the first 2 * pairs dimensions by the row's table row, queries staged [row][q_head][dim] bf16,
// K and V rows quantized into the slot of token committed + row through the page table.
// qkv row = [q_heads x (q[D], gate[D] if gated)] [kv_heads x k[D]] [kv_heads x v[D]].
SO_API void so_attn_store(const uint16_t *qkv, uint32_t qkv_stride, uint32_t rows, uint32_t q_heads, uint32_t gated,
                          const float *q_norm, const float *k_norm, const float *cosine, const float *sine,
                          uint32_t pairs, const SoKvLayer *cache, const uint32_t *page_table, uint32_t committed,
                          uint16_t *queries) {
  const uint32_t D = cache->head_dim, KH = cache->kv_heads, qs = gated ? 2 * D : D;
  std::vector<float> n(D);
  auto norm_rope = [&](const uint16_t *src, const float *w, uint32_t row, uint16_t *dst) {
    float ss = 0.0f;
    // HeadDim / 32 partials of 32 dimensions each, added in order (attention_qkv_prepare.h:59-65).
    for (uint32_t g = 0; g < D / 32; ++g) {
      float part = 0.0f;
      for (uint32_t i = 0; i < 32; ++i) {
        const float v = bf2f(src[32 * g + i]);
        part += v * v;
      }
      ss += part;
    }
    const float inv = 1.0f / std::sqrt(ss / D + kRmsEps);
    for (uint32_t d = 0; d < D; ++d) n[d] = rbf(bf2f(src[d]) * inv * w[d]);
    for (uint32_t d = 0; d < D; ++d) {
      float r = n[d];
      if (d < 2 * pairs) {
        const uint32_t p = d % pairs;
        const float a = n[p], b = n[p + pairs], c = cosine[size_t(row) * pairs + p], s = sine[size_t(row) * pairs + p];
        r = d < pairs ? rbf(a * c - b * s) : rbf(b * c + a * s);
      }
      dst[d] = f2bf(r);
    }
  };
  std::vector<uint16_t> kn(D);
  for (uint32_t r = 0; r < rows; ++r) {
    const uint16_t *row = qkv + size_t(r) * qkv_stride;
    for (uint32_t h = 0; h < q_heads; ++h) norm_rope(row + h * qs, q_norm, r, queries + (size_t(r) * q_heads + h) * D);
    const uint32_t tok = committed + r, page = page_table[tok / cache->page_tokens], pt = tok % cache->page_tokens;
    for (uint32_t h = 0; h < KH; ++h) {
      norm_rope(row + q_heads * qs + h * D, k_norm, r, kn.data());
      const uint16_t *vsrc = row + q_heads * qs + KH * D + h * D;
      float km = 0.0f, vm = 0.0f;
      for (uint32_t d = 0; d < D; ++d) {
        km = std::max(km, std::fabs(bf2f(kn[d])));
        vm = std::max(vm, std::fabs(bf2f(vsrc[d])));
      }
      for (uint32_t d = 0; d < D; ++d) {
        cache->k[kv_elem(*cache, page, h, pt) + d] = kv_code(bf2f(kn[d]), km);
        cache->v[kv_elem(*cache, page, h, pt) + d] = kv_code(bf2f(vsrc[d]), vm);
      }
      store_scale(cache->k_scale, kv_sc(*cache, page, h, pt), cache->scale_f16, kv_scale(km));
      store_scale(cache->v_scale, kv_sc(*cache, page, h, pt), cache->scale_f16, kv_scale(vm));
    }
  }
}

// Attention of `rows` chain rows of one sequence over the stored INT8 pages, in fp64: row r sees
// tokens [0, committed + r]; score = (q . k_code) * k_scale / sqrt(D); out = softmax . (v_code * v_scale),
// rounded to bf16, then (gated) times sigmoid(gate) and rounded again. `tree` (optional, 8 bytes a
// row: ancestors u32, parent u16, depth u16) restricts a row to its ancestors inside the block.
SO_API void so_attention(const uint16_t *queries, const uint16_t *qkv, uint32_t qkv_stride, uint32_t rows,
                         uint32_t q_heads, uint32_t gated, const SoKvLayer *cache, const uint32_t *page_table,
                         uint32_t committed, const uint32_t *tree, uint16_t *out, uint32_t out_stride,
                         double *out_f64) {
  const uint32_t D = cache->head_dim, KH = cache->kv_heads, G = q_heads / KH, qs = gated ? 2 * D : D;
  const double scale = 1.0 / std::sqrt(double(D));
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t r = 0; r < int64_t(rows); ++r)
    for (int64_t h = 0; h < int64_t(q_heads); ++h) {
      const uint32_t kvh = uint32_t(h) / G;
      const uint16_t *q = queries + (size_t(r) * q_heads + h) * D;
      uint32_t visible = committed + uint32_t(r) + 1, ancestors = 0xffffffffu;
      if (tree) {
        ancestors = tree[2 * r];
        const uint32_t depth = tree[2 * r + 1] >> 16;
        visible = committed + rows;  // block rows are filtered by the ancestor mask below
        (void)depth;
      }
      std::vector<double> s(visible);
      double mx = -INFINITY;
      for (uint32_t t = 0; t < visible; ++t) {
        if (tree && t >= committed && !((ancestors >> (t - committed)) & 1u)) { s[t] = -INFINITY; continue; }
        const uint32_t page = page_table[t / cache->page_tokens], pt = t % cache->page_tokens;
        const int8_t *k = cache->k + kv_elem(*cache, page, kvh, pt);
        double dot = 0;
        for (uint32_t d = 0; d < D; ++d) dot += double(bf2f(q[d])) * k[d];
        s[t] = dot * load_scale(cache->k_scale, kv_sc(*cache, page, kvh, pt), cache->scale_f16) * scale;
        mx = std::max(mx, s[t]);
      }
      std::vector<double> acc(D, 0.0);
      double den = 0;
      for (uint32_t t = 0; t < visible; ++t) {
        if (s[t] == -INFINITY) continue;
        const uint32_t page = page_table[t / cache->page_tokens], pt = t % cache->page_tokens;
        const double p = std::exp(s[t] - mx);
        den += p;
        const double pv = p * load_scale(cache->v_scale, kv_sc(*cache, page, kvh, pt), cache->scale_f16);
        const int8_t *v = cache->v + kv_elem(*cache, page, kvh, pt);
        for (uint32_t d = 0; d < D; ++d) acc[d] += pv * v[d];
      }
      for (uint32_t d = 0; d < D; ++d) {
        const double o = den > 0 ? acc[d] / den : 0.0;
        float v = rbf(float(o));
        double exact = o;
        if (gated) {
          const float gate = bf2f(qkv[size_t(r) * qkv_stride + h * qs + D + d]);
          exact = double(v) * double(sigmoid(gate));
          v = v * sigmoid(gate);
        }
        out[size_t(r) * out_stride + h * D + d] = f2bf(v);
        if (out_f64) out_f64[(size_t(r) * q_heads + h) * D + d] = exact;
      }
    }
}

// Moves the accepted path's rows' K/V (codes and scales) from slot committed + row to slot
// committed + depth, in depth order; a chain's rows are already in place.
SO_API void so_kv_path_commit(const SoKvLayer *cache, const uint32_t *page_table, uint32_t committed, uint32_t path_mask) {
  const uint32_t D = cache->head_dim;
  uint32_t depth = 0;
  for (uint32_t row = 0; row < 32; ++row) {
    if (!((path_mask >> row) & 1u)) continue;
    if (row != depth) {
      const uint32_t s = committed + row, t = committed + depth;
      const uint32_t sp = page_table[s / cache->page_tokens], st = s % cache->page_tokens;
      const uint32_t tp = page_table[t / cache->page_tokens], tt = t % cache->page_tokens;
      for (uint32_t h = 0; h < cache->kv_heads; ++h) {
        memcpy(cache->k + kv_elem(*cache, tp, h, tt), cache->k + kv_elem(*cache, sp, h, st), D);
        memcpy(cache->v + kv_elem(*cache, tp, h, tt), cache->v + kv_elem(*cache, sp, h, st), D);
        store_scale(cache->k_scale, kv_sc(*cache, tp, h, tt), cache->scale_f16,
                    load_scale(cache->k_scale, kv_sc(*cache, sp, h, st), cache->scale_f16));
        store_scale(cache->v_scale, kv_sc(*cache, tp, h, tt), cache->scale_f16,
                    load_scale(cache->v_scale, kv_sc(*cache, sp, h, st), cache->scale_f16));
      }
    }
    ++depth;
  }
}

// ---- selection ----
constexpr uint32_t kSentinel = 0xFFFFFFFFu;
constexpr uint32_t kShard = 256;  // ids per shard of the mass sums

// Greedy: the largest finite logit, ties to the lowest id; none selectable -> the sentinel.
static uint32_t argmax_row(const float *l, uint32_t vocab) {
  uint32_t best = kSentinel;
  float bv = -INFINITY;
  for (uint32_t v = 0; v < vocab; ++v) {
    const float x = l[v];
    if (std::isnan(x) || x == -INFINITY) continue;
    if (best == kSentinel || x > bv) best = v, bv = x;
  }
  return best;
}

// Selection of every row of one lane (a chain of `rows` rows; row r's drafted child is the input
// token of row r + 1). temperature == 0: greedy. Otherwise weights w_v = exp((l_v - max) / T)
// (non-finite logits weigh 0); each shard of 256 ids is summed in id order and the shards in order;
// the drafted child is accepted iff u_child * Z < w_child (q = 1 for a deterministic draft), else the
// row draws from the residual (w_child removed) with its own uniform: target = u_row * Z', the first id
// whose running sum exceeds it; the last row always draws from the full
// distribution. uniforms: [0,16) row draws, 16 + 4 * row child tests.
// Order-preserving key of a selectable logit (larger logit, larger key; -0 counts as +0).
static uint32_t logit_key(float x) {
  if (x == 0.0f) x = 0.0f;
  uint32_t u;
  memcpy(&u, &x, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// The end of a row's distribution in the order (logit descending, id ascending): a token stays iff its key is
// above cut_key, or equal to it with an id up to cut_id (sampling.metal:604-668 distribution_end):
//   min_p  tokens weighing at least min_p of the heaviest: logits >= max + T * log(min_p);
//   top_k  then the k first of those;
//   top_p  then the shortest prefix whose mass exceeds top_p of the mass the first two cuts keep; where several
//          tokens tie at the last logit, 1 + floor((nucleus - mass above) / weight) of them stay, lowest ids first.
// Masses are sums of exp((l - max) / T) over shards of 256 ids in id order, shards in order; a cut logit is found
// bit by bit from the top of the key (32 measurements), which is what the CUDA kernel does too.
struct RowCut {
  uint32_t key = 0, id = kSentinel;  // keep everything selectable
};
static bool cut_keeps(const RowCut &c, float x, uint32_t v) {
  if (std::isnan(x) || x == -INFINITY) return false;
  const uint32_t k = logit_key(x);
  return k > c.key || (k == c.key && v <= c.id);
}
struct Measure {
  uint32_t count;
  float mass;
};
// Count and mass of the tokens the cut keeps whose key is at least `key` (strictly above it when `strict`).
static Measure measure(const float *l, uint32_t vocab, const RowCut &c, uint32_t key, bool strict, float mx, float inv_t) {
  Measure m{0, 0.0f};
  const uint32_t shards = (vocab + kShard - 1) / kShard;
  for (uint32_t s = 0; s < shards; ++s) {
    float sum = 0.0f;
    for (uint32_t v = s * kShard; v < std::min(vocab, (s + 1) * kShard); ++v) {
      if (!cut_keeps(c, l[v], v)) continue;
      const uint32_t k = logit_key(l[v]);
      if (strict ? k > key : k >= key) {
        ++m.count;
        sum += expf((l[v] - mx) * inv_t);
      }
    }
    m.mass += sum;
  }
  return m;
}
// The id of the n-th (1-based) kept token whose key equals `key`, in id order.
static uint32_t nth_tie(const float *l, uint32_t vocab, const RowCut &c, uint32_t key, uint32_t n) {
  for (uint32_t v = 0; v < vocab; ++v)
    if (cut_keeps(c, l[v], v) && logit_key(l[v]) == key && --n == 0) return v;
  return kSentinel;
}
static float key_logit(uint32_t key) {
  const uint32_t u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
  float x;
  memcpy(&x, &u, 4);
  return x;
}
static RowCut distribution_end(const float *l, uint32_t vocab, float mx, float temperature, float min_p, uint32_t top_k, float top_p) {
  const float inv_t = 1.0f / temperature;
  RowCut cut;
  Measure kept = measure(l, vocab, cut, 0, false, mx, inv_t);
  if (min_p > 0.0f) {
    const float t = std::min(mx + temperature * logf(min_p), mx);
    const Measure m = measure(l, vocab, cut, logit_key(t), false, mx, inv_t);
    if (m.count < kept.count) cut.key = logit_key(t), cut.id = kSentinel, kept = m;
  }
  if (top_k > 0 && top_k < kept.count) {
    uint32_t key = 0;  // the largest key with at least top_k kept tokens at or above it
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = key | (1u << bit);
      if (measure(l, vocab, cut, cand, false, mx, inv_t).count >= top_k) key = cand;
    }
    const Measure above = measure(l, vocab, cut, key, true, mx, inv_t);
    const uint32_t need = top_k - above.count;
    const uint32_t id = nth_tie(l, vocab, cut, key, need);
    cut.key = key, cut.id = id;
    kept.count = top_k;
    kept.mass = above.mass + float(need) * expf((key_logit(key) - mx) * inv_t);
  }
  if (top_p > 0.0f && top_p < 1.0f) {
    const float nucleus = top_p * kept.mass;
    uint32_t key = 0;  // the largest key whose kept tokens at or above it weigh more than the nucleus
    bool found = false;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = key | (1u << bit);
      if (measure(l, vocab, cut, cand, false, mx, inv_t).mass > nucleus) key = cand, found = true;
    }
    if (!found) found = measure(l, vocab, cut, 0, false, mx, inv_t).mass > nucleus;
    if (found) {  // rounding may leave the nucleus unreached: then everything kept so far stays
      const Measure above = measure(l, vocab, cut, key, true, mx, inv_t);
      const Measure at = measure(l, vocab, cut, key, false, mx, inv_t);
      const uint32_t ties = at.count - above.count;
      if (ties > 0) {
        const float w = expf((key_logit(key) - mx) * inv_t);
        const float q = std::min(std::max((nucleus - above.mass) / w, 0.0f), float(ties - 1));
        const uint32_t keep = 1u + uint32_t(q);
        cut.id = nth_tie(l, vocab, cut, key, keep);
        cut.key = key;
      }
    }
  }
  return cut;
}

SO_API void so_sample_verify_filtered(const float *logits, uint32_t logit_stride, uint32_t vocab, uint32_t rows,
                                      const uint32_t *input_tokens, float temperature, float min_p, uint32_t top_k, float top_p,
                                      const float *uniforms, uint32_t *selected, double *decision_margin, uint32_t *cut_out) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float *l = logits + size_t(r) * logit_stride;
    if (decision_margin) decision_margin[r] = INFINITY;
    const uint32_t top = argmax_row(l, vocab);
    if (cut_out) cut_out[2 * r] = 0, cut_out[2 * r + 1] = kSentinel;
    if (temperature == 0.0f || top == kSentinel) { selected[r] = top; continue; }
    const float mx = l[top], inv_t = 1.0f / temperature;
    const RowCut cut = distribution_end(l, vocab, mx, temperature, min_p, top_k, top_p);
    if (cut_out) cut_out[2 * r] = cut.key, cut_out[2 * r + 1] = cut.id;
    const uint32_t shards = (vocab + kShard - 1) / kShard;
    std::vector<float> w(vocab), shard(shards, 0.0f);
    for (uint32_t v = 0; v < vocab; ++v) w[v] = cut_keeps(cut, l[v], v) ? expf((l[v] - mx) * inv_t) : 0.0f;
    const bool has_child = r + 1 < rows;
    const uint32_t child = has_child ? input_tokens[r + 1] : kSentinel;
    auto mass = [&](bool drop_child, std::vector<float> &sh) {
      float total = 0.0f;
      for (uint32_t s = 0; s < shards; ++s) {
        float sum = 0.0f;
        for (uint32_t v = s * kShard; v < std::min(vocab, (s + 1) * kShard); ++v)
          sum += (drop_child && v == child) ? 0.0f : w[v];
        sh[s] = sum;
        total += sum;
      }
      return total;
    };
    const float z = mass(false, shard);
    bool drop = false;
    if (has_child && child < vocab) {
      const float u = uniforms[16 + 4 * r];
      if (decision_margin) decision_margin[r] = std::fabs(double(u) * z - w[child]) / std::max(double(z), 1e-30);
      if (u * z < w[child]) { selected[r] = child; continue; }
      drop = true;
    }
    const float zr = drop ? mass(true, shard) : z;
    // The first id whose running sum exceeds the target; the running sum of an id is the sum of the
    // shards before its shard (added in order) plus its shard's ids up to it (added in order from 0).
    const float target = uniforms[r] * zr;
    float run = 0.0f;
    uint32_t pick = kSentinel;
    for (uint32_t s = 0; s < shards && pick == kSentinel; ++s) {
      if (run + shard[s] > target) {
        float loc = 0.0f;
        for (uint32_t v = s * kShard; v < std::min(vocab, (s + 1) * kShard); ++v) {
          loc += (drop && v == child) ? 0.0f : w[v];
          if (run + loc > target) { pick = v; break; }
        }
      }
      run += shard[s];
    }
    if (pick == kSentinel)  // rounding put the target at or past the total: the last id that weighs
      for (uint32_t v = vocab; v-- > 0;)
        if (w[v] > 0.0f && !(drop && v == child)) { pick = v; break; }
    selected[r] = pick;
  }
}

// Sampled rows whose children are the draws of a draft (runtime/metal/kernels/decode/sampling.metal:693-885, uniforms
// runtime/metal/abi/Sampling.h:12-31): per row 16 candidate ids with the draft's probabilities q and the candidate indices
// of up to 4 drawn children in the order drawn (0xff past them). Recursive rejection sampling without replacement: child c
// is taken iff u[16 + 4 r + c] q < p; after a rejection p <- max(p - q, 0) / sum and the mass outside the candidates is
// renormalised with it, q loses the child and is renormalised; a row that takes none draws with u[r] from the last
// residual, its candidates first (cumulative in candidate order), else a token outside them by the target's own weights:
// the shard (256 ids, weights summed in id order, the candidates' taken out) the point falls in, then its ids in order.
// decision_margin[r]: the smallest relative distance of a test or of the final point from its threshold.
SO_API void so_sample_verify_draws(const float *logits, uint32_t logit_stride, uint32_t vocab, uint32_t rows, float temperature,
                                   float min_p, uint32_t top_k, float top_p, const float *uniforms, const uint32_t *candidate_ids,
                                   const float *candidate_q, const uint8_t *draws, uint32_t *selected, double *decision_margin) {
  constexpr uint32_t C = 16;
  for (uint32_t r = 0; r < rows; ++r) {
    const float *l = logits + size_t(r) * logit_stride;
    double margin = INFINITY;
    auto near = [&](double a, double b, double scale) { margin = std::min(margin, std::fabs(a - b) / std::max(scale, 1e-30)); };
    const uint32_t top = argmax_row(l, vocab);
    if (decision_margin) decision_margin[r] = INFINITY;
    if (temperature == 0.0f || top == kSentinel) { selected[r] = top; continue; }
    const float mx = l[top], inv_t = 1.0f / temperature;
    const RowCut cut = distribution_end(l, vocab, mx, temperature, min_p, top_k, top_p);
    const uint32_t shards = (vocab + kShard - 1) / kShard;
    std::vector<float> w(vocab), shard(shards, 0.0f);
    for (uint32_t v = 0; v < vocab; ++v) w[v] = cut_keeps(cut, l[v], v) ? expf((l[v] - mx) * inv_t) : 0.0f;
    float z = 0.0f;
    for (uint32_t s = 0; s < shards; ++s) {
      float sum = 0.0f;
      for (uint32_t v = s * kShard; v < std::min(vocab, (s + 1) * kShard); ++v) sum += w[v];
      shard[s] = sum;
      z += sum;
    }
    const uint32_t *ids = candidate_ids + C * r;
    const uint8_t *dr = draws + 4 * r;
    uint32_t pick = kSentinel;
    bool done = false;
    float p[C], q[C];
    float outside_weight = z, outside = 1.0f;
    const bool children = dr[0] != 0xff && z > 0.0f;
    if (children) {
      for (uint32_t i = 0; i < C; ++i) {
        const float wi = ids[i] < vocab ? w[ids[i]] : 0.0f;
        if (ids[i] < vocab) shard[ids[i] / kShard] = std::max(shard[ids[i] / kShard] - wi, 0.0f);
        p[i] = wi / z;
        q[i] = candidate_q[C * r + i];
      }
      outside_weight = 0.0f;
      for (uint32_t s = 0; s < shards; ++s) outside_weight += shard[s];
      outside = outside_weight / z;
      for (uint32_t c = 0; c < 4 && !done; ++c) {
        const uint32_t dc = dr[c];
        if (dc >= C) break;
        const float lhs = uniforms[16 + 4 * r + c] * q[dc];
        near(lhs, p[dc], std::max(p[dc], q[dc]));
        if (lhs < p[dc]) { pick = ids[dc], done = true; break; }
        float residual = outside;
        for (uint32_t i = 0; i < C; ++i) residual += std::max(p[i] - q[i], 0.0f);
        if (!(residual > 0.0f)) break;
        for (uint32_t i = 0; i < C; ++i) p[i] = std::max(p[i] - q[i], 0.0f) / residual;
        outside /= residual;
        q[dc] = 0.0f;
        float rest = 0.0f;
        for (uint32_t i = 0; i < C; ++i) rest += q[i];
        for (uint32_t i = 0; rest > 0.0f && i < C; ++i) q[i] /= rest;
      }
    }
    float target = uniforms[r] * z;
    bool excluding = false;
    if (children && !done) {
      float inside = 0.0f;
      for (uint32_t i = 0; i < C; ++i) inside += p[i];
      const float point = uniforms[r] * (inside + outside);
      float cumulative = 0.0f;
      uint32_t last = C;
      for (uint32_t i = 0; i < C && !(point < cumulative); ++i)
        if (p[i] > 0.0f) {
          last = i, cumulative += p[i];
          near(point, cumulative, inside + outside);
        }
      if (last < C && (point < cumulative || !(outside > 0.0f))) pick = ids[last], done = true;
      else excluding = true, target = (point - inside) / outside * outside_weight;
    }
    if (!done) {
      auto excluded = [&](uint32_t v) {
        if (!excluding) return false;
        for (uint32_t i = 0; i < C; ++i)
          if (ids[i] == v) return true;
        return false;
      };
      float run = 0.0f, shard_target = 0.0f;
      uint32_t at = kSentinel;
      for (uint32_t s = 0; s < shards; ++s) {
        if (!(shard[s] > 0.0f)) continue;
        at = s, shard_target = target - run;
        run += shard[s];
        near(run, target, outside_weight);
        if (run > target) break;
      }
      if (at != kSentinel) {
        float loc = 0.0f;
        for (uint32_t v = at * kShard; v < std::min(vocab, (at + 1) * kShard); ++v) {
          const float wv = excluded(v) ? 0.0f : w[v];
          if (wv > 0.0f) pick = v;
          loc += wv;
          if (wv > 0.0f) near(loc, shard_target, outside_weight);
          if (wv > 0.0f && loc > shard_target) break;
        }
      }
    }
    selected[r] = pick;
    if (decision_margin) decision_margin[r] = margin;
  }
}

SO_API void so_sample_verify(const float *logits, uint32_t logit_stride, uint32_t vocab, uint32_t rows,
                             const uint32_t *input_tokens, float temperature, const float *uniforms,
                             uint32_t *selected, double *decision_margin) {
  so_sample_verify_filtered(logits, logit_stride, vocab, rows, input_tokens, temperature, 0.0f, 0, 1.0f, uniforms, selected,
                            decision_margin, nullptr);
}

// Acceptance of one lane (sampling.metal:2044-2083): from row 0 follow the child whose parent is
// the row and whose input token is the row's selection; kept = min(accepted + 1, remaining); the
// path's selections move to the first kept slots; a stop token truncates.
// tree: 8 bytes a row (ancestors u32, parent u16 | depth u16 << 16).
SO_API void so_accept(const uint32_t *input_tokens, const uint32_t *tree, uint32_t *tokens, uint32_t rows,
                      uint32_t remaining, const uint32_t *stop_tokens, uint32_t n_stop, uint32_t *retained,
                      uint32_t *accepted_count, uint32_t *retained_rows) {
  uint32_t path[32];
  path[0] = 0;
  uint32_t accepted = 0;
  for (uint32_t row = 0;;) {
    const uint32_t token = tokens[row];
    uint32_t next = 0;
    for (uint32_t child = row + 1; child < rows && !next; ++child)
      next = ((tree[2 * child + 1] & 0xffffu) == row && input_tokens[child] == token) ? child : 0;
    if (!next) break;
    path[++accepted] = next;
    row = next;
  }
  uint32_t kept = std::min(accepted + 1, remaining);
  for (uint32_t i = 0; i < kept; ++i) {
    const uint32_t token = tokens[path[i]];
    tokens[i] = token;
    for (uint32_t s = 0; s < n_stop; ++s)
      if (stop_tokens[s] == token) kept = i + 1;
  }
  *accepted_count = std::min(accepted, kept);
  *retained = kept;
  *retained_rows = tree[2 * path[kept - 1]];
}

// ---- sampling penalties (runtime/metal/kernels/decode/sampling.metal:985-1048) ----
// One logit: repetition divides a positive logit and multiplies a negative one when the prompt or the output holds
// the token; presence and frequency lower it by the output's count; the result saturates; NaN and -inf stay.
static bool unselectable_logit(float v) {
  uint32_t b;
  memcpy(&b, &v, 4);
  return (b & 0x7fffffffu) > 0x7f800000u || b == 0xff800000u;
}
SO_API float so_penalize_logit(float value, uint32_t count, float repetition, float repetition_inverse, float presence, float frequency) {
  if (unselectable_logit(value)) return value;
  value *= value > 0.0f ? repetition_inverse : repetition;
  if (count) value -= frequency * float(count) + presence;
  const float mx = 3.402823466e+38f;
  return value < -mx ? -mx : value > mx ? mx : value;
}
// One lane's selected rows rewritten in place. words[token]: the output's count of the token (low 31 bits) and the
// prompt bit (bit 31); a row's context adds the draft tokens on its path: bit r of `drafted` is set when input row r
// (r >= 1) holds the token, and row `row` counts the bits of its ancestors but the anchor. tree: 8 bytes a row
// (ancestors u32 first).
// Admission (TargetRow::admits, runtime/metal/kernels/decode/sampling.metal:33-46): a token whose bit in the row's mask is
// clear, or that is excluded, is not selectable: its logit becomes -inf.
SO_API void so_sample_admit(float *logits, uint32_t logit_stride, uint32_t vocab, uint32_t rows, const uint32_t *masks, uint32_t mask_words,
                            const uint32_t *excluded, uint32_t n_excluded) {
  for (uint32_t row = 0; row < rows; ++row)
    for (uint32_t token = 0; token < vocab; ++token) {
      bool out = masks && !((masks[size_t(row) * mask_words + token / 32] >> (token % 32)) & 1u);
      for (uint32_t i = 0; i < n_excluded; ++i) out = out || excluded[i] == token;
      if (out) logits[size_t(row) * logit_stride + token] = -INFINITY;
    }
}

SO_API void so_sample_penalize(float *logits, uint32_t logit_stride, uint32_t vocab, uint32_t rows, const uint32_t *words,
                               const uint32_t *input_tokens, const uint32_t *tree, float repetition, float presence, float frequency) {
  const float mx = 3.402823466e+38f;
  const float inverse = std::min(1.0f / repetition, mx);
#pragma omp parallel for
  for (int64_t token = 0; token < int64_t(vocab); ++token) {
    uint32_t drafted = 0;
    for (uint32_t row = 1; row < rows; ++row) drafted |= uint32_t(input_tokens[row] == uint32_t(token)) << row;
    const uint32_t word = words[token];
    if (!word && !drafted) continue;
    for (uint32_t row = 0; row < rows; ++row) {
      const uint32_t path = tree[2 * row];
      const uint32_t count = (word & 0x7fffffffu) + uint32_t(__builtin_popcount(drafted & path & ~1u));
      if (!count && !(word & 0x80000000u)) continue;
      float &logit = logits[size_t(row) * logit_stride + size_t(token)];
      logit = so_penalize_logit(logit, count, repetition, inverse, presence, frequency);
    }
  }
}

// ---- MoE routing (runtime/metal/kernels/shared/moe.metal:22-111) ----
// Per row: the top_k experts by fp32 score, descending score then ascending id; their weights the softmax of their
// scores, w_r = exp2((s_r - s_0) log2 e) / sum (sigmoid_normalized: sigmoid(s_r) / (sum of the top_k's sigmoids + 1e-20)),
// summed in rank order; with shared_gate, route top_k is the shared expert (id `experts`) weighted by
// sigmoid(x . shared_gate), the dot product summed as 256 strided partial sums, then lanes, then the 8 groups in order.
SO_API void so_moe_route(const float *scores, uint32_t rows, uint32_t experts, uint32_t slots, uint32_t top_k, uint32_t sigmoid_normalized,
                         const uint16_t *input, uint32_t input_size, const float *shared_gate, uint32_t *selected, float *weights) {
  const uint32_t routes = top_k + (shared_gate ? 1u : 0u);
  for (uint32_t r = 0; r < rows; ++r) {
    std::vector<float> sc(scores + size_t(r) * slots, scores + size_t(r) * slots + experts);
    std::vector<float> ordered(top_k);
    for (uint32_t rank = 0; rank < top_k; ++rank) {
      uint32_t best = 0xFFFFFFFFu;
      float bv = -INFINITY;
      for (uint32_t e = 0; e < experts; ++e)
        if (sc[e] > bv) bv = sc[e], best = e;  // ascending scan: the lowest id among equals
      if (best == 0xFFFFFFFFu) best = 0;  // no score above -inf left: the reference's lane 0 holds the candidate
      ordered[rank] = bv;
      selected[size_t(r) * routes + rank] = best;
      sc[best] = -INFINITY;
    }
    float den = 0.0f;
    for (uint32_t o = 0; o < top_k; ++o)
      den += sigmoid_normalized ? sigmoid(ordered[o]) : exp2f((ordered[o] - ordered[0]) * 1.44269504089f);
    for (uint32_t rank = 0; rank < top_k; ++rank)
      weights[size_t(r) * routes + rank] = sigmoid_normalized ? sigmoid(ordered[rank]) / (den + 1e-20f)
                                                              : exp2f((ordered[rank] - ordered[0]) * 1.44269504089f) / den;
    if (shared_gate) {
      float partial[256];
      for (uint32_t t = 0; t < 256; ++t) {
        float a = 0.0f;
        for (uint32_t d = t; d < input_size; d += 256) a += bf2f(input[size_t(r) * input_size + d]) * shared_gate[d];
        partial[t] = a;
      }
      float total = 0.0f;
      for (uint32_t g = 0; g < 8; ++g) {
        float lanes[32];
        for (uint32_t l = 0; l < 32; ++l) lanes[l] = partial[32 * g + l];
        for (uint32_t o = 16; o; o >>= 1)
          for (uint32_t l = 0; l < o; ++l) lanes[l] += lanes[l + o];  // the butterfly's lane 0
        total += lanes[0];
      }
      selected[size_t(r) * routes + top_k] = experts;
      weights[size_t(r) * routes + top_k] = sigmoid(total);
    }
  }
}

// ---- MoE expert passes and combine (runtime/metal/kernels/shared/moe_gguf.metal:94-160, moe.metal:367-392) ----
// Per route (row, expert): intermediate = bf16(bf16(up . x) * silu(bf16(gate . x))); y = bf16(down . intermediate);
// out = bf16(residual + sum over the row's routes in slot order of weight * float(y)). Dot products in fp64 over the
// effective weights d sc q - dmin m (so_dequant); y64 (optional, [rows * routes][hidden]) receives the down sums before
// rounding, for tolerance gates.
SO_API int so_moe_experts(const uint16_t *input, const uint16_t *residual, const uint32_t *selected, const float *weights,
                          const uint8_t *gate, const uint8_t *up, const uint8_t *down, uint32_t rows, uint32_t routes, uint32_t hidden,
                          uint32_t inter, uint32_t experts_total, uint16_t *out, double *y64) {
  const uint64_t gu_row = so_row_bytes(0, hidden), dn_row = so_row_bytes(0, inter);
  std::vector<float> y(size_t(rows) * routes * hidden);
  int status = 0;
#pragma omp parallel for schedule(dynamic)
  for (int64_t route = 0; route < int64_t(rows) * routes; ++route) {
    const uint32_t row = uint32_t(route / routes), e = std::min(selected[route], experts_total - 1);
    std::vector<float> wg(size_t(inter) * hidden), wu(size_t(inter) * hidden), wd(size_t(hidden) * inter), mid(inter);
    if (so_dequant(0, gate + size_t(e) * inter * gu_row, inter, hidden, wg.data()) || so_dequant(0, up + size_t(e) * inter * gu_row, inter, hidden, wu.data()) ||
        so_dequant(0, down + size_t(e) * hidden * dn_row, hidden, inter, wd.data()))
      status = -1;
    for (uint32_t c = 0; c < inter; ++c) {
      double g = 0.0, u = 0.0;
      for (uint32_t k = 0; k < hidden; ++k) {
        const double x = bf2f(input[size_t(row) * hidden + k]);
        g += double(wg[size_t(c) * hidden + k]) * x, u += double(wu[size_t(c) * hidden + k]) * x;
      }
      mid[c] = rbf(rbf(float(u)) * silu(rbf(float(g))));
    }
    for (uint32_t c = 0; c < hidden; ++c) {
      double v = 0.0;
      for (uint32_t k = 0; k < inter; ++k) v += double(wd[size_t(c) * inter + k]) * mid[k];
      if (y64) y64[size_t(route) * hidden + c] = v;
      y[size_t(route) * hidden + c] = rbf(float(v));
    }
  }
  for (uint32_t row = 0; row < rows; ++row)
    for (uint32_t c = 0; c < hidden; ++c) {
      float acc = 0.0f;
      for (uint32_t s = 0; s < routes; ++s) acc += weights[size_t(row) * routes + s] * y[(size_t(row) * routes + s) * hidden + c];
      out[size_t(row) * hidden + c] = f2bf((residual ? bf2f(residual[size_t(row) * hidden + c]) : 0.0f) + acc);
    }
  return status;
}
