// TEST INFRASTRUCTURE - CPU oracle, not part of the product library.
//
// Gated-DeltaNet verify step of one lane and one layer, restated from the reference's decode kernel:
//   prologue (conv + SiLU, q/k RMS norm and scales, gates, tape)  runtime/metal/kernels/decode/gdn.metal:139-264
//   fold of the previous step's accepted rows into the state      :270-298
//   chain scan from the committed state (outputs only)            :312-415
//   gated RMSNorm                                                 :489-526
//   primitives (conv, gates, head order)    runtime/metal/kernels/common/gdn_primitives.h:63-106
// The step: (1) fold the `pending` rows of the previous step's tape into the state and store it as
// the committed state; the conv history becomes the last three input rows before this block;
// (2) per row: conv (4 taps over the row's path), SiLU, q/k normalised and scaled, beta and decay;
// (3) scan the rows from the committed state, keeping only their outputs; (4) gate; (5) write this
// step's tape. The state after the block is not stored: the next step folds what was accepted.
// Rounding points follow the kernel (bf16 where it rounds, fp32 sums); sums run in index order, so
// tests compare with the reference's gates (state 1e-4 relative, hidden 3 bf16 ulp), not bitwise.
// No vectors of this kernel are stored in the reference; parity is pinned against the fp64 models of the
// reference's kernel test (dev/tests/engine/gdn_decode_metal_test.mm:371-407, 474-522) compiled into
// oracle/_ref (oracle/ref_models_shim.cpp, tests/test_oracle_ref_models.py); trees are held to chains of
// their paths (tests/test_oracle_ops.py).
#include "so_common.h"

#include <algorithm>
#include <cmath>
#include <vector>

using namespace so;

struct SoGdnTape {
  uint16_t *inputs;  // bf16 [rows][conv_dim]: q, k, v conv inputs
  uint16_t *k;       // bf16 [rows][key_heads * 128], normalised and scaled keys
  uint16_t *v;       // bf16 [rows][value_heads * 128], conv outputs
  uint16_t *beta;    // bf16 [rows][value_heads]
  float *decay;      // f32  [rows][value_heads]
};

struct SoGdnArgs {
  const uint16_t *qkvz;  // bf16 [rows][qkvz_stride]: q | k | v | z
  const uint16_t *b, *a; // bf16 [rows][ab_stride]
  const uint16_t *conv_w;      // bf16 [conv_dim][4]
  const float *a_scale;        // f32 [value_heads]
  const uint16_t *dt_bias;     // bf16 [value_heads]
  const float *norm_w;         // f32 [128]
  const uint16_t *conv_state_in;  // bf16 [3][conv_dim]
  uint16_t *conv_state_out;
  const float *state_in;       // f32 [value_heads][128][128] (value dim, key dim)
  float *state_out;
  SoGdnTape pending, step;
  uint16_t *hidden;            // bf16 [rows][value_heads * 128]
  uint32_t rows, pending_rows, key_heads, value_heads, qkvz_stride, ab_stride, hidden_stride, tiled;
  // Trees (runtime/metal/kernels/decode/gdn.metal:131-137, 418-478): tree = 8 bytes a row, ancestors u32 first (the row's
  // path from the anchor, itself included), NULL for a chain; pending_path = the row mask of the previous step's
  // accepted path in its tape (0: its first pending_rows rows).
  const uint32_t *tree;
  uint32_t pending_path;
};

// Row of the n-th token (from the anchor) of a path mask.
static uint32_t path_row(uint32_t path, uint32_t n) {
  for (uint32_t i = 0; i < n; ++i) path &= path - 1;
  return uint32_t(__builtin_ctz(path));
}

SO_API void so_gdn_verify(const SoGdnArgs *p) {
  constexpr uint32_t D = 128, Taps = 4;
  const uint32_t KH = p->key_heads, VH = p->value_heads, KW = KH * D, VW = VH * D, C = 2 * KW + VW, per_key = VH / KH;
  const uint32_t pending_path = p->pending_path ? p->pending_path : (p->pending_rows >= 32 ? ~0u : (1u << p->pending_rows) - 1u);
  const uint32_t pending_count = uint32_t(__builtin_popcount(pending_path));
  auto row_path = [&](uint32_t r) { return (p->tree ? (p->tree[2 * r] & ((2u << r) - 1u)) : ((2u << r) - 1u)) | (1u << r); };
  // (1) conv history = last 3 rows of (conv_state_in ++ the pending path's inputs).
  std::vector<uint16_t> hist(3 * size_t(C));
  for (int i = 0; i < 3; ++i) {
    const int src = int(pending_count) - 3 + i;  // index into the pending path; negative -> carried rows
    const uint16_t *row = src >= 0 ? p->pending.inputs + size_t(path_row(pending_path, uint32_t(src))) * C : p->conv_state_in + size_t(3 + src) * C;
    std::copy(row, row + C, hist.begin() + size_t(i) * C);
  }
  std::copy(hist.begin(), hist.end(), p->conv_state_out);
  // (2) rows' conv, norms and gates.
  std::vector<float> q(size_t(p->rows) * KW), k(size_t(p->rows) * KW), v(size_t(p->rows) * VW);
  std::vector<float> beta(size_t(p->rows) * VH), decay(size_t(p->rows) * VH);
  auto input = [&](int row, uint32_t ch) -> float {
    if (row >= 0) return bf2f(p->qkvz[size_t(row) * p->qkvz_stride + ch]);
    return bf2f(hist[size_t(3 + row) * C + ch]);
  };
  // A row's taps are the last four tokens of its path, itself last; tokens before the anchor come from the history.
  auto conv = [&](uint32_t row, uint32_t ch) {
    const uint32_t path = row_path(row);
    const int depth = __builtin_popcount(path) - 1;
    float value = 0.0f;
    for (uint32_t tap = 0; tap < Taps; ++tap) {
      const int at = depth - 3 + int(tap);  // the tap's token, counted from the anchor
      value += input(at >= 0 ? int(path_row(path, uint32_t(at))) : at, ch) * bf2f(p->conv_w[size_t(ch) * Taps + tap]);
    }
    value = rbf(value);
    return rbf(silu(value));
  };
  for (uint32_t r = 0; r < p->rows; ++r) {
    for (uint32_t ch = 0; ch < C; ++ch) p->step.inputs[size_t(r) * C + ch] = p->qkvz[size_t(r) * p->qkvz_stride + ch];
    for (uint32_t kh = 0; kh < KH; ++kh) {
      float qs = 0.0f, ks = 0.0f;
      std::vector<float> qc(D), kc(D);
      for (uint32_t d = 0; d < D; ++d) {
        qc[d] = conv(r, kh * D + d);
        kc[d] = conv(r, KW + kh * D + d);
        qs += qc[d] * qc[d];
        ks += kc[d] * kc[d];
      }
      const float qn = 1.0f / std::sqrt(qs / D + kRmsEps), kn = 1.0f / std::sqrt(ks / D + kRmsEps);
      for (uint32_t d = 0; d < D; ++d) {
        q[size_t(r) * KW + kh * D + d] = rbf(rbf(qc[d] * qn) * 0.0078125f);
        const float key = rbf(rbf(kc[d] * kn) * 0.08838834765f);
        k[size_t(r) * KW + kh * D + d] = key;
        p->step.k[size_t(r) * KW + kh * D + d] = f2bf(key);
      }
    }
    for (uint32_t c = 0; c < VW; ++c) {
      v[size_t(r) * VW + c] = conv(r, 2 * KW + c);
      p->step.v[size_t(r) * VW + c] = f2bf(v[size_t(r) * VW + c]);
    }
    for (uint32_t h = 0; h < VH; ++h) {
      const float bb = bf2f(p->b[size_t(r) * p->ab_stride + h]);
      const float be = rbf(sigmoid(bb));
      const float x = rbf(bf2f(p->a[size_t(r) * p->ab_stride + h]) + bf2f(p->dt_bias[h]));
      const float sp = rbf(std::max(x, 0.0f) + log2f(1.0f + exp2f(-1.44269504089f * std::fabs(x))) * 0.69314718056f);
      const float de = expf(p->a_scale[h] * sp);
      beta[size_t(r) * VH + h] = be;
      decay[size_t(r) * VH + h] = de;
      p->step.beta[size_t(r) * VH + h] = f2bf(be);
      p->step.decay[size_t(r) * VH + h] = de;
    }
  }
  // (1b), (3), (4) per value head.
#pragma omp parallel for schedule(static)
  for (int64_t h = 0; h < int64_t(VH); ++h) {
    const uint32_t kh = uint32_t(h) / per_key;
    std::vector<float> S(p->state_in + size_t(h) * D * D, p->state_in + size_t(h + 1) * D * D);
    auto advance = [&](const float *key, const float *val, float d, float b, const float *query, float *out) {
      for (uint32_t vd = 0; vd < D; ++vd) {
        float *row = S.data() + size_t(vd) * D;
        float mem = 0.0f;
        for (uint32_t i = 0; i < D; ++i) {
          row[i] *= d;
          mem += row[i] * key[i];
        }
        const float delta = (val[vd] - mem) * b;
        float res = 0.0f;
        for (uint32_t i = 0; i < D; ++i) {
          row[i] += key[i] * delta;
          if (query) res += row[i] * query[i];
        }
        if (out) out[vd] = res;
      }
    };
    std::vector<float> key(D), val(D);
    for (uint32_t n = 0; n < pending_count; ++n) {
      const uint32_t t = path_row(pending_path, n);
      for (uint32_t i = 0; i < D; ++i) {
        key[i] = bf2f(p->pending.k[size_t(t) * KW + kh * D + i]);
        val[i] = bf2f(p->pending.v[size_t(t) * VW + h * D + i]);
      }
      advance(key.data(), val.data(), p->pending.decay[size_t(t) * VH + h], bf2f(p->pending.beta[size_t(t) * VH + h]),
              nullptr, nullptr);
    }
    std::copy(S.begin(), S.end(), p->state_out + size_t(h) * D * D);
    std::vector<float> o(D);
    const uint32_t out_head = p->tiled ? (uint32_t(h) % per_key) * KH + uint32_t(h) / per_key : uint32_t(h);
    const std::vector<float> committed = S;
    for (uint32_t r = 0; r < p->rows; ++r) {
      const uint32_t path = row_path(r);
      if (path == (2u << r) - 1u && (r == 0 || row_path(r - 1) == (2u << (r - 1)) - 1u)) {
        // the chain so far: the state carries on from the row before
        advance(k.data() + size_t(r) * KW + kh * D, v.data() + size_t(r) * VW + h * D, decay[size_t(r) * VH + h],
                beta[size_t(r) * VH + h], q.data() + size_t(r) * KW + kh * D, o.data());
      } else {
        // a tree row: from the committed state along its own path, by definition
        S = committed;
        for (uint32_t up = path; up; up &= up - 1) {
          const uint32_t t = uint32_t(__builtin_ctz(up));
          advance(k.data() + size_t(t) * KW + kh * D, v.data() + size_t(t) * VW + h * D, decay[size_t(t) * VH + h],
                  beta[size_t(t) * VH + h], t == r ? q.data() + size_t(r) * KW + kh * D : nullptr, t == r ? o.data() : nullptr);
        }
      }
      float total = 0.0f;
      for (uint32_t d = 0; d < D; ++d) {
        o[d] = rbf(o[d]);
        total += o[d] * o[d];
      }
      const float inv = 1.0f / std::sqrt(total / D + kRmsEps);
      for (uint32_t d = 0; d < D; ++d) {
        const float normalized = rbf((o[d] * inv) * p->norm_w[d]);
        const float z = bf2f(p->qkvz[size_t(r) * p->qkvz_stride + C + h * D + d]);
        p->hidden[size_t(r) * p->hidden_stride + out_head * D + d] =
            f2bf((normalized * z) / (1.0f + exp2f(-1.44269504089f * z)));
      }
    }
  }
}
