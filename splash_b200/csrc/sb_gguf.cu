// C ABI of the GGUF reader and of the loader that fills a target model from a GGUF of the Qwen3.5 hybrid family
// (include/splash_b200.h, "GGUF files"). The reader is host code (model/GgufReader.hpp) and needs no device; the loader
// goes through the same tensor addresses sb_target_tensor hands out.
//
// Tensor names, shapes and conversions follow the reference's image builder (runtime/model/GgufImage.cpp:477-520 mixers
// and FFNs, :541-556 the hybrid's norms, :272-319 alpha/beta, convolution and per-head vectors; metadata keys :902-933).
// The value heads of a GGUF lie in llama.cpp's tiled order (value head j of every key head side by side); the rows that
// carry a value head index (the v rows of attn_qkv, attn_gate, ssm_beta / ssm_alpha, the convolution's v channels, ssm_a,
// ssm_dt.bias) are gathered into grouped order as the reference does (runtime/model/GgufPreparation.cpp:28-39), and the
// GDN output, whose columns ssm_out reads as stored, keeps the tiled order (SbTargetConfig.tiled_heads = 1).
#include <memory>
#include <string>
#include <vector>

#include "model/GgufReader.hpp"
#include "sb_internal.h"

using splash::b200::model::GgufError;
using splash::b200::model::GgufReader;
using splash::b200::model::GgufTensor;
namespace ggml = splash::b200::model::ggml;

namespace {

struct OpenFile {
  std::unique_ptr<GgufReader> file;
};

// Host-only entry points report failures like the rest of the ABI: a status and the thread's message.
template <class F> int host_guarded(F &&f) {
  try {
    return f();
  } catch (const GgufError &e) {
    return sb::fail(SB_ERR_INVALID, "%s", e.what());
  } catch (const std::bad_alloc &) {
    return sb::fail(SB_ERR_OOM, "out of host memory");
  } catch (const std::exception &e) {
    return sb::fail(SB_ERR_INVALID, "%s", e.what());
  }
}

void fill(const GgufTensor &t, SbGgufTensor *out) {
  out->name = t.name.c_str();
  out->type = t.type;
  out->n_dims = uint32_t(t.dims.size());
  for (int d = 0; d < 4; ++d) out->dims[d] = d < int(t.dims.size()) ? t.dims[d] : 1;
  out->data = t.data;
  out->bytes = t.bytes;
}

// The weight format of a ggml tensor type, or -1 for one no kernel of this library reads.
int format_of(uint32_t type) {
  switch (type) {
    case ggml::kF32: return SB_FMT_F32;
    case ggml::kF16: return SB_FMT_F16;
    case ggml::kBF16: return SB_FMT_BF16;
    case ggml::kQ8_0: return SB_FMT_Q80;
    case ggml::kQ4_K: return SB_FMT_Q4K;
    case ggml::kQ6_K: return SB_FMT_Q6K;
    default: return -1;
  }
}

float bf16_to_float(uint16_t v) {
  const uint32_t u = uint32_t(v) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t float_to_bf16(float f) {  // round to nearest even
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u && (u & 0x7fffffu)) return uint16_t((u >> 16) | 0x40u);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}
float half_to_float(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16, exponent = (h >> 10) & 31u, fraction = h & 0x3ffu;
  uint32_t u;
  if (exponent == 31) u = sign | 0x7f800000u | (fraction << 13);
  else if (exponent) u = sign | ((exponent + 112u) << 23) | (fraction << 13);
  else if (!fraction) u = sign;
  else {
    int shift = 0;
    uint32_t f = fraction;
    while (!(f & 0x400u)) f <<= 1, ++shift;
    u = sign | ((113u - uint32_t(shift)) << 23) | ((f & 0x3ffu) << 13);
  }
  float out;
  memcpy(&out, &u, 4);
  return out;
}

// The values of a float tensor (F32, F16 or BF16) as fp32.
std::vector<float> floats_of(const GgufTensor &t) {
  const uint64_t n = t.elements();
  std::vector<float> v(n);
  if (t.type == ggml::kF32) memcpy(v.data(), t.data, n * 4);
  else if (t.type == ggml::kBF16)
    for (uint64_t i = 0; i < n; ++i) v[i] = bf16_to_float(reinterpret_cast<const uint16_t *>(t.data)[i]);
  else if (t.type == ggml::kF16)
    for (uint64_t i = 0; i < n; ++i) v[i] = half_to_float(reinterpret_cast<const uint16_t *>(t.data)[i]);
  else throw GgufError(t.name + " is " + splash::b200::model::ggmlTypeName(t.type) + "; F32, F16 or BF16 expected");
  return v;
}

// Rows of value heads in grouped order: image row `row` (at or past `from`) of head h = (row - from) / head_rows comes
// from the stored row of head (h % per_key) * key_heads + h / per_key.
struct RowOrder {
  uint64_t from = UINT64_MAX;  // UINT64_MAX: as stored
  uint32_t head_rows = 0, key_heads = 0, per_key = 0;
  uint64_t source(uint64_t row) const {
    if (row < from) return row;
    const uint64_t head = (row - from) / head_rows;
    return from + ((head % per_key) * key_heads + head / per_key) * head_rows + (row - from) % head_rows;
  }
};

struct Loader {
  void *target;
  const GgufReader &file;
  SbTargetConfig c;
  std::vector<uint8_t> staging;

  const GgufTensor &need(const std::string &name) const { return file.require(name); }
  void shape(const GgufTensor &t, uint64_t rows, uint64_t columns) const {
    if (t.rows() != rows || t.columns() != columns)
      throw GgufError("unexpected shape for " + t.name + ": [" + std::to_string(t.rows()) + ", " + std::to_string(t.columns()) + "], expected [" +
                      std::to_string(rows) + ", " + std::to_string(columns) + "]");
  }
  // The device tensor `name` of `layer` and its extent.
  uint8_t *device(int layer, const char *name, uint64_t &bytes) const {
    void *p = nullptr;
    if (sb_target_tensor(target, layer, name, &p, &bytes) != SB_OK) throw GgufError(sb_last_error());
    return static_cast<uint8_t *>(p);
  }
  void put(uint8_t *dst, uint64_t capacity, uint64_t offset, const void *src, uint64_t bytes, const std::string &what) const {
    if (offset + bytes > capacity) throw GgufError(what + " does not fit the target's tensor (" + std::to_string(offset + bytes) + " of " + std::to_string(capacity) + " bytes)");
    if (cudaMemcpy(dst + offset, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) throw GgufError("copy of " + what + " to the device failed");
  }
  // Quantized rows [rows, columns] of GGUF tensor `name` into rows [row0, row0 + rows) of the target's `tensor`.
  void rows(int layer, const char *tensor, uint64_t row0, const std::string &name, uint64_t rows_, uint64_t columns, RowOrder order = {}) {
    const GgufTensor &t = need(name);
    shape(t, rows_, columns);
    uint32_t format = 0;
    if (sb_target_tensor_format(target, layer, tensor, &format) != SB_OK) throw GgufError(sb_last_error());
    if (format_of(t.type) != int(format))
      throw GgufError(name + " is " + splash::b200::model::ggmlTypeName(t.type) + " but the target holds it in format " + std::to_string(format) +
                      " (a target made by sb_target_create has one format for its projections, one for the down projections, one for the head and one for the "
                      "embedding; sb_target_create_from_gguf takes every tensor's from the file)");
    const uint64_t rb = sb_row_bytes(format, uint32_t(columns));
    if (!rb || rb * rows_ != t.bytes) throw GgufError(name + ": rows of " + std::to_string(columns) + " inputs are not whole blocks");
    uint64_t capacity = 0;
    uint8_t *dst = device(layer, tensor, capacity);
    if (order.from == UINT64_MAX) return put(dst, capacity, row0 * rb, t.data, t.bytes, name);
    staging.resize(t.bytes);
    for (uint64_t r = 0; r < rows_; ++r) memcpy(staging.data() + r * rb, t.data + order.source(r) * rb, rb);
    put(dst, capacity, row0 * rb, staging.data(), t.bytes, name);
  }
  // A float tensor of `elements` values as fp32 (or bf16) at element offset `at` of the target's `tensor`; rows of
  // `row_elements` values in `order`.
  void values(int layer, const char *tensor, uint64_t at, const std::string &name, uint64_t elements, bool to_bf16 = false, uint64_t row_elements = 1,
              RowOrder order = {}) {
    const GgufTensor &t = need(name);
    if (t.elements() != elements) throw GgufError("unexpected shape for " + name + ": " + std::to_string(t.elements()) + " values, expected " + std::to_string(elements));
    std::vector<float> v = floats_of(t);
    if (order.from != UINT64_MAX) {
      std::vector<float> g(v.size());
      for (uint64_t r = 0; r < elements / row_elements; ++r) memcpy(g.data() + r * row_elements, v.data() + order.source(r) * row_elements, row_elements * 4);
      v.swap(g);
    }
    uint64_t capacity = 0;
    uint8_t *dst = device(layer, tensor, capacity);
    if (!to_bf16) return put(dst, capacity, at * 4, v.data(), elements * 4, name);
    std::vector<uint16_t> h(elements);
    for (uint64_t i = 0; i < elements; ++i) h[i] = float_to_bf16(v[i]);
    put(dst, capacity, at * 2, h.data(), elements * 2, name);
  }

  void layer(uint32_t l) {
    const std::string p = "blk." + std::to_string(l) + ".";
    const uint64_t H = c.hidden, D = c.head_dim;
    values(int(l), "attn_norm", 0, p + "attn_norm.weight", H);
    values(int(l), "ffn_norm", 0, p + "post_attention_norm.weight", H);
    if ((l + 1) % c.attention_interval == 0) {
      const uint64_t q = uint64_t(c.q_heads) * D * (c.gated_attention ? 2 : 1), kv = uint64_t(c.kv_heads) * D;
      rows(int(l), "attn_q", 0, p + "attn_q.weight", q, H);   // (the parts of the fused input projection, in its column order)
      rows(int(l), "attn_k", 0, p + "attn_k.weight", kv, H);
      rows(int(l), "attn_v", 0, p + "attn_v.weight", kv, H);
      values(int(l), "q_norm", 0, p + "attn_q_norm.weight", D);
      values(int(l), "k_norm", 0, p + "attn_k_norm.weight", D);
      rows(int(l), "out_proj", 0, p + "attn_output.weight", H, uint64_t(c.q_heads) * D);
    } else {
      const uint32_t KH = c.gdn_key_heads, VH = c.gdn_value_heads, per_key = VH / KH;
      const uint64_t KW = uint64_t(KH) * 128, VW = uint64_t(VH) * 128, conv = 2 * KW + VW;
      rows(int(l), "attn_qkv", 0, p + "attn_qkv.weight", conv, H, RowOrder{2 * KW, 128, KH, per_key});
      rows(int(l), "attn_gate", 0, p + "attn_gate.weight", VW, H, RowOrder{0, 128, KH, per_key});
      const RowOrder heads{0, 1, KH, per_key};
      values(int(l), "ssm_ab", 0, p + "ssm_beta.weight", uint64_t(VH) * H, false, H, heads);
      values(int(l), "ssm_ab", uint64_t(VH) * H, p + "ssm_alpha.weight", uint64_t(VH) * H, false, H, heads);
      values(int(l), "ssm_conv", 0, p + "ssm_conv1d.weight", conv * 4, true, 4, RowOrder{2 * KW, 128, KH, per_key});
      values(int(l), "ssm_a", 0, p + "ssm_a", VH, false, 1, heads);
      values(int(l), "ssm_dt_bias", 0, p + "ssm_dt.bias", VH, true, 1, heads);
      values(int(l), "ssm_norm", 0, p + "ssm_norm.weight", 128);
      rows(int(l), "out_proj", 0, p + "ssm_out.weight", H, VW);
    }
    if (c.moe_experts) {
      const uint64_t E = c.moe_experts, I = c.moe_intermediate;
      values(int(l), "ffn_router", 0, p + "ffn_gate_inp.weight", E * H);
      values(int(l), "ffn_shared_gate", 0, p + "ffn_gate_inp_shexp.weight", H);
      // Stacked experts [E][rows][columns]: a GGUF holds them as one tensor of three extents, the expert the slowest.
      auto stacked = [&](const char *tensor, const std::string &name, uint64_t rows_, uint64_t columns) {
        const GgufTensor &t = need(name);
        if (t.dims.size() != 3 || t.dims[0] != columns || t.dims[1] != rows_ || t.dims[2] != E) throw GgufError("unexpected shape for " + name);
        if (format_of(t.type) != int(c.fmt_proj)) throw GgufError(name + " is " + splash::b200::model::ggmlTypeName(t.type) + " but the target holds its experts in format " + std::to_string(c.fmt_proj));
        uint64_t capacity = 0;
        uint8_t *dst = device(int(l), tensor, capacity);
        put(dst, capacity, 0, t.data, t.bytes, name);
      };
      stacked("ffn_gate_exps", p + "ffn_gate_exps.weight", I, H);
      stacked("ffn_up_exps", p + "ffn_up_exps.weight", I, H);
      stacked("ffn_down_exps", p + "ffn_down_exps.weight", H, I);
      rows(int(l), "ffn_gate_exps", E * I, p + "ffn_gate_shexp.weight", I, H);   // the shared expert last
      rows(int(l), "ffn_up_exps", E * I, p + "ffn_up_shexp.weight", I, H);
      rows(int(l), "ffn_down_exps", E * H, p + "ffn_down_shexp.weight", H, I);
    } else {
      rows(int(l), "ffn_gate", 0, p + "ffn_gate.weight", c.intermediate, H);
      rows(int(l), "ffn_up", 0, p + "ffn_up.weight", c.intermediate, H);
      rows(int(l), "ffn_down", 0, p + "ffn_down.weight", H, c.intermediate);
    }
  }
  void all() {
    rows(-1, "token_embd", 0, "token_embd.weight", c.vocab, c.hidden);
    values(-1, "output_norm", 0, "output_norm.weight", c.hidden);
    // A GGUF without an output tensor ties the head to the embedding.
    rows(-1, "output", 0, file.find("output.weight") ? "output.weight" : "token_embd.weight", c.vocab, c.hidden);
    for (uint32_t l = 0; l < c.layers; ++l) layer(l);
  }
};

}  // namespace

extern "C" {

int sb_gguf_open(const char *path, void **out_file) {
  if (!path || !out_file) return sb::fail(SB_ERR_INVALID, "sb_gguf_open: null pointer");
  return host_guarded([&] {
    auto f = std::make_unique<OpenFile>();
    f->file = std::make_unique<GgufReader>(path);
    *out_file = f.release();
    return int(SB_OK);
  });
}
int sb_gguf_open_parts(const char *const *paths, uint32_t count, void **out_file) {
  if (!paths || !count || !out_file) return sb::fail(SB_ERR_INVALID, "sb_gguf_open_parts: null pointer or no part");
  return host_guarded([&] {
    std::vector<std::string> all;
    for (uint32_t i = 0; i < count; ++i) {
      if (!paths[i]) throw GgufError("sb_gguf_open_parts: null path");
      all.emplace_back(paths[i]);
    }
    auto f = std::make_unique<OpenFile>();
    f->file = std::make_unique<GgufReader>(all);
    *out_file = f.release();
    return int(SB_OK);
  });
}
int sb_gguf_meta_array(void *file, const char *key, const double **out_values, uint64_t *out_count) {
  if (!file || !key || !out_values || !out_count) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_array: null pointer");
  const std::vector<double> *v = static_cast<OpenFile *>(file)->file->numericArray(key);
  if (!v) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_array: no numeric array %s", key);
  *out_values = v->data(), *out_count = v->size();
  return SB_OK;
}
int sb_gguf_close(void *file) {
  delete static_cast<OpenFile *>(file);
  return SB_OK;
}
int sb_gguf_tensor_count(void *file, uint64_t *out_count) {
  if (!file || !out_count) return sb::fail(SB_ERR_INVALID, "sb_gguf_tensor_count: null pointer");
  *out_count = static_cast<OpenFile *>(file)->file->tensors().size();
  return SB_OK;
}
int sb_gguf_tensor(void *file, uint64_t index, SbGgufTensor *out) {
  if (!file || !out) return sb::fail(SB_ERR_INVALID, "sb_gguf_tensor: null pointer");
  const auto &tensors = static_cast<OpenFile *>(file)->file->tensors();
  if (index >= tensors.size()) return sb::fail(SB_ERR_INVALID, "sb_gguf_tensor: index %llu of %zu tensors", (unsigned long long)index, tensors.size());
  fill(tensors[index], out);
  return SB_OK;
}
int sb_gguf_find(void *file, const char *name, SbGgufTensor *out) {
  if (!file || !name || !out) return sb::fail(SB_ERR_INVALID, "sb_gguf_find: null pointer");
  const GgufTensor *t = static_cast<OpenFile *>(file)->file->find(name);
  if (!t) return sb::fail(SB_ERR_INVALID, "sb_gguf_find: the GGUF has no tensor %s", name);
  fill(*t, out);
  return SB_OK;
}
int sb_gguf_meta_u64(void *file, const char *key, uint64_t *out) {
  if (!file || !key || !out) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_u64: null pointer");
  const auto v = static_cast<OpenFile *>(file)->file->metadata().integer(key);
  if (!v) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_u64: no integer key %s", key);
  *out = *v;
  return SB_OK;
}
int sb_gguf_meta_f64(void *file, const char *key, double *out) {
  if (!file || !key || !out) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_f64: null pointer");
  const auto v = static_cast<OpenFile *>(file)->file->metadata().number(key);
  if (!v) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_f64: no numeric key %s", key);
  *out = *v;
  return SB_OK;
}
int sb_gguf_meta_str(void *file, const char *key, const char **out) {
  if (!file || !key || !out) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_str: null pointer");
  const auto &strings = static_cast<OpenFile *>(file)->file->metadata().strings;
  const auto it = strings.find(std::string_view(key));
  if (it == strings.end()) return sb::fail(SB_ERR_INVALID, "sb_gguf_meta_str: no string key %s", key);
  *out = it->second.c_str();
  return SB_OK;
}

int sb_gguf_target_config(void *file, SbTargetConfig *config) {
  if (!file || !config) return sb::fail(SB_ERR_INVALID, "sb_gguf_target_config: null pointer");
  return host_guarded([&] {
    const GgufReader &f = *static_cast<OpenFile *>(file)->file;
    const std::string arch = f.metadata().architecture();
    if (arch != "qwen35" && arch != "qwen35moe") throw GgufError("GGUF architecture is '" + arch + "'; qwen35 or qwen35moe is loaded");
    auto u = [&](const char *key) {
      const auto v = f.metadata().integer(arch + "." + key);
      if (!v) throw GgufError("the GGUF's metadata has no " + arch + "." + key);
      return uint32_t(*v);
    };
    SbTargetConfig &c = *config;
    c.layers = u("block_count") - uint32_t(f.metadata().integer(arch + ".nextn_predict_layers").value_or(0));
    c.hidden = u("embedding_length");
    c.q_heads = u("attention.head_count"), c.kv_heads = u("attention.head_count_kv"), c.head_dim = u("attention.key_length");
    if (u("attention.value_length") != c.head_dim) throw GgufError("attention.value_length differs from attention.key_length");
    c.rotary_pairs = u("rope.dimension_count") / 2;
    const auto theta = f.metadata().number(arch + ".rope.freq_base");
    if (!theta) throw GgufError("the GGUF's metadata has no " + arch + ".rope.freq_base");
    c.rope_theta = float(*theta);
    if (const auto scaling = f.metadata().text(arch + ".rope.scaling.type"); scaling && *scaling != "none")
      throw GgufError("rope.scaling.type " + *scaling + " (none is run)");
    if (const auto eps = f.metadata().number(arch + ".attention.layer_norm_rms_epsilon"); eps && std::abs(*eps - 1e-6) > 1e-12)
      throw GgufError("attention.layer_norm_rms_epsilon is not 1e-6");
    c.attention_interval = u("full_attention_interval");
    if (u("ssm.conv_kernel") != 4 || u("ssm.state_size") != 128) throw GgufError("ssm.conv_kernel / ssm.state_size other than 4 / 128");
    c.gdn_key_heads = u("ssm.group_count"), c.gdn_value_heads = u("ssm.time_step_rank");
    if (u("ssm.inner_size") != c.gdn_value_heads * 128) throw GgufError("ssm.inner_size is not time_step_rank x 128");
    c.tiled_heads = 1;
    const GgufTensor &embd = f.require("token_embd.weight");
    c.vocab = uint32_t(embd.rows());
    auto format = [&](const GgufTensor &t) {
      const int fmt = format_of(t.type);
      if (fmt < 0) throw GgufError(t.name + " is " + splash::b200::model::ggmlTypeName(t.type) + ", which no kernel of this library reads");
      return uint32_t(fmt);
    };
    c.fmt_embed = format(embd);
    c.fmt_head = format(f.find("output.weight") ? f.require("output.weight") : embd);
    // The formats of the first layer of each kind stand for the model's; the loader refuses a tensor that differs.
    const bool first_is_attention = c.attention_interval == 1;
    const GgufTensor &proj = f.require(first_is_attention ? "blk.0.attn_q.weight" : "blk.0.attn_qkv.weight");
    c.fmt_proj = format(proj);
    if (arch == "qwen35moe") {
      c.moe_experts = u("expert_count"), c.moe_top_k = u("expert_used_count"), c.moe_intermediate = u("expert_feed_forward_length");
      c.intermediate = c.moe_intermediate;  // (a MoE target does not use it, but a target's configuration holds a width)
      c.fmt_down = c.fmt_proj;
    } else {
      c.moe_experts = c.moe_top_k = c.moe_intermediate = 0;
      c.intermediate = u("feed_forward_length");
      c.fmt_down = format(f.require("blk.0.ffn_down.weight"));
    }
    // Gated attention: the queries' projection holds a gate beside every head's queries.
    const uint32_t first_attention = c.attention_interval - 1;
    if (first_attention < c.layers) {
      const uint64_t q_rows = f.require("blk." + std::to_string(first_attention) + ".attn_q.weight").rows();
      if (q_rows != uint64_t(c.q_heads) * c.head_dim && q_rows != 2ull * c.q_heads * c.head_dim) throw GgufError("attn_q holds neither the heads' queries nor queries and gates");
      c.gated_attention = q_rows == 2ull * c.q_heads * c.head_dim;
    }
    return int(SB_OK);
  });
}

int sb_target_create_with_formats(const SbTargetConfig *config, uint32_t (*format_of)(void *, uint32_t, const char *, uint32_t), void *context, void **out_target);

int sb_target_create_from_gguf(void *file, const SbTargetConfig *runtime, void **out_target) {
  SB_NEED_DEVICE();
  if (!file || !runtime || !out_target) return sb::fail(SB_ERR_INVALID, "sb_target_create_from_gguf: null pointer");
  return host_guarded([&] {
    SbTargetConfig c = *runtime;
    int st = sb_gguf_target_config(file, &c);
    if (st != SB_OK) return st;
    const GgufReader &f = *static_cast<OpenFile *>(file)->file;
    // Every projection tensor's type is one a kernel reads: checked here, so that the formats' lookup below cannot fail.
    for (const GgufTensor &t : f.tensors())
      if (t.dims.size() >= 2 && t.name.rfind("blk.", 0) == 0 && t.name.size() > 7 && t.name.compare(t.name.size() - 7, 7, ".weight") == 0 &&
          t.name.find("ssm_conv1d") == std::string::npos && t.name.find("ssm_alpha") == std::string::npos && t.name.find("ssm_beta") == std::string::npos &&
          t.name.find("ffn_gate_inp") == std::string::npos && format_of(t.type) < 0)
        throw GgufError(t.name + " is " + splash::b200::model::ggmlTypeName(t.type) + ", which no kernel of this library reads");
    auto lookup = [](void *context, uint32_t layer, const char *stem, uint32_t configured) -> uint32_t {
      const GgufReader &file_ = *static_cast<const GgufReader *>(context);
      const GgufTensor *t = file_.find("blk." + std::to_string(layer) + "." + stem + ".weight");
      const int fmt = t ? format_of(t->type) : -1;
      return fmt < 0 ? configured : uint32_t(fmt);  // (a missing tensor is reported by name when the file is loaded)
    };
    void *target = nullptr;
    st = sb_target_create_with_formats(&c, lookup, const_cast<GgufReader *>(&f), &target);
    if (st != SB_OK) return st;
    st = sb_target_load_gguf(target, file);
    if (st != SB_OK) {
      const std::string message = sb_last_error();
      sb_target_destroy(target);
      return sb::fail(st, "%s", message.c_str());
    }
    *out_target = target;
    return int(SB_OK);
  });
}

int sb_target_load_gguf(void *target, void *file) {
  SB_NEED_DEVICE();
  if (!target || !file) return sb::fail(SB_ERR_INVALID, "sb_target_load_gguf: null pointer");
  return host_guarded([&] {
    Loader loader{target, *static_cast<OpenFile *>(file)->file, {}, {}};
    if (sb_target_config(target, &loader.c) != SB_OK) return int(SB_ERR_INVALID);
    const SbTargetConfig &c = loader.c;
    if (c.tp_world > 1 || c.ep_world > 1) throw GgufError("sb_target_load_gguf fills a whole model on one GPU (no tensor or expert parallel shares)");
    SbTargetConfig g = c;
    const int st = sb_gguf_target_config(file, &g);
    if (st != SB_OK) return st;
    auto same = [&](const char *what, uint64_t a, uint64_t b) {
      if (a != b) throw GgufError(std::string("the GGUF's ") + what + " is " + std::to_string(b) + ", the target's " + std::to_string(a));
    };
    same("layers", c.layers, g.layers), same("hidden size", c.hidden, g.hidden), same("vocabulary", c.vocab, g.vocab);
    if (!c.moe_experts) same("intermediate size", c.intermediate, g.intermediate);
    same("query heads", c.q_heads, g.q_heads), same("KV heads", c.kv_heads, g.kv_heads);
    same("head dimension", c.head_dim, g.head_dim), same("rotary pairs", c.rotary_pairs, g.rotary_pairs), same("GDN key heads", c.gdn_key_heads, g.gdn_key_heads);
    same("GDN value heads", c.gdn_value_heads, g.gdn_value_heads), same("attention interval", c.attention_interval, g.attention_interval);
    same("experts", c.moe_experts, g.moe_experts), same("experts per token", c.moe_top_k, g.moe_top_k), same("expert width", c.moe_intermediate, g.moe_intermediate);
    same("gated attention", c.gated_attention, g.gated_attention);
    if (c.rope_theta != g.rope_theta) throw GgufError("the GGUF's rope.freq_base differs from the target's");
    if (!c.tiled_heads) throw GgufError("a GGUF's GDN output is in tiled head order: the target needs tiled_heads = 1");
    if (cudaDeviceSynchronize() != cudaSuccess) throw GgufError("the device is not idle");
    loader.all();
    return int(SB_OK);
  });
}

}  // extern "C"
