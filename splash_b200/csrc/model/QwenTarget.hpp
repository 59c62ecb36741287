// The target model's verify step on the host operator layer: the layer loop of the reference's
// Qwen3_5Target::addPrefillLayer run on a decode chunk (runtime/model/QwenTarget.cpp:206-255 GDN mixer,
// :263-347 attention mixer, :351-368 dense FFN, :384-395 and :490-496 final norm and vocabulary projection;
// layer order runtime/model/QwenHybridLayout.hpp:132-135), followed by the step's commit
// (runtime/model/Runtime.cpp:2883-2892: selection, acceptance, path commit).
//
// State kept on the device between steps, so a step replays as a CUDA graph: the lane's committed token
// count, the accepted rows of the previous step's GDN tape, the double-buffered GDN cells (current / next
// alternate by step parity, as do the tapes: runtime/model/Runtime.cpp:2701-2707).
#pragma once
#include <array>
#include <map>
#include <string>
#include <vector>

#include "../ops/GDN.hpp"
#include "../ops/Glue.hpp"
#include "../ops/Linear.hpp"
#include "../ops/MoE.hpp"
#include <functional>

#include "../ops/PagedAttention.hpp"
#include "../ops/Sampling.hpp"
#include "../ops/ExpertParallel.hpp"
#include "../ops/TensorParallel.hpp"

namespace splash::b200::model {

constexpr uint32_t kVerifyRows = 16;

struct LayerWeights {
  bool attention = false;
  ops::NormWeights attnNorm, ffnNorm;
  ops::QuantizedSegment inProj, outProj, ffnGate, ffnUp, ffnDown;
  // The input projection fuses several tensors of a checkpoint (attn_q | attn_k | attn_v, or attn_qkv | attn_gate). Where
  // their formats differ (a Q4_K_M file keeps attn_v in Q6_K) it is held as one segment per tensor, each writing its
  // columns of the fused output in a launch of its own, and inProj stays empty (the reference's fused column segments,
  // runtime/ops/LinearGguf.cpp:25,78-86).
  std::vector<ops::QuantizedSegment> inParts;
  std::vector<const ops::QuantizedSegment *> inSegments() const {
    std::vector<const ops::QuantizedSegment *> v;
    if (inParts.empty()) v.push_back(&inProj);
    for (const ops::QuantizedSegment &part : inParts) v.push_back(&part);
    return v;
  }
  ops::MoeWeights moe;  // MoE feed-forward block (then ffnGate / ffnUp / ffnDown are empty)
  // GDN
  Buffer ssmAb, ssmConv, ssmA, ssmDtBias, ssmNorm;
  std::array<ops::GdnCell, 2> cells;
  std::array<ops::GdnTape, 2> tapes;
  // attention
  Buffer qNorm, kNorm;
  ops::kv::LayerPages pages;
};

// Rank tp_rank's share of the whole model's dimensions (include/splash_b200.h, "tensor parallelism"): heads in
// contiguous ranges, a KV head shared by tp_world / kv_heads ranks when there are more ranks than KV heads, the
// intermediate width in super-blocks of 256 and the vocabulary in units of 64, the first ranks taking the remainder.
inline SbTargetShare shareOf(const SbTargetConfig &c) {
  const uint32_t W = std::max(1u, c.tp_world), r = c.tp_rank;
  if (W > 8 || r >= W) throw std::invalid_argument("QwenTarget: rank " + std::to_string(r) + " of " + std::to_string(W) + " ranks (at most 8)");
  auto even = [&](uint32_t total, const char *what) {
    if (total % W) throw std::invalid_argument(std::string("QwenTarget: ") + what + " do not divide among the ranks");
    return total / W;
  };
  auto ragged = [&](uint32_t units, uint32_t &first) {
    const uint32_t base = units / W, extra = units % W;
    first = r * base + std::min(r, extra);
    return base + (r < extra ? 1u : 0u);
  };
  SbTargetShare s{};
  s.q_heads = even(c.q_heads, "query heads"), s.q_head0 = r * s.q_heads;
  if (c.kv_heads >= W) {
    s.kv_heads = even(c.kv_heads, "KV heads"), s.kv_head0 = r * s.kv_heads;
  } else {
    if (!c.kv_heads || W % c.kv_heads) throw std::invalid_argument("QwenTarget: the ranks do not divide among the KV heads");
    s.kv_heads = 1, s.kv_head0 = r / (W / c.kv_heads);
  }
  s.gdn_key_heads = even(c.gdn_key_heads, "GDN key heads"), s.gdn_key_head0 = r * s.gdn_key_heads;
  s.gdn_value_heads = even(c.gdn_value_heads, "GDN value heads"), s.gdn_value_head0 = r * s.gdn_value_heads;
  uint32_t first = 0;
  s.intermediate = 256 * ragged(c.intermediate / 256, first), s.intermediate0 = 256 * first;
  const uint32_t units = ragged((c.vocab + 63) / 64, first);
  s.vocab0 = std::min(c.vocab, 64 * first), s.vocab = std::min(c.vocab, 64 * (first + units)) - s.vocab0;
  if (W > 1 && (!s.intermediate || !s.vocab || c.vocab % 4)) throw std::invalid_argument("QwenTarget: a rank without a share, or a vocabulary that is not a multiple of 4");
  return s;
}

class QwenTarget {
 public:
  // formatOf (optional): the weight format of a checkpoint tensor of a layer by its GGUF stem ("attn_q", "attn_k", "attn_v",
  // "attn_qkv", "attn_gate", "attn_output", "ssm_out", "ffn_gate", "ffn_up", "ffn_down"), given the configuration's format
  // for its kind; without it every tensor takes the configuration's.
  using FormatOf = std::function<uint32_t(uint32_t layer, const char *stem, uint32_t configured)>;
  explicit QwenTarget(const SbTargetConfig &whole, const FormatOf &formatOf = {});
  // The format of the rows behind a weight tensor's name (find), SB_FMT_F32 for the fp32 tensors; false for no such tensor.
  bool formatOfTensor(int layer, const std::string &name, uint32_t &format) const;

  // Appends one verify step of `rows` rows to the graph. `parity` selects which GDN cell is current.
  // `treeGiven`: the `tree` buffer holds the block's rows (a tree); otherwise the step writes a chain's there.
  // `keepPending` (only without `advance`): the lane's pending GDN rows stay as they are instead of being cleared, so
  // a held lane folds the same rows in every step (a steady-state timing loop).
  // `draws`: sampled rows take their children from the `candidates` / `candidateQ` / `draws` buffers (the draft's
  // candidates per row, their probabilities and the children it drew) instead of the next row's input token.
  void encodeVerify(CommandGraph &graph, uint32_t rows, float temperature, uint32_t parity, bool advance, bool treeGiven = false,
                    bool keepPending = false, bool draws = false);

  const SbTargetConfig &config() const { return cfg_; }   // the whole model
  const SbTargetConfig &local() const { return loc_; }    // this rank's heads and intermediate width (the vocabulary stays whole)
  const SbTargetShare &share() const { return share_; }
  ops::TensorParallel *tensorParallel() { return tp_.get(); }
  ops::ExpertParallel *expertParallel() { return ep_.get(); }
  // Exchanges of one step: one after every out_proj and down, one for the logits.
  uint32_t exchangesPerStep() const { return 2 * cfg_.layers + 1; }
  bool find(int layer, const std::string &name, Buffer &out) const;
  std::vector<struct InputPart> inputParts(const LayerWeights &w) const;
  std::vector<LayerWeights> &layers() { return layers_; }

  // Bytes one step streams: weights once, the visible INT8 cache, the GDN state in and out.
  // (MoE blocks: a step reads the routed experts only, every route its own expert's three matrices)
  // (the rows of several lanes are grouped by expert: every expert the rank holds streams once)
  uint64_t weightBytes(uint32_t rows = kVerifyRows) const {
    const uint64_t experts = wide_ ? (ep_ ? ep_->local().expertsTotal() : moe_.expertsTotal()) : uint64_t(rows) * moe_.routes();
    return weightBytes_ + uint64_t(moeLayers_) * experts * moeExpertBytes_;
  }
  uint64_t kvBytes(uint32_t visible) const;
  uint64_t stateBytes() const;

  // Sampling penalties of the lane (off by default): `penaltyWords` holds, per vocabulary token, the output's count and
  // the prompt bit (runtime/metal/abi/Sampling.h:124-125); the host keeps it current between steps.
  ops::SamplingPenalties penalties;
  Buffer penaltyWords;
  Buffer pendingPath;  // the row mask, in the previous step's tape, of the path it accepted (tree steps)
  Buffer candidates, candidateQ, draws;  // per row: 16 draft candidates (u32), their draft probabilities (fp32), 4 drawn children (u8)
  Buffer tokens, uniforms, committed, pendingRows, results, selected, logits, hidden[2], tree, positions, invFreq, cosine, sine;
  uint32_t committedHost = 0;  // bound of the device's committed word(s), for extents and the attention plan
  uint32_t step = 0;
  uint32_t lanes() const { return lanes_; }
  // The images of the Q6_K / NVFP4 projections are out of date: set when a weight tensor's address is handed out or the
  // weights are filled, cleared by buildImages, which the next step runs first.
  bool imagesStale = true;
  // Measurements with synthetic routing: the blocks route by the host's `moe_scores` instead of their router's scores.
  bool routerScoresGiven = false;
  // Admission (sb_target_set_admission): the rows' constraint masks, filled by the host when `constrained`; the tokens no row
  // selects.
  Buffer constraintMasks, excludedTokens;  // u32 [16 x lanes][maskWords()]; u32 [16]
  bool constrained = false;
  uint32_t excludedCount = 0;
  // A policy a lane (sb_target_set_lane_policies): SbLanePolicy [lanes] on the device, read by the selection when it runs.
  Buffer lanePolicies;
  bool lanePoliciesSet = false;
  bool manyRowStep() const { return wide_; }
  // The end of a sampled row's distribution (sb_target_set_policy): min-p, then top-k, then the top-p nucleus; off at 0 / 0 / 1.
  float minP = 0.0f, topP = 1.0f;
  uint32_t topK = 0;
  uint32_t maskWords() const { return (cfg_.vocab + 31) / 32; }
  Buffer tickets;  // u32 [64]: the selection launch's count of finished rows a lane (zero between launches; zeroed at creation)
  bool promptBlock = false;  // the step being encoded commits every row of its block (a block of prompt tokens)
  Buffer stopTokens;         // u32 [16]: tokens that end a lane's retained path (sb_target_set_stop_tokens)
  uint32_t stopCount = 0;
  Buffer remaining;          // u32 [64]: the tokens each lane's request may still take (0xFFFFFFFF: no bound)
  Buffer laneRows;           // u32 [64]: the rows of each lane's block, for steps whose lanes' blocks differ in length
  bool raggedStep = false;   // the step being encoded reads laneRows
  void buildImages(void *stream) {
    if (wide_)
      for (LayerWeights &w : layers_)
      {
        for (const ops::QuantizedSegment *s : {&w.outProj, &w.ffnGate, &w.ffnUp, &w.ffnDown}) ops::Linear::buildImage(stream, *s);
        for (const ops::QuantizedSegment *s : w.inSegments()) ops::Linear::buildImage(stream, *s);
      }
    if (wide_) ops::Linear::buildImage(stream, output_);
    imagesStale = false;
  }
  uint32_t pagesPerLane() const { return pagesPerLane_; }

 private:
  ops::QuantizedSegment segment(uint32_t n, uint32_t k, uint32_t format);
  Buffer floats(size_t count) { return Buffer::allocate(count * 4); }

  ops::MoeShape moe_;
  std::unique_ptr<ops::ExpertParallel> ep_;
  Buffer moeScores_, moeScoresGiven_, moeSelected_, moeWeights_, moeScratch_;
  SbTargetConfig cfg_, loc_;
  SbTargetShare share_{};
  std::unique_ptr<ops::TensorParallel> tp_;
  ops::GdnShape gdn_;
  ops::kv::Layout kv_;
  std::vector<LayerWeights> layers_;
  ops::EmbeddingWeights embedding_;
  ops::NormWeights outputNorm_;
  ops::QuantizedSegment output_;
  Buffer packed_, gates_, mixed_, queries_, act_, normed_, prepared_[2], pageTable_, sampleWorkspace_;
  Buffer partials_;  // fp32 [kMaxPartialSlices][16][hidden]: k-slice sums of out_proj / down awaiting their consumer
  static constexpr uint32_t kMaxPartialSlices = 16;
  uint32_t packedStride_ = 0;
  uint32_t lanes_ = 1, pagesPerLane_ = 0;
  bool wide_ = false;  // the step runs on the many-row projection kernel (several lanes, or NVFP4 projections)
  bool mixedInputs_ = false;  // some layer's input projection is held as segments of several formats (LayerWeights::inParts)
  Buffer preparedOther_;      // then: the layer's input converted for the other fragment layout
  Buffer widePrepared_[2], widePartials_;  // conversions for the many-row projection kernel (steps of several lanes)
  void encodeVerifyLanes(CommandGraph &graph, uint32_t rows, float temperature, uint32_t parity, bool advance, bool treeGiven, bool keepPending,
                         bool drawsGiven);
  uint64_t weightBytes_ = 0, moeExpertBytes_ = 0;
  uint32_t moeLayers_ = 0;
};

inline ops::QuantizedSegment QwenTarget::segment(uint32_t n, uint32_t k, uint32_t format) {
  ops::QuantizedSegment s;
  s.outputSize = n, s.inputSize = k, s.format = format, s.columnOffset = 0;
  const size_t bytes = size_t(n) * sb_row_bytes(format, k);
  if (!bytes) throw std::invalid_argument("QwenTarget: a projection's width is not whole blocks of its format");
  s.rows = Buffer::allocate(bytes);
  if (wide_ && format != SB_FMT_Q4K) {
    s.image = Buffer::allocate(ops::Linear::imageBytes(s));
    weightBytes_ += s.image.bytes();  // (what a step streams)
  } else {
    weightBytes_ += bytes;
  }
  return s;
}

inline QwenTarget::QwenTarget(const SbTargetConfig &whole, const FormatOf &formatOf) : cfg_(whole), loc_(whole) {
  share_ = shareOf(whole);
  loc_.q_heads = share_.q_heads, loc_.kv_heads = share_.kv_heads, loc_.gdn_key_heads = share_.gdn_key_heads;
  loc_.gdn_value_heads = share_.gdn_value_heads, loc_.intermediate = share_.intermediate;
  const SbTargetConfig &c = loc_;
  lanes_ = std::max(1u, whole.lanes);
  const uint32_t L = lanes_;
  if (L > 32) throw std::invalid_argument("QwenTarget: " + std::to_string(L) + " lanes (up to 32)");
  // The many-row projection kernel carries steps of several lanes (16 x lanes rows) and every NVFP4 projection; it takes
  // Q4_K rows as they are and Q6_K / NVFP4 rows as images made when the weights change (buildImages).
  const bool fp4 = whole.fmt_proj == SB_FMT_NVFP4 || whole.fmt_down == SB_FMT_NVFP4 || whole.fmt_head == SB_FMT_NVFP4;
  wide_ = L > 1 || fp4;
  if (wide_) {
    if (whole.tp_world > 1) throw std::invalid_argument("QwenTarget: several lanes and NVFP4 projections are offered on one GPU");
    if (whole.moe_experts && fp4) throw std::invalid_argument("QwenTarget: MoE experts are Q4_K");
    for (uint32_t f : {whole.fmt_proj, whole.fmt_down, whole.fmt_head})
      if (f != SB_FMT_Q4K && f != SB_FMT_Q6K && f != SB_FMT_Q80 && f != SB_FMT_NVFP4)
        throw std::invalid_argument("QwenTarget: several lanes and NVFP4 models take Q4_K, Q6_K, Q8_0 and NVFP4 projections (fmt_proj, fmt_down, fmt_head)");
  }
  if (whole.tp_world > 1) tp_ = std::make_unique<ops::TensorParallel>(whole.tp_world, whole.tp_rank, whole.hidden, whole.vocab);
  if (!c.layers || !c.hidden || !c.vocab || !c.intermediate || !c.attention_interval)
    throw std::invalid_argument("QwenTarget: empty configuration");
  if (c.hidden % 256 || c.intermediate % 256) throw std::invalid_argument("QwenTarget: hidden and intermediate sizes are multiples of 256");
  if (c.moe_experts) {
    if (tp_) throw std::invalid_argument("QwenTarget: MoE blocks are not offered with tensor parallelism");
    if (c.fmt_proj != SB_FMT_Q4K) throw std::invalid_argument("QwenTarget: MoE experts are Q4_K");
    moe_.experts = moe_.slots = c.moe_experts, moe_.topK = c.moe_top_k, moe_.hidden = c.hidden, moe_.intermediate = c.moe_intermediate;
    moe_.sharedExpert = moe_.sharedGate = true;
    if (!c.moe_top_k || c.moe_top_k > c.moe_experts || c.moe_experts > 256 || !c.moe_intermediate || c.moe_intermediate % 256)
      throw std::invalid_argument("QwenTarget: MoE shape (up to 256 experts, top_k of them, intermediate a multiple of 256)");
  }
  if (whole.ep_world > 1) {
    // Expert parallelism: this rank's lanes, its share of every block's experts; the blocks' rows meet their experts
    // through the ranks' exchange windows (ops::ExpertParallel).
    if (!c.moe_experts || !wide_) throw std::invalid_argument("QwenTarget: expert parallelism is offered for MoE models stepping several lanes");
    ep_ = std::make_unique<ops::ExpertParallel>(whole.ep_world, whole.ep_rank, kVerifyRows * L, moe_);
  }
  gdn_.keyHeads = c.gdn_key_heads, gdn_.valueHeads = c.gdn_value_heads;
  kv_.kvHeads = c.kv_heads, kv_.headDimension = c.head_dim, kv_.pageTokens = c.page_tokens, kv_.halfScales = c.kv_scale_f16 != 0;
  const uint32_t H = c.hidden, D = c.head_dim;
  const uint32_t attnIn = c.q_heads * (c.gated_attention ? 2 * D : D) + 2 * c.kv_heads * D;
  const uint32_t gdnIn = gdn_.convolutionWidth() + gdn_.valueWidth();
  pagesPerLane_ = (c.max_context + kVerifyRows + c.page_tokens - 1) / c.page_tokens;
  const uint32_t pages = pagesPerLane_ * L;  // a layer's pool: the lanes' pages one lane after the other
  layers_.resize(c.layers);
  for (uint32_t l = 0; l < c.layers; ++l) {
    LayerWeights &w = layers_[l];
    w.attention = (l + 1) % c.attention_interval == 0;
    w.attnNorm.buffer = floats(H), w.ffnNorm.buffer = floats(H);
    weightBytes_ += 2 * size_t(H) * 4;
    auto fmt = [&](const char *stem, uint32_t configured) { return formatOf ? formatOf(l, stem, configured) : configured; };
    // The fused input projection of `parts` (stem, rows): one segment when the tensors share a format, else one a tensor.
    auto fused = [&](std::initializer_list<std::pair<const char *, uint32_t>> parts) {
      bool same = true;
      uint32_t total = 0;
      for (const auto &[stem, n] : parts) same = same && fmt(stem, c.fmt_proj) == fmt(parts.begin()->first, c.fmt_proj), total += n;
      if (same) {
        w.inProj = segment(total, H, fmt(parts.begin()->first, c.fmt_proj));
        return;
      }
      if (whole.tp_world > 1) throw std::invalid_argument("QwenTarget: an input projection of several formats is not divided over tensor-parallel ranks");
      uint32_t at = 0;
      for (const auto &[stem, n] : parts) {
        w.inParts.push_back(segment(n, H, fmt(stem, c.fmt_proj)));
        w.inParts.back().columnOffset = at;
        at += n;
      }
      mixedInputs_ = true;
    };
    if (w.attention) {
      ++kv_.attentionLayers;
      fused({{"attn_q", c.q_heads * (c.gated_attention ? 2 * D : D)}, {"attn_k", c.kv_heads * D}, {"attn_v", c.kv_heads * D}});
      w.outProj = segment(H, c.q_heads * D, fmt("attn_output", c.fmt_proj));
      w.qNorm = floats(D), w.kNorm = floats(D);
      w.pages.pages = pages;
      w.pages.keys = Buffer::allocate(pages * kv_.dataBytesPerLayerPage());
      w.pages.values = Buffer::allocate(pages * kv_.dataBytesPerLayerPage());
      w.pages.keyScales = Buffer::allocate(pages * kv_.scaleBytesPerLayerPage());
      w.pages.valueScales = Buffer::allocate(pages * kv_.scaleBytesPerLayerPage());
    } else {
      fused({{"attn_qkv", gdn_.convolutionWidth()}, {"attn_gate", gdn_.valueWidth()}});
      w.outProj = segment(H, gdn_.valueWidth(), fmt("ssm_out", c.fmt_proj));
      w.ssmAb = floats(size_t(2) * gdn_.valueHeads * H);
      weightBytes_ += size_t(2) * gdn_.valueHeads * H * 4;
      w.ssmConv = Buffer::allocate(size_t(gdn_.convolutionWidth()) * 4 * 2);
      w.ssmA = floats(gdn_.valueHeads), w.ssmDtBias = Buffer::allocate(gdn_.valueHeads * 2), w.ssmNorm = floats(128);
      for (int i = 0; i < 2; ++i) {  // (arrays over the lanes)
        w.cells[i].state = Buffer::allocate(gdn_.stateBytes() * L);
        w.cells[i].convolution = Buffer::allocate(gdn_.convolutionStateBytes() * L);
        w.tapes[i] = ops::GdnTape::allocate(gdn_, kVerifyRows * L);
      }
    }
    if (c.moe_experts) {
      const uint32_t total = ep_ ? ep_->local().expertsTotal() : moe_.expertsTotal();  // (the router stays whole)
      w.moe.router = floats(size_t(moe_.slots) * H), w.moe.sharedGate = floats(H);
      const size_t pair = size_t(total) * moe_.intermediate * sb_row_bytes(c.fmt_proj, H), down = size_t(total) * H * sb_row_bytes(c.fmt_proj, moe_.intermediate);
      w.moe.gate = Buffer::allocate(pair), w.moe.up = Buffer::allocate(pair), w.moe.down = Buffer::allocate(down);
      weightBytes_ += size_t(moe_.slots + 1) * H * 4;
      moeExpertBytes_ = (2 * pair + down) / total;
      ++moeLayers_;
    } else {
      if (fmt("ffn_gate", c.fmt_proj) != fmt("ffn_up", c.fmt_proj))
        throw std::invalid_argument("QwenTarget: a layer's ffn_gate and ffn_up tensors share one format (they run as one launch)");
      w.ffnGate = segment(c.intermediate, H, fmt("ffn_gate", c.fmt_proj));
      w.ffnUp = segment(c.intermediate, H, fmt("ffn_up", c.fmt_proj));
      w.ffnDown = segment(H, c.intermediate, fmt("ffn_down", c.fmt_down));
    }
  }
  embedding_.rows = Buffer::allocate(size_t(c.vocab) * sb_row_bytes(c.fmt_embed, H));
  embedding_.vocabulary = c.vocab, embedding_.width = H, embedding_.format = c.fmt_embed;
  outputNorm_.buffer = floats(H);
  output_ = segment(share_.vocab, H, c.fmt_head);

  packedStride_ = std::max(attnIn, gdnIn);
  const size_t R = size_t(kVerifyRows) * L;  // row slots of a step
  packed_ = Buffer::allocate(R * packedStride_ * 2);
  gates_ = Buffer::allocate(R * 2 * std::max(1u, gdn_.valueHeads) * 2);
  mixed_ = Buffer::allocate(R * std::max(gdn_.valueWidth(), c.q_heads * D) * 2);
  queries_ = Buffer::allocate(R * c.q_heads * D * 2);
  act_ = Buffer::allocate(R * c.intermediate * 2);
  normed_ = Buffer::allocate(R * H * 2);
  partials_ = Buffer::allocate(size_t(kMaxPartialSlices) * 16 * H * 4);
  const uint32_t widest = std::max(std::max(H, c.intermediate), std::max(gdn_.valueWidth(), c.q_heads * D));
  for (auto &p : prepared_) p = Buffer::allocate(ops::Linear::preparedBytes((widest + 255) / 256 * 256));
  if (mixedInputs_) preparedOther_ = Buffer::allocate(ops::Linear::preparedBytes(H));
  if (wide_) {
    for (auto &p : widePrepared_) p = Buffer::allocate(ops::Linear::wideBytes(uint32_t(R), (widest + 255) / 256 * 256));
    const uint32_t splits = std::max(ops::Linear::wideSplits(H, c.intermediate), std::max(ops::Linear::wideSplits(H, gdn_.valueWidth()), ops::Linear::wideSplits(H, c.q_heads * D)));
    widePartials_ = Buffer::allocate(size_t(splits) * R * H * 4);
  }
  for (auto &h : hidden) h = Buffer::allocate(R * H * 2);
  logits = tp_ ? tp_->gathered() : Buffer::allocate(R * c.vocab * 4);
  tokens = Buffer::allocate(R * 4), selected = Buffer::allocate(R * 4), results = Buffer::allocate(16 * L);
  uniforms = Buffer::allocate(80 * 4 * L), committed = Buffer::allocate(4 * L), pendingRows = Buffer::allocate(4 * L), pendingPath = Buffer::allocate(4 * L);
  tree = Buffer::allocate(R * 8), positions = Buffer::allocate(R * 4);
  invFreq = Buffer::allocate(std::max(1u, c.rotary_pairs) * 4);
  cosine = Buffer::allocate(R * std::max(1u, c.rotary_pairs) * 4);
  sine = Buffer::allocate(R * std::max(1u, c.rotary_pairs) * 4);
  pageTable_ = Buffer::allocate(size_t(pages) * 4);
  sampleWorkspace_ = Buffer::allocate(ops::Sampling::workspace(uint32_t(R), c.vocab));
  tickets = Buffer::allocate(64 * 4);
  laneRows = Buffer::allocate(64 * 4);
  remaining = Buffer::allocate(64 * 4);
  stopTokens = Buffer::allocate(16 * 4);
  penaltyWords = Buffer::allocate(size_t(c.vocab) * 4 * L);
  lanePolicies = Buffer::allocate(sizeof(SbLanePolicy) * 64);
  constraintMasks = Buffer::allocate(size_t(kVerifyRows) * L * ((c.vocab + 31) / 32) * 4), excludedTokens = Buffer::allocate(16 * 4);
  candidates = Buffer::allocate(R * 16 * 4), candidateQ = Buffer::allocate(R * 16 * 4), draws = Buffer::allocate(R * 4);
  if (c.moe_experts) {
    moeScores_ = Buffer::allocate(R * moe_.slots * 4), moeScoresGiven_ = Buffer::allocate(R * moe_.slots * 4);
    moeSelected_ = Buffer::allocate(R * moe_.routes() * 4), moeWeights_ = Buffer::allocate(R * moe_.routes() * 4);
    moeScratch_ = Buffer::allocate(ops::MoE::scratchBytes(moe_, uint32_t(R)));
  }
}

inline uint64_t QwenTarget::kvBytes(uint32_t visible) const {  // (every lane at `visible` tokens)
  return uint64_t(lanes_) * kv_.attentionLayers * 2 * visible * kv_.kvHeads * (kv_.headDimension + (kv_.halfScales ? 2 : 4));
}
inline uint64_t QwenTarget::stateBytes() const {
  uint64_t gdnLayers = 0;
  for (const LayerWeights &w : layers_) gdnLayers += !w.attention;
  return gdnLayers * 2 * gdn_.stateBytes() * lanes_;
}

// The checkpoint tensors behind a layer's input projection: their stems, rows (a view of the fused segment, or the
// tensor's own segment) and formats, in the order of the fused output's columns.
struct InputPart {
  const char *stem;
  Buffer rows;
  uint32_t format;
};
inline std::vector<InputPart> QwenTarget::inputParts(const LayerWeights &w) const {
  const SbTargetConfig &c = loc_;
  const uint32_t D = c.head_dim;
  std::vector<std::pair<const char *, uint32_t>> parts;
  if (w.attention) parts = {{"attn_q", c.q_heads * (c.gated_attention ? 2 * D : D)}, {"attn_k", c.kv_heads * D}, {"attn_v", c.kv_heads * D}};
  else parts = {{"attn_qkv", gdn_.convolutionWidth()}, {"attn_gate", gdn_.valueWidth()}};
  std::vector<InputPart> out;
  size_t at = 0;
  for (size_t i = 0; i < parts.size(); ++i) {
    if (!w.inParts.empty()) {
      out.push_back({parts[i].first, w.inParts[i].rows, w.inParts[i].format});
      continue;
    }
    const size_t bytes = size_t(parts[i].second) * sb_row_bytes(w.inProj.format, c.hidden);
    out.push_back({parts[i].first, w.inProj.rows.view(at, bytes), w.inProj.format});
    at += bytes;
  }
  return out;
}
inline bool QwenTarget::formatOfTensor(int layer, const std::string &name, uint32_t &format) const {
  if (layer < 0) {
    if (name == "token_embd") format = cfg_.fmt_embed;
    else if (name == "output") format = output_.format;
    else return false;
    return true;
  }
  if (size_t(layer) >= layers_.size()) return false;
  const LayerWeights &w = layers_[layer];
  for (const InputPart &part : inputParts(w))
    if (name == part.stem) return format = part.format, true;
  if (name == "in_proj" && w.inParts.empty()) return format = w.inProj.format, true;
  if (name == "out_proj") return format = w.outProj.format, true;
  if (cfg_.moe_experts) {
    if (name == "ffn_gate_exps" || name == "ffn_up_exps" || name == "ffn_down_exps") return format = cfg_.fmt_proj, true;
    return false;
  }
  if (name == "ffn_gate") return format = w.ffnGate.format, true;
  if (name == "ffn_up") return format = w.ffnUp.format, true;
  if (name == "ffn_down") return format = w.ffnDown.format, true;
  return false;
}

inline bool QwenTarget::find(int layer, const std::string &name, Buffer &out) const {
  if (layer < 0) {
    const std::map<std::string, Buffer> g = {{"token_embd", embedding_.rows}, {"output_norm", outputNorm_.buffer}, {"output", output_.rows},
                                             {"logits", logits}, {"selected", selected}, {"results", results}, {"hidden", hidden[0]},
                                             {"hidden1", hidden[1]}, {"tokens", tokens}, {"uniforms", uniforms}, {"committed", committed},
                                             {"pending_rows", pendingRows}, {"tree", tree}, {"page_table", pageTable_}, {"inv_freq", invFreq},
                                             {"positions", positions}, {"packed", packed_}, {"mixed", mixed_}, {"act", act_}, {"penalty_words", penaltyWords}, {"constraint_masks", constraintMasks}, {"remaining", remaining},
                                             {"candidates", candidates}, {"candidate_q", candidateQ}, {"draws", draws}, {"pending_path", pendingPath},
                                             {"moe_scores", moeScoresGiven_}};
    auto it = g.find(name);
    if (it == g.end()) return false;
    out = it->second;
    return true;
  }
  if (size_t(layer) >= layers_.size()) return false;
  const LayerWeights &w = layers_[layer];
  std::map<std::string, Buffer> m = {{"attn_norm", w.attnNorm.buffer}, {"ffn_norm", w.ffnNorm.buffer},
                                     {"out_proj", w.outProj.rows}, {"ffn_gate", w.ffnGate.rows}, {"ffn_up", w.ffnUp.rows},
                                     {"ffn_down", w.ffnDown.rows}};
  // The fused input projection whole (when it is one segment) and tensor by tensor under the checkpoint's stems.
  for (const InputPart &part : inputParts(w)) m.insert({part.stem, part.rows});
  if (w.inParts.empty()) m.insert({"in_proj", w.inProj.rows});
  // (the images the many-row kernel reads, where a projection has one: for measurements of that kernel by itself)
  for (auto &[tensor, seg] : {std::pair<const char *, const ops::QuantizedSegment &>{"ffn_gate_image", w.ffnGate}, {"ffn_up_image", w.ffnUp}, {"ffn_down_image", w.ffnDown}})
    if (seg.image) m.insert({tensor, seg.image});
  if (cfg_.moe_experts)
    m.insert({{"ffn_router", w.moe.router}, {"ffn_shared_gate", w.moe.sharedGate}, {"ffn_gate_exps", w.moe.gate}, {"ffn_up_exps", w.moe.up},
              {"ffn_down_exps", w.moe.down}});
  if (w.attention) {
    m.insert({{"q_norm", w.qNorm}, {"k_norm", w.kNorm}, {"kv_k", w.pages.keys}, {"kv_v", w.pages.values},
              {"kv_ks", w.pages.keyScales}, {"kv_vs", w.pages.valueScales}});
  } else {
    m.insert({{"ssm_ab", w.ssmAb}, {"ssm_conv", w.ssmConv}, {"ssm_a", w.ssmA}, {"ssm_dt_bias", w.ssmDtBias}, {"ssm_norm", w.ssmNorm},
              {"state0", w.cells[0].state}, {"state1", w.cells[1].state}, {"conv0", w.cells[0].convolution},
              {"conv1", w.cells[1].convolution}});
    for (int i = 0; i < 2; ++i) {
      const std::string s = std::to_string(i);
      m.insert({{"tape_inputs" + s, w.tapes[i].inputs}, {"tape_k" + s, w.tapes[i].keys}, {"tape_v" + s, w.tapes[i].values},
                {"tape_beta" + s, w.tapes[i].beta}, {"tape_decay" + s, w.tapes[i].decay}});
    }
  }
  auto it = m.find(name);
  if (it == m.end()) return false;
  out = it->second;
  return true;
}

// Launched before and after the operator sequence (sb_target.cu).
void launchStepBegin(CommandGraph &graph, const Buffer &committed, const Buffer &tree, const Buffer &positions, uint32_t rows, bool treeGiven,
                     uint32_t lanes = 1);
// (with a tensor-parallel group the step's end also advances the group's exchange count by `exchanges`)
// advance: 0 the lane holds its position and its pending rows are cleared, 1 it commits, 2 it holds and keeps them,
// 3 | rows << 8 it commits all `rows` rows of its block
void launchStepEnd(CommandGraph &graph, const Buffer &results, const Buffer &committed, const Buffer &pendingRows, const Buffer &pendingPath,
                   uint32_t advance, void *tpGroup, uint32_t exchanges, uint32_t lanes = 1);

inline void QwenTarget::encodeVerify(CommandGraph &graph, uint32_t rows, float temperature, uint32_t parity, bool advance, bool treeGiven, bool keepPending, bool drawsGiven) {
  using namespace ops;
  if (rows < 1 || rows > kVerifyRows) throw std::invalid_argument("QwenTarget::encodeVerify: 1 to 16 rows");
  if (committedHost + rows > cfg_.max_context + kVerifyRows) throw std::invalid_argument("QwenTarget::encodeVerify: past the context bound");
  if (wide_) {
    return encodeVerifyLanes(graph, rows, temperature, parity, advance, treeGiven, keepPending, drawsGiven);
  }
  const SbTargetConfig &c = loc_;
  const uint32_t H = c.hidden, D = c.head_dim;
  if (tp_ && !tp_->connected()) throw std::invalid_argument("QwenTarget::encodeVerify: the tensor-parallel ranks are not connected");
  uint32_t exchange = 0;  // the place of the next exchange among the step's
  launchStepBegin(graph, committed, tree, positions, rows, treeGiven);
  if (c.rotary_pairs) RoPE::addTreeTables(graph, positions, invFreq, cosine, sine, rows, 1.0f, c.rotary_pairs);
  Embedding::add(graph, tokens, embedding_, hidden[0], rows, H);
  uint32_t cur = 0;
  // out_proj and down leave their k-slices' sums unreduced (Epilogue::Partials); the conversion of the next
  // projection's input adds them and the residual and writes the new hidden state, so no projection ends on a
  // split-K exchange. `pending` = slices waiting in partials_ whose residual is hidden[cur] and whose sum goes to
  // hidden[cur ^ 1].
  uint32_t pending = 0;
  auto convert = [&](const Buffer *norm, uint32_t format, const Buffer &scratch, const Buffer *normedOutput) {
    if (!pending) return Linear::prepare(graph, hidden[cur], rows, H, H, norm, format, scratch, normedOutput);
    PreparedInput in = tp_ ? tp_->prepareSum(graph, exchange++, partials_, pending, H, hidden[cur], hidden[cur ^ 1], rows, H, H, norm, format, scratch, normedOutput)
                           : Linear::prepareSum(graph, partials_, pending, H, hidden[cur], hidden[cur ^ 1], rows, H, H, norm, format, scratch, normedOutput);
    cur ^= 1;
    pending = 0;
    return in;
  };
  auto project = [&](const QuantizedSegment &seg, uint32_t inputSize, const PreparedInput &in) {
    Projection proj{H, inputSize, Destination::BFloat16, {seg}};
    LinearPlan plan = Linear::plan(proj, rows, Epilogue::Partials);
    if (plan.kernel.slices > kMaxPartialSlices) {  // a shape with more slices than the scratch holds reduces in the kernel
      if (tp_) throw std::invalid_argument("QwenTarget::encodeVerify: a rank's share of a projection has more k-slices than the exchange takes");
      LinearBuffers b{Buffer(), hidden[cur ^ 1], hidden[cur], inputSize, H};
      Linear::add(graph, b, proj, Linear::plan(proj, rows, Epilogue::Residual), in);
      cur ^= 1;
      return;
    }
    LinearBuffers b{Buffer(), partials_, Buffer(), inputSize, H};
    Linear::add(graph, b, proj, plan, in);
    pending = plan.kernel.slices;
  };
  for (LayerWeights &w : layers_) {
    // mixer: h += mixer(norm(h))
    LinearBuffers inB{Buffer(), packed_, Buffer(), H, packedStride_};
    if (w.inParts.empty()) {
      PreparedInput in = convert(&w.attnNorm.buffer, w.inProj.format, prepared_[0], w.attention ? nullptr : &normed_);
      Projection inProj{w.inProj.outputSize, H, Destination::BFloat16, {w.inProj}};
      Linear::add(graph, inB, inProj, Linear::plan(inProj, rows, Epilogue::None), in);
    } else {
      // Segments of several formats: the input is converted once per fragment layout among them (Q4_K's, or the one
      // Q6_K and Q8_0 share), and every segment writes its columns in a launch of its own.
      const uint32_t first = w.inParts.front().format;
      PreparedInput in = convert(&w.attnNorm.buffer, first, prepared_[0], w.attention ? nullptr : &normed_);
      PreparedInput other;
      uint32_t total = 0;
      for (const QuantizedSegment &part : w.inParts) total += part.outputSize;
      for (const QuantizedSegment &part : w.inParts) {
        const bool same = (part.format == SB_FMT_Q4K) == (first == SB_FMT_Q4K);
        if (!same && !other.buffer) other = Linear::prepare(graph, hidden[cur], rows, H, H, &w.attnNorm.buffer, part.format, preparedOther_);
        Projection one{total, H, Destination::BFloat16, {part}};
        Linear::add(graph, inB, one, Linear::plan(one, rows, Epilogue::None), same ? in : other);
      }
    }
    uint32_t mixedWidth;
    if (w.attention) {
      PagedAttention::addProjection(graph, kv_, w.pages, packed_, packedStride_, w.qNorm, w.kNorm, cosine, sine, pageTable_, queries_, rows,
                                    c.q_heads, c.gated_attention != 0, c.rotary_pairs, committedHost, &committed);
      mixedWidth = c.q_heads * D;
      PagedAttention::addAttention(graph, kv_, w.pages, queries_, packed_, packedStride_, pageTable_, treeGiven ? &tree : nullptr, mixed_, mixedWidth, rows,
                                   c.q_heads, c.gated_attention != 0, committedHost, &committed);
    } else {
      // The alpha / beta projection of the normalised input runs inside the GDN kernel (same sums as
      // Linear::addFloat would give), which takes one dependent launch per layer off the step.
      GdnDecodeBuffers g;
      g.gateWeights = &w.ssmAb, g.gateInput = &normed_, g.gateInputSize = H;
      g.packed = packed_, g.gates = gates_, g.convolutionWeights = w.ssmConv, g.decayWeights = w.ssmA, g.timeBias = w.ssmDtBias;
      g.mixerNorm = w.ssmNorm, g.current = w.cells[parity], g.next = w.cells[parity ^ 1];
      g.pendingTape = &w.tapes[parity ^ 1], g.stepTape = &w.tapes[parity];
      mixedWidth = gdn_.valueWidth();
      g.hidden = mixed_, g.packedStride = packedStride_, g.hiddenStride = mixedWidth;
      if (treeGiven) g.treeRows = &tree, g.pendingPathDevice = &pendingPath;
      else g.pendingRowsDevice = &pendingRows;
      g.tiledHeads = c.tiled_heads != 0;
      g.stateSettled = true;  // the current cell was written by the previous step's launch of this layer
      GDN::addDecode(graph, g, gdn_, rows);
    }
    PreparedInput mixedIn = Linear::prepare(graph, mixed_, rows, mixedWidth, mixedWidth, nullptr, w.outProj.format, prepared_[1]);
    project(w.outProj, mixedWidth, mixedIn);
    if (c.moe_experts) {
      // MoE block: h += sum over the row's routes of weight * expert(norm(h)) (runtime/model/Qwen3_6Moe.hpp:27-52). The
      // conversion is run for its side products: the new hidden state and the normalised rows.
      convert(&w.ffnNorm.buffer, c.fmt_proj, prepared_[0], &normed_);
      MoeBuffers mb{normed_, hidden[cur], moeScores_, moeSelected_, moeWeights_, moeScratch_, hidden[cur ^ 1]};
      MoE::addRouting(graph, moe_, w.moe, mb, rows, routerScoresGiven ? &moeScoresGiven_ : nullptr);
      MoE::addRouted(graph, moe_, w.moe, mb, rows);
      cur ^= 1;
      continue;
    }
    // FFN: h += down(silu(gate(norm(h))) * up(norm(h)))
    PreparedInput ffnIn = convert(&w.ffnNorm.buffer, w.ffnGate.format, prepared_[0], nullptr);
    Linear::addGateUp(graph, act_, c.intermediate, w.ffnGate, w.ffnUp, rows, ffnIn);
    PreparedInput actIn = Linear::prepare(graph, act_, rows, c.intermediate, c.intermediate, nullptr, w.ffnDown.format, prepared_[1]);
    project(w.ffnDown, c.intermediate, actIn);
  }
  // logits of every row
  PreparedInput headIn = convert(&outputNorm_.buffer, output_.format, prepared_[0], nullptr);
  // (a rank projects its vocabulary columns into its place of the whole matrix; the ranks then gather the rest)
  Projection head{share_.vocab, H, Destination::Float32, {output_}};
  LinearBuffers headB{Buffer(), logits.view(size_t(share_.vocab0) * 4, logits.bytes() - size_t(share_.vocab0) * 4), Buffer(), H, c.vocab};
  Linear::add(graph, headB, head, Linear::plan(head, rows, Epilogue::None), headIn);
  if (tp_) tp_->allGather(graph, exchange++, rows, share_.vocab0, share_.vocab);
  // selection, acceptance, commit
  SamplingBuffers sb;
  sb.logits = logits, sb.inputTokens = tokens, sb.uniforms = uniforms, sb.selected = selected, sb.workspace = sampleWorkspace_;
  sb.logitStride = c.vocab;
  if (drawsGiven) sb.candidateIds = &candidates, sb.candidateQ = &candidateQ, sb.draws = &draws;
  else if (treeGiven && temperature > 0.0f)
    throw std::invalid_argument("QwenTarget::encodeVerify: a sampled tree block needs the draft's candidates and draws (SB_TARGET_DRAWS)");
  if (constrained || excludedCount) {  // the rows' admission first: what a row does not admit is not selectable
    SbAdmitArgs ad{logits.as<float>(), constrained ? constraintMasks.as<uint32_t>() : nullptr, excludedCount ? excludedTokens.as<uint32_t>() : nullptr,
                   rows, c.vocab, c.vocab, maskWords(), excludedCount, 1};
    check(sb_sample_admit(graph.stream, &ad));
    ++graph.launches;
  }
  Sampling::addPenalties(graph, penalties, sb, penaltyWords, tree, rows, c.vocab);  // (nothing when the penalties are off)
  AcceptanceBuffers ab;
  ab.inputTokens = tokens, ab.treeRows = tree, ab.outputTokens = selected, ab.results = results;
  ab.stopTokens = stopTokens, ab.stopTokenCount = stopCount;  // (a retained stop token ends the retained path)
  // One launch selects, accepts and, where nothing has to come between (a tree's path commit reads the lane's position
  // before it moves; a tensor-parallel step's end also numbers the next step's exchanges), ends the step.
  const uint32_t stepAdvance = promptBlock ? 3u | rows << 8 : advance ? 1u : keepPending ? 2u : 0u;
  const bool endsHere = !tp_ && !(treeGiven && advance);
  const Sampling::LaneCommit lc{committed, pendingRows, pendingPath, stepAdvance};
  Sampling::addVerifyAndAcceptance(graph, SamplingPolicy{temperature, minP, topK, topP}, sb, ab, rows, c.vocab, kVerifyRows, 1, tickets, endsHere ? &lc : nullptr, &remaining);
  if (tp_ && exchange != exchangesPerStep()) throw std::logic_error("QwenTarget::encodeVerify: exchange count");
  // The accepted path's KV rows move from their rows' slots to their depths' (a chain's are there already).
  if (treeGiven && advance) {
    const Buffer pathMask = results.view(8, 4);
    for (LayerWeights &w : layers_)
      if (w.attention) PagedAttention::addPathCommit(graph, kv_, w.pages, pageTable_, committedHost, pathMask, &committed);
  }
  if (!endsHere) launchStepEnd(graph, results, committed, pendingRows, pendingPath, stepAdvance, tp_ ? tp_->group() : nullptr, exchange);
}

// A step of several lanes (SbTargetConfig.lanes): every lane a chain of `rows` rows in its 16 row slots, the projections
// over all 16 x lanes slots at once on the many-row kernel (RMSNorm inside its conversion, the residual in its epilogue),
// attention, GDN, selection and acceptance gridded over the lanes with each lane's own position, pages, cell and tapes.
inline void QwenTarget::encodeVerifyLanes(CommandGraph &graph, uint32_t rows, float temperature, uint32_t parity, bool advance, bool treeGiven,
                                          bool keepPending, bool drawsGiven) {
  using namespace ops;
  const SbTargetConfig &c = loc_;
  const uint32_t H = c.hidden, D = c.head_dim, L = lanes_, R = kVerifyRows * L;
  if (treeGiven && temperature > 0.0f && !drawsGiven)
    throw std::invalid_argument("QwenTarget::encodeVerify: a sampled tree block needs the draft's candidates and draws (SB_TARGET_DRAWS)");
  launchStepBegin(graph, committed, tree, positions, rows, treeGiven, L);
  if (c.rotary_pairs) RoPE::addTreeTables(graph, positions, invFreq, cosine, sine, R, 1.0f, c.rotary_pairs);
  Embedding::add(graph, tokens, embedding_, hidden[0], R, H);
  uint32_t cur = 0;
  // The projections back into the hidden width (out_proj, down) are narrow: they divide k over the SMs and leave their
  // splits' sums in widePartials_; the conversion in front of the next projection adds them onto the residual and writes
  // the new hidden rows. `owed`: splits the rows of hidden[cur] still lack.
  uint32_t owed = 0;
  // (normedOutput: the conversion also leaves the normalised rows, for the fp32 projections that read the same input)
  auto convert = [&](const Buffer *norm, const Buffer *normedOutput = nullptr) {
    if (!owed) return Linear::prepareWide(graph, hidden[cur], R, H, H, norm, widePrepared_[0], normedOutput);
    PreparedInput in = Linear::prepareWideSum(graph, widePartials_, owed, hidden[cur], hidden[cur ^ 1], R, H, norm, widePrepared_[0], normedOutput);
    cur ^= 1, owed = 0;
    return in;
  };
  for (LayerWeights &w : layers_) {
    // mixer: h += mixer(norm(h))
    PreparedInput in = convert(&w.attnNorm.buffer, w.attention ? nullptr : &normed_);  // (a GDN layer's own alpha / beta projection reads the normalised rows)
    for (const QuantizedSegment *part : w.inSegments())  // (one segment, or one a checkpoint tensor where their formats differ)
      Linear::addWide(graph, *part, nullptr, in, R, Epilogue::None, nullptr,
                      part->columnOffset ? packed_.view(size_t(part->columnOffset) * 2, packed_.bytes() - size_t(part->columnOffset) * 2) : packed_, packedStride_);
    uint32_t mixedWidth;
    if (w.attention) {
      mixedWidth = c.q_heads * D;
      SbAttnStoreArgs sa{packed_.as(), w.qNorm.as<float>(), w.kNorm.as<float>(), cosine.as<float>(), sine.as<float>(), pageTable_.as<uint32_t>(),
                         queries_.as(), PagedAttention::describe(kv_, w.pages), committed.as<uint32_t>(), rows, c.q_heads,
                         c.gated_attention ? 1u : 0u, c.rotary_pairs, packedStride_, committedHost, L, pagesPerLane_};
      check(sb_attn_store(graph.stream, &sa));
      SbAttnArgs aa{queries_.as(), c.gated_attention ? packed_.as() : nullptr, pageTable_.as<uint32_t>(), treeGiven ? tree.as() : nullptr, mixed_.as(),
                    PagedAttention::describe(kv_, w.pages), committed.as<uint32_t>(), rows, c.q_heads, c.gated_attention ? 1u : 0u,
                    packedStride_, mixedWidth, committedHost, L, pagesPerLane_};
      check(sb_attn_verify(graph.stream, &aa));
      graph.launches += 2;
    } else {
      mixedWidth = gdn_.valueWidth();
      SbGdnArgs a{};
      a.qkvz = packed_.as(), a.gate_weight = w.ssmAb.as<float>(), a.gate_input = normed_.as(), a.gate_k = a.gate_input_stride = H;
      a.conv_w = w.ssmConv.as(), a.a_scale = w.ssmA.as<float>(), a.dt_bias = w.ssmDtBias.as(), a.norm_w = w.ssmNorm.as<float>();
      a.conv_state_in = w.cells[parity].convolution.as(), a.conv_state_out = w.cells[parity ^ 1].convolution.as();
      a.state_in = w.cells[parity].state.as<float>(), a.state_out = w.cells[parity ^ 1].state.as<float>();
      a.pending = w.tapes[parity ^ 1].describe(), a.step = w.tapes[parity].describe();
      a.hidden = mixed_.as(), a.pending_rows_dev = pendingRows.as<uint32_t>();
      if (treeGiven) a.tree = tree.as(), a.pending_path_dev = pendingPath.as<uint32_t>();  // (a tree step's pending rows are a path of the tape)
      a.rows = rows, a.key_heads = gdn_.keyHeads, a.value_heads = gdn_.valueHeads, a.qkvz_stride = packedStride_, a.ab_stride = 2 * gdn_.valueHeads;
      a.hidden_stride = mixedWidth, a.tiled = c.tiled_heads != 0, a.flags = SB_GDN_STATE_SETTLED, a.lanes = L;
      check(sb_gdn_verify(graph.stream, &a));
      ++graph.launches;
    }
    PreparedInput mixedIn = Linear::prepareWide(graph, mixed_, R, mixedWidth, mixedWidth, nullptr, widePrepared_[1]);
    Linear::addWide(graph, w.outProj, nullptr, mixedIn, R, Epilogue::Partials, nullptr, widePartials_, H);
    owed = Linear::wideSplits(H, mixedWidth);
    if (c.moe_experts) {
      // MoE block: h += sum over the row's routes of weight * expert(norm(h)). The conversion is run for the hidden rows it
      // leaves (residual + out_proj's splits); the routes of all lanes' rows are grouped by expert (MoE::addRouted).
      convert(&w.ffnNorm.buffer, &normed_);  // (its normalised rows are the block's input)
      MoeBuffers mb{normed_, hidden[cur], moeScores_, moeSelected_, moeWeights_, moeScratch_, hidden[cur ^ 1]};
      MoE::addRouting(graph, moe_, w.moe, mb, R, routerScoresGiven ? &moeScoresGiven_ : nullptr);
      if (ep_) ep_->addRouted(graph, w.moe, mb);
      else MoE::addRouted(graph, moe_, w.moe, mb, R);
      cur ^= 1;
      continue;
    }
    // FFN: h += down(silu(gate(norm(h))) * up(norm(h)))
    PreparedInput ffnIn = convert(&w.ffnNorm.buffer);
    Linear::addWide(graph, w.ffnGate, &w.ffnUp, ffnIn, R, Epilogue::GateUp, nullptr, act_, c.intermediate);
    PreparedInput actIn = Linear::prepareWide(graph, act_, R, c.intermediate, c.intermediate, nullptr, widePrepared_[1]);
    Linear::addWide(graph, w.ffnDown, nullptr, actIn, R, Epilogue::Partials, nullptr, widePartials_, H);
    owed = Linear::wideSplits(H, c.intermediate);
  }
  PreparedInput headIn = convert(&outputNorm_.buffer);
  Linear::addWide(graph, output_, nullptr, headIn, R, Epilogue::None, nullptr, logits, c.vocab, true);
  // selection, acceptance, commit: every lane its own rows, uniforms and results
  if (constrained || excludedCount) {
    SbAdmitArgs ad{logits.as<float>(), constrained ? constraintMasks.as<uint32_t>() : nullptr, excludedCount ? excludedTokens.as<uint32_t>() : nullptr,
                   rows, c.vocab, c.vocab, maskWords(), excludedCount, L};
    check(sb_sample_admit(graph.stream, &ad));
    ++graph.launches;
  }
  if (penalties.active()) {
    SbPenaltyArgs pa{logits.as<float>(), penaltyWords.as<uint32_t>(), tokens.as<uint32_t>(), tree.as(), rows, c.vocab, c.vocab,
                     penalties.repetition, penalties.presence, penalties.frequency, L, 0};
    check(sb_sample_penalize(graph.stream, &pa));
    ++graph.launches;
  }
  // (with policies a lane, the kernel reads each lane's temperature and end of the distribution from lanePolicies)
  const bool sampled = temperature > 0.0f || lanePoliciesSet;
  SbSampleArgs sa{logits.as<float>(), tokens.as<uint32_t>(), sampled ? uniforms.as<float>() : nullptr, selected.as<uint32_t>(),
                  sampleWorkspace_.as<float>(), rows, c.vocab, c.vocab, temperature, minP, topK, topP, nullptr, nullptr, nullptr, nullptr, L, 0};
  if (lanePoliciesSet) sa.lane_policies = lanePolicies.as<SbLanePolicy>();
  if (drawsGiven && sampled) sa.candidate_ids = candidates.as<uint32_t>(), sa.candidate_q = candidateQ.as<float>(), sa.draws = draws.as<uint8_t>();
  const uint32_t stepAdvance = promptBlock ? 3u | rows << 8 : advance ? 1u : keepPending ? 2u : 0u;
  const bool endsHere = !(treeGiven && advance);  // (a tree's path commit reads the lanes' positions before they move)
  SbSelectAcceptArgs fused{};
  fused.sample = sa;
  fused.accept = SbAcceptArgs{tokens.as<uint32_t>(), tree.as(), selected.as<uint32_t>(), results.as<uint32_t>(), stopCount ? stopTokens.as<uint32_t>() : nullptr, rows,
                              kVerifyRows, stopCount, L};
  fused.tickets = tickets.as<uint32_t>();
  if (raggedStep) fused.lane_rows = laneRows.as<uint32_t>();
  fused.lane_remaining = remaining.as<uint32_t>();
  if (endsHere) {
    fused.committed = committed.as<uint32_t>(), fused.pending_rows = pendingRows.as<uint32_t>(), fused.pending_path = pendingPath.as<uint32_t>();
    fused.advance = stepAdvance;
  }
  check(sb_select_accept(graph.stream, &fused));
  ++graph.launches;
  // The accepted paths' KV rows move from their rows' slots to their depths' (a chain's are there already).
  if (treeGiven && advance)
    for (LayerWeights &w : layers_)
      if (w.attention) {
        const SbKvLayer cache = PagedAttention::describe(kv_, w.pages);
        check(sb_kv_path_commit_lanes(graph.stream, &cache, pageTable_.as<uint32_t>(), pagesPerLane_, committed.as<uint32_t>(), results.as<uint32_t>() + 2, 4, L));
        ++graph.launches;
      }
  if (!endsHere) launchStepEnd(graph, results, committed, pendingRows, pendingPath, stepAdvance, nullptr, 0, L);
}

}  // namespace splash::b200::model
