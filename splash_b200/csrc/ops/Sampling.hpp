// ops::Sampling of the reference (runtime/ops/Sampling.hpp:58-216, runtime/ops/Sampling.cpp:198-356) on
// the B200 kernels: the verify rows' selection and the lane's acceptance.
#pragma once
#include "Backend.hpp"

namespace splash::b200::ops {

struct SamplingPolicy {
  float temperature = 0.0f;  // 0: greedy
  // The end of a sampled row's distribution (runtime/ops/Sampling.hpp policy; sampling.metal:604-668): off when 0 / 0 / 1.
  float minP = 0.0f;
  uint32_t topK = 0;
  float topP = 1.0f;
};

// Penalties on the logits of tokens the context holds (runtime/ops/Sampling.hpp:16-29); the defaults change nothing.
struct SamplingPenalties {
  float repetition = 1.0f, presence = 0.0f, frequency = 0.0f;
  bool active() const noexcept { return repetition != 1.0f || presence != 0.0f || frequency != 0.0f; }
};

struct SamplingBuffers {
  Buffer logits;       // fp32 [rows, logitStride]
  Buffer inputTokens;  // u32 [rows]
  Buffer uniforms;     // fp32 [80]: row draws then child tests (runtime/metal/abi/Sampling.h:12-31)
  Buffer selected;     // u32 [rows]
  Buffer workspace;
  uint32_t logitStride = 0;
  // The children each row's draft drew (optional; runtime/metal/kernels/decode/sampling.metal:680-690 DrawChildren): per
  // row 16 candidate ids (u32), the draft's probabilities of them (fp32) and up to 4 drawn candidate indices (u8, 0xff
  // past them). Given, sampled rows select by recursive rejection sampling over these children.
  const Buffer *candidateIds = nullptr, *candidateQ = nullptr, *draws = nullptr;
};

struct AcceptanceBuffers {
  Buffer inputTokens, treeRows, outputTokens, results, stopTokens;
  uint32_t stopTokenCount = 0;
};

class Sampling {
 public:
  static size_t workspace(uint32_t rows, uint32_t vocabulary) { return sb_sample_workspace_bytes(rows, vocabulary); }

  static void addVerify(CommandGraph &graph, const SamplingPolicy &policy, const SamplingBuffers &b, uint32_t rows, uint32_t vocabulary) {
    requireBytes(b.logits, (size_t(rows - 1) * b.logitStride + vocabulary) * 4, "Sampling::addVerify logits");
    requireBytes(b.inputTokens, size_t(rows) * 4, "Sampling::addVerify input tokens");
    requireBytes(b.selected, size_t(rows) * 4, "Sampling::addVerify selected");
    if (policy.temperature > 0.0f) {
      requireBytes(b.uniforms, 80 * 4, "Sampling::addVerify uniforms");
      requireBytes(b.workspace, workspace(rows, vocabulary), "Sampling::addVerify workspace");
    }
    SbSampleArgs a{b.logits.as<float>(), b.inputTokens.as<uint32_t>(), policy.temperature > 0.0f ? b.uniforms.as<float>() : nullptr,
                   b.selected.as<uint32_t>(), b.workspace ? b.workspace.as<float>() : nullptr, rows, vocabulary, b.logitStride,
                   policy.temperature, policy.minP, policy.topK, policy.topP, nullptr, nullptr, nullptr, nullptr};
    if (b.candidateIds && policy.temperature > 0.0f) {
      if (!b.candidateQ || !b.draws) throw std::invalid_argument("Sampling::addVerify: candidates without their probabilities or draws");
      requireBytes(*b.candidateIds, size_t(rows) * 16 * 4, "Sampling::addVerify candidate ids");
      requireBytes(*b.candidateQ, size_t(rows) * 16 * 4, "Sampling::addVerify candidate probabilities");
      requireBytes(*b.draws, size_t(rows) * 4, "Sampling::addVerify draws");
      a.candidate_ids = b.candidateIds->as<uint32_t>(), a.candidate_q = b.candidateQ->as<float>(), a.draws = b.draws->as<uint8_t>();
    }
    check(sb_sample_verify(graph.stream, &a));
    ++graph.launches;
  }

  // The penalty pass over the lane's rows, before addVerify. penaltyWords: u32 [vocabulary], the output's count of each
  // token with the prompt bit (runtime/metal/abi/Sampling.h:124-125).
  static void addPenalties(CommandGraph &graph, const SamplingPenalties &penalties, const SamplingBuffers &b, const Buffer &penaltyWords,
                           const Buffer &treeRows, uint32_t rows, uint32_t vocabulary) {
    if (!penalties.active()) return;
    requireBytes(b.logits, (size_t(rows - 1) * b.logitStride + vocabulary) * 4, "Sampling::addPenalties logits");
    requireBytes(b.inputTokens, size_t(rows) * 4, "Sampling::addPenalties input tokens");
    requireBytes(penaltyWords, size_t(vocabulary) * 4, "Sampling::addPenalties penalty words");
    requireBytes(treeRows, size_t(rows) * 8, "Sampling::addPenalties tree rows");
    SbPenaltyArgs a{b.logits.as<float>(), penaltyWords.as<uint32_t>(), b.inputTokens.as<uint32_t>(), treeRows.as(), rows, vocabulary,
                    b.logitStride, penalties.repetition, penalties.presence, penalties.frequency};
    check(sb_sample_penalize(graph.stream, &a));
    ++graph.launches;
  }

  // addVerify and addAcceptance as one launch (sb_select_accept), for `lanes` lanes whose rows, uniforms and results
  // lie lane after lane in the same buffers; with `commit` the launch also ends the lanes' step (LaneCommit::advance as
  // the step's end takes it). tickets: u32 [lanes], zeroed once.
  struct LaneCommit {
    Buffer committed, pendingRows, pendingPath;
    uint32_t advance = 0;
  };
  static void addVerifyAndAcceptance(CommandGraph &graph, const SamplingPolicy &policy, const SamplingBuffers &b, const AcceptanceBuffers &ab,
                                     uint32_t rows, uint32_t vocabulary, uint32_t maximumRetained, uint32_t lanes, const Buffer &tickets,
                                     const LaneCommit *commit, const Buffer *remaining = nullptr) {
    const size_t slots = lanes > 1 ? size_t(lanes) * 16 : rows;  // (a lane's block lies in its 16 row slots)
    requireBytes(b.logits, ((slots - 1) * b.logitStride + vocabulary) * 4, "Sampling::addVerifyAndAcceptance logits");
    requireBytes(b.inputTokens, slots * 4, "Sampling::addVerifyAndAcceptance input tokens");
    requireBytes(b.selected, slots * 4, "Sampling::addVerifyAndAcceptance selected");
    requireBytes(ab.treeRows, slots * 8, "Sampling::addVerifyAndAcceptance tree rows");
    requireBytes(ab.results, size_t(16) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance results");
    requireBytes(tickets, size_t(4) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance tickets");
    if (policy.temperature > 0.0f) {
      requireBytes(b.uniforms, size_t(80) * 4 * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance uniforms");
      requireBytes(b.workspace, workspace(uint32_t(slots), vocabulary), "Sampling::addVerifyAndAcceptance workspace");
    }
    SbSelectAcceptArgs c{};
    c.sample = SbSampleArgs{b.logits.as<float>(), b.inputTokens.as<uint32_t>(), policy.temperature > 0.0f ? b.uniforms.as<float>() : nullptr,
                            b.selected.as<uint32_t>(), b.workspace ? b.workspace.as<float>() : nullptr, rows, vocabulary, b.logitStride,
                            policy.temperature, policy.minP, policy.topK, policy.topP, nullptr, nullptr, nullptr, nullptr, lanes, 0};
    if (b.candidateIds && policy.temperature > 0.0f) {
      if (!b.candidateQ || !b.draws) throw std::invalid_argument("Sampling::addVerifyAndAcceptance: candidates without their probabilities or draws");
      requireBytes(*b.candidateIds, slots * 16 * 4, "Sampling::addVerifyAndAcceptance candidate ids");
      requireBytes(*b.candidateQ, slots * 16 * 4, "Sampling::addVerifyAndAcceptance candidate probabilities");
      requireBytes(*b.draws, slots * 4, "Sampling::addVerifyAndAcceptance draws");
      c.sample.candidate_ids = b.candidateIds->as<uint32_t>(), c.sample.candidate_q = b.candidateQ->as<float>(), c.sample.draws = b.draws->as<uint8_t>();
    }
    c.accept = SbAcceptArgs{b.inputTokens.as<uint32_t>(), ab.treeRows.as(), b.selected.as<uint32_t>(), ab.results.as<uint32_t>(),
                            ab.stopTokenCount ? ab.stopTokens.as<uint32_t>() : nullptr, rows, maximumRetained, ab.stopTokenCount, lanes};
    c.tickets = tickets.as<uint32_t>();
    if (remaining) {
      requireBytes(*remaining, size_t(4) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance remaining");
      c.lane_remaining = remaining->as<uint32_t>();
    }
    if (commit) {
      requireBytes(commit->committed, size_t(4) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance committed");
      requireBytes(commit->pendingRows, size_t(4) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance pending rows");
      requireBytes(commit->pendingPath, size_t(4) * std::max(1u, lanes), "Sampling::addVerifyAndAcceptance pending path");
      c.committed = commit->committed.as<uint32_t>(), c.pending_rows = commit->pendingRows.as<uint32_t>(), c.pending_path = commit->pendingPath.as<uint32_t>();
      c.advance = commit->advance;
    }
    check(sb_select_accept(graph.stream, &c));
    ++graph.launches;
  }

  static void addAcceptance(CommandGraph &graph, const AcceptanceBuffers &b, uint32_t rows, uint32_t maximumRetained) {
    requireBytes(b.inputTokens, size_t(rows) * 4, "Sampling::addAcceptance input tokens");
    requireBytes(b.treeRows, size_t(rows) * 8, "Sampling::addAcceptance tree rows");
    requireBytes(b.outputTokens, size_t(rows) * 4, "Sampling::addAcceptance output tokens");
    requireBytes(b.results, 16, "Sampling::addAcceptance results");
    SbAcceptArgs a{b.inputTokens.as<uint32_t>(), b.treeRows.as(), b.outputTokens.as<uint32_t>(), b.results.as<uint32_t>(),
                   b.stopTokenCount ? b.stopTokens.as<uint32_t>() : nullptr, rows, maximumRetained, b.stopTokenCount};
    check(sb_accept(graph.stream, &a));
    ++graph.launches;
  }
};

}  // namespace splash::b200::ops
