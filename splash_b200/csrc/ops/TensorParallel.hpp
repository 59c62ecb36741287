// The exchanges of a tensor-parallel step on the host operator layer. The reference runs on one GPU and has no
// such operator; the class follows ops::Linear's conventions (extents checked before anything is enqueued,
// one launch per call). A group is this rank's end of the node's exchange (sb_tp_* of include/splash_b200.h).
#pragma once
#include "Linear.hpp"

namespace splash::b200::ops {

class TensorParallel {
 public:
  TensorParallel(uint32_t world, uint32_t rank, uint32_t width, uint32_t gatherWidth) : world_(world), rank_(rank), width_(width) {
    check(sb_tp_create(world, rank, width, gatherWidth, &group_));
    void *p = nullptr;
    uint64_t bytes = 0;
    check(sb_tp_gather_matrix(group_, &p, &bytes));
    gathered_ = Buffer::wrap(p, bytes);
  }
  TensorParallel(const TensorParallel &) = delete;
  TensorParallel &operator=(const TensorParallel &) = delete;
  ~TensorParallel() { sb_tp_destroy(group_); }

  void exportHandle(void *out) const { check(sb_tp_export(group_, out)); }
  void connect(const void *handles) {
    check(sb_tp_connect(group_, handles));
    connected_ = true;
  }
  bool connected() const noexcept { return connected_; }
  uint32_t world() const noexcept { return world_; }
  uint32_t rank() const noexcept { return rank_; }
  void *group() const noexcept { return group_; }
  // fp32 [16][gatherWidth], whole on every rank after allGather.
  const Buffer &gathered() const noexcept { return gathered_; }

  // Linear::prepareSum where `partials` hold this rank's share of the sum.
  PreparedInput prepareSum(CommandGraph &graph, uint32_t index, const Buffer &partials, uint32_t slices, uint32_t partialStride,
                           const Buffer &residual, const Buffer &sum, uint32_t rows, uint32_t inputSize, uint32_t inputStride,
                           const Buffer *normWeight, uint32_t format, const Buffer &scratch, const Buffer *normedOutput = nullptr) const {
    if (inputSize != width_) throw std::invalid_argument("TensorParallel::prepareSum: the group exchanges rows of another width");
    requireBytes(partials, size_t(slices) * 16 * partialStride * 4, "TensorParallel::prepareSum partial sums");
    requireBytes(residual, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "TensorParallel::prepareSum residual");
    requireBytes(sum, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "TensorParallel::prepareSum sum");
    requireBytes(scratch, Linear::preparedBytes(inputSize), "TensorParallel::prepareSum scratch");
    if (normWeight) requireBytes(*normWeight, size_t(inputSize) * 4, "TensorParallel::prepareSum norm weight");
    if (normedOutput) requireBytes(*normedOutput, size_t(rows) * inputSize * 2, "TensorParallel::prepareSum normalised output");
    check(sb_tp_prepare_sum(graph.stream, group_, index, partials.as<float>(), slices, partialStride, residual.as(), inputStride, sum.as(),
                            inputStride, rows, inputSize, normWeight ? normWeight->as() : nullptr, format, scratch.as(),
                            normedOutput ? normedOutput->as() : nullptr, graph.pdl ? SB_LINEAR_PDL : 0));
    graph.launches += 2;  // the share's push to the peers, and the conversion
    return {scratch, format == SB_FMT_Q4K ? uint32_t(SB_FMT_Q4K) : uint32_t(SB_FMT_Q6K), inputSize};
  }

  // Completes the gather matrix: this rank's columns go out, the peers' come in.
  void allGather(CommandGraph &graph, uint32_t index, uint32_t rows, uint32_t column0, uint32_t columns) const {
    check(sb_tp_all_gather(graph.stream, group_, index, rows, column0, columns));
    ++graph.launches;
  }

 private:
  void *group_ = nullptr;
  Buffer gathered_;
  uint32_t world_, rank_, width_;
  bool connected_ = false;
};

}  // namespace splash::b200::ops
