// Expert parallelism of the MoE blocks between the GPUs of one node (sb_ep_* of the C ABI): a rank steps its own lanes,
// holds the experts [rank E / W, (rank + 1) E / W) and a copy of the shared expert, and meets the other ranks twice a block:
// dispatch (everybody's normalised rows and routes to everybody) and combine (a rank's weighted sums to the rows' owners).
// The reference runs MoE::addRouted on one device (runtime/ops/MoE.cpp:122-187,260-270); this is the same block cut by experts.
#pragma once
#include "MoE.hpp"

namespace splash::b200::ops {

class ExpertParallel {
 public:
  ExpertParallel(uint32_t world, uint32_t rank, uint32_t rows, const MoeShape &whole) : world_(world), rank_(rank), rows_(rows), whole_(whole) {
    if (whole.experts % world) throw std::invalid_argument("ExpertParallel: the experts do not divide over the ranks");
    check(sb_ep_create(world, rank, rows, whole.hidden, whole.routes(), &group_));
    void *r = nullptr;
    uint32_t *s = nullptr;
    float *w = nullptr;
    check(sb_ep_gathered(group_, &r, &s, &w));
    const size_t all = size_t(world) * rows;
    gatheredRows_ = Buffer::wrap(r, all * whole.hidden * 2);
    gatheredSelected_ = Buffer::wrap(s, all * whole.routes() * 4), gatheredWeights_ = Buffer::wrap(w, all * whole.routes() * 4);
    partial_ = Buffer::allocate(all * whole.hidden * 4);
    local_ = whole;
    local_.experts = local_.slots = whole.experts / world;
    scratch_ = Buffer::allocate(sb_moe_scratch_bytes(std::max<uint32_t>(17, uint32_t(all)), whole.routes(), whole.hidden, whole.intermediate));
  }
  ExpertParallel(const ExpertParallel &) = delete;
  ExpertParallel &operator=(const ExpertParallel &) = delete;
  ~ExpertParallel() { sb_ep_destroy(group_); }

  void exportHandle(void *out) const { check(sb_ep_export(group_, out)); }
  void connect(const void *handles) {
    check(sb_ep_connect(group_, handles));
    connected_ = true;
  }
  bool connected() const noexcept { return connected_; }
  uint32_t world() const noexcept { return world_; }
  uint32_t rank() const noexcept { return rank_; }
  // The rank's experts: whole.experts / world routed ones, then the shared one.
  const MoeShape &local() const noexcept { return local_; }

  // The block for this rank's rows: b.input / b.selected / b.weights are its own rows' (MoE::addRouting has run), `w` holds the
  // rank's experts. output = bf16(residual + every rank's weighted sums for these rows).
  void addRouted(CommandGraph &graph, const MoeWeights &w, const MoeBuffers &b) const {
    if (!connected_) throw std::invalid_argument("ExpertParallel::addRouted: the ranks are not connected");
    requireBytes(b.input, size_t(rows_) * whole_.hidden * 2, "ExpertParallel::addRouted input");
    requireBytes(b.output, size_t(rows_) * whole_.hidden * 2, "ExpertParallel::addRouted output");
    check(sb_ep_dispatch(graph.stream, group_, b.input.as(), b.selected.as<uint32_t>(), b.weights.as<float>()));
    const uint32_t all = world_ * rows_;
    SbMoeExpertArgs a{gatheredRows_.as(), nullptr, gatheredSelected_.as<uint32_t>(), gatheredWeights_.as<float>(), w.gate.as(), w.up.as(), w.down.as(),
                      scratch_.as(), partial_.as(), all, whole_.routes(), whole_.hidden, whole_.intermediate, SB_FMT_Q4K, local_.expertsTotal()};
    check(sb_moe_experts_partial(graph.stream, &a, rank_ * local_.experts, local_.experts, whole_.sharedExpert ? whole_.experts : 0xffffffffu,
                                 rank_ * rows_, rows_));
    check(sb_ep_combine(graph.stream, group_, partial_.as<float>(), b.residual ? b.residual.as() : nullptr, b.output.as()));
    graph.launches += 8;
  }

 private:
  uint32_t world_, rank_, rows_;
  MoeShape whole_, local_;
  void *group_ = nullptr;
  Buffer gatheredRows_, gatheredSelected_, gatheredWeights_, partial_, scratch_;
  bool connected_ = false;
};

}  // namespace splash::b200::ops
