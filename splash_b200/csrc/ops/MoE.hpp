// ops::MoE of the reference (runtime/ops/MoE.hpp, runtime/ops/MoE.cpp:211-247 addRouting, :260-270 addRouted) on the
// B200 kernels, for the rows of one lane's verify block (up to 16 rows: a route streams its expert by itself) or of several
// lanes' blocks (routes grouped by expert on the many-row kernel): the router's fp32 scores
// (Linear::addFloat over the router's rows), the routes and their weights, the expert passes and the combine.
#pragma once
#include "Linear.hpp"

namespace splash::b200::ops {

struct MoeShape {
  uint32_t experts = 0, slots = 0, topK = 0, hidden = 0, intermediate = 0;
  bool sharedExpert = false, sharedGate = false, sigmoidNormalized = false;
  uint32_t routes() const noexcept { return topK + (sharedExpert ? 1u : 0u); }
  uint32_t expertsTotal() const noexcept { return experts + (sharedExpert ? 1u : 0u); }
};

struct MoeWeights {
  Buffer router;      // fp32 [slots, hidden]
  Buffer sharedGate;  // fp32 [hidden], with MoeShape::sharedGate
  Buffer gate, up;    // native Q4_K rows [expertsTotal][intermediate][hidden]; the shared expert last
  Buffer down;        // native Q4_K rows [expertsTotal][hidden][intermediate]
};

struct MoeBuffers {
  Buffer input;     // bf16 [rows, hidden]: the normalised rows
  Buffer residual;  // bf16 [rows, hidden]
  Buffer scores;    // fp32 [rows, slots]
  Buffer selected;  // u32 [rows, routes]
  Buffer weights;   // fp32 [rows, routes]
  Buffer scratch;   // MoE::scratchBytes
  Buffer output;    // bf16 [rows, hidden]
};

class MoE {
 public:
  static size_t scratchBytes(const MoeShape &s, uint32_t rows) { return sb_moe_scratch_bytes(rows, s.routes(), s.hidden, s.intermediate); }

  // Router scores, then each row's routes and weights. `given` (measurements with synthetic routing): the routes come from
  // these scores (fp32 [rows, slots]) instead; the router's projection still runs.
  static void addRouting(CommandGraph &graph, const MoeShape &s, const MoeWeights &w, const MoeBuffers &b, uint32_t rows, const Buffer *given = nullptr) {
    if (s.sharedGate && !s.sharedExpert) throw std::invalid_argument("MoE::addRouting: a shared gate without a shared expert");
    if (s.sharedExpert && !s.sharedGate) throw std::invalid_argument("MoE::addRouting: an ungated shared expert is not offered (weight 1 routes)");
    Linear::addFloat(graph, w.router, b.input, s.hidden, rows, s.slots, s.hidden, b.scores, s.slots, Destination::Float32, nullptr);
    requireBytes(b.selected, size_t(rows) * s.routes() * 4, "MoE::addRouting selected");
    requireBytes(b.weights, size_t(rows) * s.routes() * 4, "MoE::addRouting weights");
    if (s.sharedGate) requireBytes(w.sharedGate, size_t(s.hidden) * 4, "MoE::addRouting shared gate");
    if (given) requireBytes(*given, size_t(rows) * s.slots * 4, "MoE::addRouting given scores");
    SbMoeRouteArgs a{given ? given->as<float>() : b.scores.as<float>(), b.input.as(), s.sharedGate ? w.sharedGate.as<float>() : nullptr, b.selected.as<uint32_t>(),
                     b.weights.as<float>(), rows, s.experts, s.slots, s.topK, s.hidden, s.sigmoidNormalized ? 1u : 0u};
    check(sb_moe_route(graph.stream, &a));
    ++graph.launches;
  }

  // The routed rows through their experts, and residual + the weighted sum of their outputs.
  static void addRouted(CommandGraph &graph, const MoeShape &s, const MoeWeights &w, const MoeBuffers &b, uint32_t rows) {
    const size_t pair = size_t(s.expertsTotal()) * s.intermediate * sb_row_bytes(SB_FMT_Q4K, s.hidden);
    requireBytes(w.gate, pair, "MoE::addRouted gate experts");
    requireBytes(w.up, pair, "MoE::addRouted up experts");
    requireBytes(w.down, size_t(s.expertsTotal()) * s.hidden * sb_row_bytes(SB_FMT_Q4K, s.intermediate), "MoE::addRouted down experts");
    requireBytes(b.input, size_t(rows) * s.hidden * 2, "MoE::addRouted input");
    requireBytes(b.output, size_t(rows) * s.hidden * 2, "MoE::addRouted output");
    requireBytes(b.scratch, scratchBytes(s, rows), "MoE::addRouted scratch");
    SbMoeExpertArgs a{b.input.as(), b.residual ? b.residual.as() : nullptr, b.selected.as<uint32_t>(), b.weights.as<float>(), w.gate.as(), w.up.as(),
                      w.down.as(), b.scratch.as(), b.output.as(), rows, s.routes(), s.hidden, s.intermediate, SB_FMT_Q4K, s.expertsTotal()};
    check(sb_moe_experts(graph.stream, &a));
    graph.launches += rows > 16 ? 6 : 3;  // (grouping, two conversions, two grouped passes, combine)
  }
};

}  // namespace splash::b200::ops
