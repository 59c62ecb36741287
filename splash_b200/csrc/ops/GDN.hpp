// ops::GDN of the reference (runtime/ops/GDN.hpp:106-201, runtime/ops/GDN.cpp:225-328) on the B200 kernel.
#pragma once
#include "Backend.hpp"

namespace splash::b200::ops {

struct GdnShape {
  uint32_t keyHeads = 0, valueHeads = 0;
  static constexpr uint32_t headDimension = 128, convolutionTaps = 4;
  uint32_t keyWidth() const { return keyHeads * headDimension; }
  uint32_t valueWidth() const { return valueHeads * headDimension; }
  uint32_t convolutionWidth() const { return 2 * keyWidth() + valueWidth(); }
  size_t stateBytes() const { return size_t(valueHeads) * headDimension * headDimension * 4; }
  size_t convolutionStateBytes() const { return size_t(convolutionTaps - 1) * convolutionWidth() * 2; }
};

// A step's rows as the next step folds them (GdnTapeLane, runtime/ops/GDN.hpp:112-119).
struct GdnTape {
  Buffer inputs, keys, values, beta, decay;
  static GdnTape allocate(const GdnShape &s, uint32_t rows) {
    GdnTape t;
    t.inputs = Buffer::allocate(size_t(rows) * s.convolutionWidth() * 2);
    t.keys = Buffer::allocate(size_t(rows) * s.keyWidth() * 2);
    t.values = Buffer::allocate(size_t(rows) * s.valueWidth() * 2);
    t.beta = Buffer::allocate(size_t(rows) * s.valueHeads * 2);
    t.decay = Buffer::allocate(size_t(rows) * s.valueHeads * 4);
    return t;
  }
  SbGdnTape describe() const { return SbGdnTape{inputs.as(), keys.as(), values.as(), beta.as(), decay.as<float>()}; }
};

// One lane's cell: the recurrent state and the carried convolution rows, double-buffered
// (current / next, runtime/model/Runtime.cpp:2701-2707).
struct GdnCell {
  Buffer state, convolution;
};

struct GdnDecodeBuffers {
  Buffer packed;              // bf16 [rows, packedStride]: q | k | v | z
  Buffer gates;               // bf16 [rows, 2 * valueHeads]: b then a; unused when the kernel projects them itself
  // Fused gate projection (optional): the fp32 alpha / beta rows [2 * valueHeads, gateInputSize], b rows first, and
  // the layer's normalised input bf16 [rows, gateInputSize]. Takes the place of a separate Linear::addFloat.
  const Buffer *gateWeights = nullptr, *gateInput = nullptr;
  uint32_t gateInputSize = 0;
  Buffer convolutionWeights;  // bf16 [convolutionWidth, 4]
  Buffer decayWeights;        // fp32 [valueHeads] (ssm_a)
  Buffer timeBias;            // bf16 [valueHeads]
  Buffer mixerNorm;           // fp32 [128]
  GdnCell current, next;
  const GdnTape *pendingTape = nullptr, *stepTape = nullptr;
  Buffer hidden;              // bf16 [rows, hiddenStride]
  const Buffer *pendingRowsDevice = nullptr;  // accepted rows of the previous step, written on the device
  uint32_t packedStride = 0, hiddenStride = 0, pendingRows = 0;
  bool tiledHeads = false;
  // Trees (runtime/ops/GDN.hpp:112-119 GdnTapeLane, runtime/metal/abi/VerifyTree.h:24-45): the block's tree rows (none: a
  // chain), and the path the previous step accepted as a row mask of its tape, on the host or as a device word (neither:
  // the tape's first pendingRows rows).
  const Buffer *treeRows = nullptr, *pendingPathDevice = nullptr;
  uint32_t pendingPath = 0;
  // The caller vouches that nothing still running on the stream writes `current.state` (the model's step: the cell
  // was written a whole step earlier), so the kernel may fetch it before waiting for the launch ahead
  // (SB_GDN_STATE_SETTLED). Leave it off for addFold followed at once by addDecode on the swapped cells.
  bool stateSettled = false;
};

class GDN {
 public:
  static void addDecode(CommandGraph &graph, const GdnDecodeBuffers &b, const GdnShape &s, uint32_t rows) {
    requireBytes(b.packed, (size_t(rows ? rows - 1 : 0) * b.packedStride + s.convolutionWidth() + s.valueWidth()) * 2, "GDN::addDecode packed rows");
    if (b.gateWeights) {
      if (!b.gateInput || !b.gateInputSize) throw std::invalid_argument("GDN::addDecode: fused gates without their input");
      requireBytes(*b.gateWeights, size_t(2) * s.valueHeads * b.gateInputSize * 4, "GDN::addDecode gate weights");
      requireBytes(*b.gateInput, size_t(rows) * b.gateInputSize * 2, "GDN::addDecode gate input");
    } else {
      requireBytes(b.gates, size_t(rows) * 2 * s.valueHeads * 2, "GDN::addDecode gates");
    }
    requireBytes(b.convolutionWeights, size_t(s.convolutionWidth()) * 4 * 2, "GDN::addDecode convolution weights");
    requireBytes(b.decayWeights, size_t(s.valueHeads) * 4, "GDN::addDecode decay weights");
    requireBytes(b.timeBias, size_t(s.valueHeads) * 2, "GDN::addDecode time bias");
    requireBytes(b.mixerNorm, 128 * 4, "GDN::addDecode mixer norm");
    requireBytes(b.current.state, s.stateBytes(), "GDN::addDecode current state");
    requireBytes(b.next.state, s.stateBytes(), "GDN::addDecode next state");
    requireBytes(b.current.convolution, s.convolutionStateBytes(), "GDN::addDecode current convolution rows");
    requireBytes(b.next.convolution, s.convolutionStateBytes(), "GDN::addDecode next convolution rows");
    requireBytes(b.hidden, (size_t(rows ? rows - 1 : 0) * b.hiddenStride + s.valueWidth()) * 2, "GDN::addDecode hidden");
    if (!b.pendingTape || !b.stepTape) throw std::invalid_argument("GDN::addDecode: a tape is missing");
    SbGdnArgs a{};
    a.qkvz = b.packed.as();
    if (b.gateWeights) {
      a.gate_weight = b.gateWeights->as<float>(), a.gate_input = b.gateInput->as();
      a.gate_k = a.gate_input_stride = b.gateInputSize;
    } else {
      a.b = b.gates.as();
      a.a = b.gates.as<uint16_t>() + s.valueHeads;
    }
    a.conv_w = b.convolutionWeights.as(), a.a_scale = b.decayWeights.as<float>(), a.dt_bias = b.timeBias.as();
    a.norm_w = b.mixerNorm.as<float>();
    a.conv_state_in = b.current.convolution.as(), a.conv_state_out = b.next.convolution.as();
    a.state_in = b.current.state.as<float>(), a.state_out = b.next.state.as<float>();
    a.pending = b.pendingTape->describe(), a.step = b.stepTape->describe();
    a.hidden = b.hidden.as();
    a.pending_rows_dev = b.pendingRowsDevice ? b.pendingRowsDevice->as<uint32_t>() : nullptr;
    if (b.treeRows) {
      requireBytes(*b.treeRows, size_t(rows) * 8, "GDN::addDecode tree rows");
      a.tree = b.treeRows->as();
    }
    if (b.pendingPathDevice) {
      requireBytes(*b.pendingPathDevice, 4, "GDN::addDecode pending path");
      a.pending_path_dev = b.pendingPathDevice->as<uint32_t>();
    }
    a.pending_path = b.pendingPath;
    a.flags = b.stateSettled ? SB_GDN_STATE_SETTLED : 0;
    a.rows = rows, a.pending_rows = b.pendingRows, a.key_heads = s.keyHeads, a.value_heads = s.valueHeads;
    a.qkvz_stride = b.packedStride, a.ab_stride = 2 * s.valueHeads, a.hidden_stride = b.hiddenStride, a.tiled = b.tiledHeads;
    check(sb_gdn_verify(graph.stream, &a));
    ++graph.launches;
  }
  // Materialises the state after the pending rows alone (GDN::addFold, runtime/ops/GDN.cpp:299-328):
  // the decode with no rows of its own.
  static void addFold(CommandGraph &graph, const GdnDecodeBuffers &b, const GdnShape &s) { addDecode(graph, b, s, 0); }
};

}  // namespace splash::b200::ops
