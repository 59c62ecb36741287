// ops::Linear of the reference (runtime/ops/Linear.hpp:73-347, runtime/ops/LinearGguf.cpp:212-362) on
// the B200 kernels: a projection's plan (k-slices, CTAs, ring), its prepared input, and the dispatch
// with an epilogue. A projection is one or more column segments of native GGUF rows
// (runtime/ops/Weights.hpp:108-225); segments of quantized rows run sb_linear, F32 rows sb_linear_f32.
#pragma once
#include <vector>

#include "Backend.hpp"

namespace splash::b200::ops {

enum class Epilogue { None = SB_EPILOGUE_NONE, Residual = SB_EPILOGUE_RESIDUAL, UpWithGate = SB_EPILOGUE_UP_WITH_GATE,
                      GateUp = SB_EPILOGUE_GATE_UP, Partials = SB_EPILOGUE_PARTIALS, GateUpPartials = SB_EPILOGUE_GATE_UP_PARTIALS };
enum class Destination { BFloat16, Float32 };

// One tensor's rows: `outputSize` rows of `inputSize` weights in `format`, written at `columnOffset`.
struct QuantizedSegment {
  Buffer rows;
  uint32_t outputSize = 0, inputSize = 0, columnOffset = 0, format = SB_FMT_Q4K;
  Buffer image;  // Q6_K / NVFP4 rows as the many-row kernel reads them (Linear::buildImage); empty otherwise
};

struct Projection {
  uint32_t outputSize = 0, inputSize = 0;
  Destination destination = Destination::BFloat16;
  std::vector<QuantizedSegment> segments;
};

// The input of a projection converted once for a format's fragment layout; several projections of the
// same input share it (PreparedInput, runtime/ops/Linear.hpp:287-347).
struct PreparedInput {
  Buffer buffer;
  uint32_t format = SB_FMT_Q4K;  // layout family: Q4_K's, or Q6_K / Q8_0's
  uint32_t inputSize = 0;
};

struct LinearBuffers {
  Buffer input;     // bf16 [rows, inputStride]
  Buffer output;    // bf16 or fp32 [rows, outputStride]
  Buffer residual;  // bf16 [rows, outputStride]: Residual's addend or UpWithGate's gate
  uint32_t inputStride = 0, outputStride = 0;
};

struct LinearPlan {
  SbLinearPlan kernel{};
  uint32_t rows = 0;
  Epilogue epilogue = Epilogue::None;
};

class Linear {
 public:
  static LinearPlan plan(const Projection &p, uint32_t rows, Epilogue epilogue) {
    if (p.segments.empty()) throw std::invalid_argument("Linear::plan: a projection without segments");
    LinearPlan plan;
    plan.rows = rows;
    plan.epilogue = epilogue;
    const QuantizedSegment &s = p.segments.front();
    if (s.format != SB_FMT_F32) check(sb_linear_plan(s.format, s.outputSize, s.inputSize, rows, uint32_t(epilogue), &plan.kernel));
    return plan;
  }

  static uint64_t preparedBytes(uint32_t inputSize) { return sb_linear_prepared_bytes(inputSize); }

  // Converts `input` (optionally through an RMSNorm with fp32 weights) for projections of `format`.
  static PreparedInput prepare(CommandGraph &graph, const Buffer &input, uint32_t rows, uint32_t inputSize,
                               uint32_t inputStride, const Buffer *normWeight, uint32_t format, const Buffer &scratch,
                               const Buffer *normedOutput = nullptr) {
    requireBytes(input, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "Linear::prepare input");
    requireBytes(scratch, preparedBytes(inputSize), "Linear::prepare scratch");
    if (normWeight) requireBytes(*normWeight, size_t(inputSize) * 4, "Linear::prepare norm weight");
    if (normedOutput) requireBytes(*normedOutput, size_t(rows) * inputSize * 2, "Linear::prepare normalised output");
    check(sb_linear_prepare(graph.stream, input.as(), rows, inputSize, inputStride, normWeight ? normWeight->as() : nullptr,
                            format, scratch.as(), normedOutput ? normedOutput->as() : nullptr, graph.pdl ? SB_LINEAR_PDL : 0));
    ++graph.launches;
    return {scratch, format == SB_FMT_Q4K ? uint32_t(SB_FMT_Q4K) : uint32_t(SB_FMT_Q6K), inputSize};
  }

  // The same conversion over input = bf16(residual + the k-slices' partial sums a projection left with
  // Epilogue::Partials): that projection's residual epilogue, done where its result is consumed. `sum` receives the
  // input, i.e. the new hidden state.
  static PreparedInput prepareSum(CommandGraph &graph, const Buffer &partials, uint32_t slices, uint32_t partialStride, const Buffer &residual,
                                  const Buffer &sum, uint32_t rows, uint32_t inputSize, uint32_t inputStride, const Buffer *normWeight,
                                  uint32_t format, const Buffer &scratch, const Buffer *normedOutput = nullptr) {
    requireBytes(partials, size_t(slices) * 16 * partialStride * 4, "Linear::prepareSum partial sums");
    requireBytes(residual, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "Linear::prepareSum residual");
    requireBytes(sum, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "Linear::prepareSum sum");
    requireBytes(scratch, preparedBytes(inputSize), "Linear::prepareSum scratch");
    if (normWeight) requireBytes(*normWeight, size_t(inputSize) * 4, "Linear::prepareSum norm weight");
    if (normedOutput) requireBytes(*normedOutput, size_t(rows) * inputSize * 2, "Linear::prepareSum normalised output");
    check(sb_linear_prepare_sum(graph.stream, partials.as<float>(), slices, partialStride, residual.as(), inputStride, sum.as(), inputStride,
                                rows, inputSize, normWeight ? normWeight->as() : nullptr, format, scratch.as(),
                                normedOutput ? normedOutput->as() : nullptr, graph.pdl ? SB_LINEAR_PDL : 0));
    ++graph.launches;
    return {scratch, format == SB_FMT_Q4K ? uint32_t(SB_FMT_Q4K) : uint32_t(SB_FMT_Q6K), inputSize};
  }

  // ---- many rows (a step of several lanes, or a chunk): the tensor-memory kernel (sb_linear_wide) ----
  // The conversion for it (another layout than prepare's); `scratch` holds wideBytes(rows, inputSize).
  static uint64_t wideBytes(uint32_t rows, uint32_t inputSize) { return sb_linear_wide_prepared_bytes(rows, inputSize); }
  static PreparedInput prepareWide(CommandGraph &graph, const Buffer &input, uint32_t rows, uint32_t inputSize, uint32_t inputStride,
                                   const Buffer *normWeight, const Buffer &scratch, const Buffer *normedOutput = nullptr) {
    requireBytes(input, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "Linear::prepareWide input");
    requireBytes(scratch, wideBytes(rows, inputSize), "Linear::prepareWide scratch");
    if (normWeight) requireBytes(*normWeight, size_t(inputSize) * 4, "Linear::prepareWide norm weight");
    if (normedOutput) requireBytes(*normedOutput, size_t(rows) * inputSize * 2, "Linear::prepareWide normalised output");
    check(sb_linear_wide_prepare_normed(graph.stream, nullptr, 0, 0, nullptr, 0, input.as(), inputStride, rows, inputSize,
                                        normWeight ? normWeight->as() : nullptr, scratch.as(), normedOutput ? normedOutput->as() : nullptr,
                                        graph.pdl ? SB_LINEAR_PDL : 0));
    graph.launches += (rows + 127) / 128;
    return {scratch, 0xFFFFu, inputSize};  // (format tag of the wide layout)
  }
  // k-splits of a projection left as Epilogue::Partials, and the conversion that adds them: x = bf16(residual + the
  // splits' sums in split order) goes to `sumOut` (the new hidden rows), then the conversion of x as prepareWide does it.
  static uint32_t wideSplits(uint32_t outputSize, uint32_t inputSize) { return sb_linear_wide_splits(outputSize, inputSize); }
  static PreparedInput prepareWideSum(CommandGraph &graph, const Buffer &partials, uint32_t splits, const Buffer &residual, const Buffer &sumOut,
                                      uint32_t rows, uint32_t inputSize, const Buffer *normWeight, const Buffer &scratch,
                                      const Buffer *normedOutput = nullptr) {
    if (normedOutput) requireBytes(*normedOutput, size_t(rows) * inputSize * 2, "Linear::prepareWideSum normalised output");
    requireBytes(partials, size_t(splits) * rows * inputSize * 4, "Linear::prepareWideSum partial sums");
    requireBytes(residual, size_t(rows) * inputSize * 2, "Linear::prepareWideSum residual");
    requireBytes(sumOut, size_t(rows) * inputSize * 2, "Linear::prepareWideSum sum");
    requireBytes(scratch, wideBytes(rows, inputSize), "Linear::prepareWideSum scratch");
    if (normWeight) requireBytes(*normWeight, size_t(inputSize) * 4, "Linear::prepareWideSum norm weight");
    check(sb_linear_wide_prepare_normed(graph.stream, partials.as<float>(), splits, inputSize, residual.as(), inputSize, sumOut.as(), inputSize, rows,
                                        inputSize, normWeight ? normWeight->as() : nullptr, scratch.as(), normedOutput ? normedOutput->as() : nullptr,
                                        graph.pdl ? SB_LINEAR_PDL : 0));
    graph.launches += (rows + 127) / 128;
    return {scratch, 0xFFFFu, inputSize};
  }
  // The image of a Q6_K / NVFP4 segment's rows for addWide (made when the weights are loaded or changed; Q4_K has none).
  static uint64_t imageBytes(const QuantizedSegment &s) { return sb_linear_wide_image_bytes(s.format, s.outputSize, s.inputSize); }
  static void buildImage(void *stream, const QuantizedSegment &s) {
    if (!s.image) return;
    requireBytes(s.image, imageBytes(s), "Linear::buildImage image");
    check(sb_linear_wide_image(stream, s.format, s.rows.as(), s.outputSize, s.inputSize, s.image.as()));
  }
  // One segment over `rows` rows (Q4_K rows, or the image of Q6_K / NVFP4 rows): epilogues None / Residual / UpWithGate,
  // GateUp with `up` given, or Partials (output: fp32 [wideSplits][rows][outputStride]).
  static void addWide(CommandGraph &graph, const QuantizedSegment &s, const QuantizedSegment *up, const PreparedInput &prepared, uint32_t rows,
                      Epilogue epilogue, const Buffer *aux, const Buffer &output, uint32_t outputStride, bool float32 = false) {
    if (prepared.format != 0xFFFFu || prepared.inputSize != s.inputSize) throw std::invalid_argument("Linear::addWide: not a wide conversion of this width");
    if ((epilogue == Epilogue::GateUp) != (up != nullptr)) throw std::invalid_argument("Linear::addWide: the up tensor comes with GateUp");
    requireBytes(s.rows, size_t(s.outputSize) * sb_row_bytes(s.format, s.inputSize), "Linear::addWide segment rows");
    if (up) requireBytes(up->rows, size_t(up->outputSize) * sb_row_bytes(up->format, up->inputSize), "Linear::addWide up rows");
    if (epilogue == Epilogue::Partials) {
      float32 = true;
      requireBytes(output, size_t(wideSplits(s.outputSize, s.inputSize)) * rows * outputStride * 4, "Linear::addWide partial sums");
    } else {
      requireBytes(output, (size_t(rows - 1) * outputStride + s.outputSize) * (float32 ? 4 : 2), "Linear::addWide output");
    }
    if (aux) requireBytes(*aux, (size_t(rows - 1) * outputStride + s.outputSize) * 2, "Linear::addWide residual or gate");
    SbLinearArgs a{};
    const bool image = s.format != SB_FMT_Q4K;
    if (image && (!s.image || (up && !up->image))) throw std::invalid_argument("Linear::addWide: the segment's image has not been made");
    a.weights = image ? s.image.as() : s.rows.as(), a.weights2 = up ? (image ? up->image.as() : up->rows.as()) : nullptr, a.prepared = prepared.buffer.as();
    a.aux = aux ? aux->as() : nullptr, a.out = output.as();
    a.format = s.format, a.n = s.outputSize, a.k = s.inputSize, a.rows = rows;
    a.aux_stride = aux ? outputStride : 0, a.out_stride = outputStride, a.epilogue = uint32_t(epilogue), a.out_f32 = float32;
    a.flags = (graph.pdl ? SB_LINEAR_PDL : 0) | (image ? SB_LINEAR_WIDE_IMAGE : 0);
    check(sb_linear_wide(graph.stream, &a));
    graph.launches += (rows + 127) / 128;
  }

  // One projection over a prepared input; every segment writes its columns of the output.
  static void add(CommandGraph &graph, const LinearBuffers &b, const Projection &p, const LinearPlan &plan,
                  const PreparedInput &prepared) {
    const uint32_t esize = p.destination == Destination::Float32 || plan.epilogue == Epilogue::Partials ? 4 : 2;
    if (plan.epilogue == Epilogue::Partials) {
      // Every k-slice's sums, fp32 [slices][16][outputStride]; Linear::prepareSum adds them where they are consumed.
      if (p.segments.size() != 1) throw std::invalid_argument("Linear::add: partial sums of a single segment only");
      requireBytes(b.output, size_t(plan.kernel.slices) * 16 * b.outputStride * 4, "Linear::add partial sums");
    } else {
      requireBytes(b.output, (size_t(plan.rows - 1) * b.outputStride + p.outputSize) * esize, "Linear::add output");
    }
    if (plan.epilogue == Epilogue::Residual || plan.epilogue == Epilogue::UpWithGate)
      requireBytes(b.residual, (size_t(plan.rows - 1) * b.outputStride + p.outputSize) * 2, "Linear::add residual");
    if (prepared.inputSize != p.inputSize) throw std::invalid_argument("Linear::add: prepared input of another width");
    for (const QuantizedSegment &s : p.segments) {
      if (s.inputSize != p.inputSize || s.columnOffset + s.outputSize > p.outputSize)
        throw std::invalid_argument("Linear::add: a segment outside its projection");
      requireBytes(s.rows, size_t(s.outputSize) * sb_row_bytes(s.format, s.inputSize), "Linear::add segment rows");
      const bool q4 = s.format == SB_FMT_Q4K;
      if (q4 != (prepared.format == SB_FMT_Q4K)) throw std::invalid_argument("Linear::add: prepared input of another layout");
      SbLinearArgs a{};
      a.weights = s.rows.as();
      a.prepared = prepared.buffer.as();
      a.aux = b.residual ? b.residual.as<uint8_t>() + size_t(s.columnOffset) * 2 : nullptr;
      a.out = b.output.as<uint8_t>() + size_t(s.columnOffset) * esize;
      a.format = s.format, a.n = s.outputSize, a.k = s.inputSize, a.rows = plan.rows;
      a.aux_stride = a.aux ? b.outputStride : 0, a.out_stride = b.outputStride;
      a.epilogue = uint32_t(plan.epilogue), a.out_f32 = p.destination == Destination::Float32 || plan.epilogue == Epilogue::Partials;
      a.flags = graph.pdl ? SB_LINEAR_PDL : 0;
      check(sb_linear(graph.stream, &a));
      ++graph.launches;
    }
  }

  // SwiGLU's first half in one pass over the gate and up tensors: bf16(bf16(up) * silu(bf16(gate)))
  // (Linear::addSwiGlu, runtime/ops/Linear.cpp:290-308).
  static void addGateUp(CommandGraph &graph, const Buffer &output, uint32_t outputStride, const QuantizedSegment &gate,
                        const QuantizedSegment &up, uint32_t rows, const PreparedInput &prepared) {
    if (gate.format != up.format || gate.outputSize != up.outputSize || gate.inputSize != up.inputSize)
      throw std::invalid_argument("Linear::addGateUp: gate and up tensors differ in shape or format");
    requireBytes(output, (size_t(rows - 1) * outputStride + gate.outputSize) * 2, "Linear::addGateUp output");
    requireBytes(gate.rows, size_t(gate.outputSize) * sb_row_bytes(gate.format, gate.inputSize), "Linear::addGateUp gate");
    requireBytes(up.rows, size_t(up.outputSize) * sb_row_bytes(up.format, up.inputSize), "Linear::addGateUp up");
    SbLinearArgs a{};
    a.weights = gate.rows.as(), a.weights2 = up.rows.as(), a.prepared = prepared.buffer.as(), a.out = output.as();
    a.format = gate.format, a.n = gate.outputSize, a.k = gate.inputSize, a.rows = rows, a.out_stride = outputStride;
    a.epilogue = SB_EPILOGUE_GATE_UP, a.flags = graph.pdl ? SB_LINEAR_PDL : 0;
    check(sb_linear(graph.stream, &a));
    ++graph.launches;
  }

  // The same pass leaving every k-slice's gate and up sums unreduced in `partials` (fp32 [slices][16][partialStride],
  // gate at column c, up at gate.outputSize + c); prepareGateUp adds them and applies the activation. Returns the slices.
  static uint32_t addGateUpPartials(CommandGraph &graph, const Buffer &partials, uint32_t partialStride, const QuantizedSegment &gate,
                                    const QuantizedSegment &up, uint32_t rows, const PreparedInput &prepared) {
    if (gate.format != up.format || gate.outputSize != up.outputSize || gate.inputSize != up.inputSize)
      throw std::invalid_argument("Linear::addGateUpPartials: gate and up tensors differ in shape or format");
    SbLinearPlan plan{};
    check(sb_linear_plan(gate.format, gate.outputSize, gate.inputSize, rows, SB_EPILOGUE_GATE_UP_PARTIALS, &plan));
    if (partialStride < 2 * gate.outputSize) throw std::invalid_argument("Linear::addGateUpPartials: partial rows hold gate and up columns");
    requireBytes(partials, size_t(plan.slices) * 16 * partialStride * 4, "Linear::addGateUpPartials partial sums");
    requireBytes(gate.rows, size_t(gate.outputSize) * sb_row_bytes(gate.format, gate.inputSize), "Linear::addGateUpPartials gate");
    requireBytes(up.rows, size_t(up.outputSize) * sb_row_bytes(up.format, up.inputSize), "Linear::addGateUpPartials up");
    SbLinearArgs a{};
    a.weights = gate.rows.as(), a.weights2 = up.rows.as(), a.prepared = prepared.buffer.as(), a.out = partials.as();
    a.format = gate.format, a.n = gate.outputSize, a.k = gate.inputSize, a.rows = rows, a.out_stride = partialStride, a.out_f32 = 1;
    a.epilogue = SB_EPILOGUE_GATE_UP_PARTIALS, a.flags = graph.pdl ? SB_LINEAR_PDL : 0;
    check(sb_linear(graph.stream, &a));
    ++graph.launches;
    return plan.slices;
  }

  // The conversion of the SwiGLU result for the down projection, from the pair's unreduced sums; `activation` (bf16
  // [rows, activationStride]) receives the result as Linear::addGateUp would have written it.
  static PreparedInput prepareGateUp(CommandGraph &graph, const Buffer &partials, uint32_t slices, uint32_t partialStride, uint32_t width,
                                     const Buffer &activation, uint32_t activationStride, uint32_t rows, uint32_t format, const Buffer &scratch) {
    requireBytes(partials, size_t(slices) * 16 * partialStride * 4, "Linear::prepareGateUp partial sums");
    requireBytes(activation, (size_t(rows - 1) * activationStride + width) * 2, "Linear::prepareGateUp activation");
    requireBytes(scratch, preparedBytes(width), "Linear::prepareGateUp scratch");
    check(sb_linear_prepare_gate_up(graph.stream, partials.as<float>(), slices, partialStride, width, activation.as(), activationStride, rows,
                                    format, scratch.as(), graph.pdl ? SB_LINEAR_PDL : 0));
    ++graph.launches;
    return {scratch, format == SB_FMT_Q4K ? uint32_t(SB_FMT_Q4K) : uint32_t(SB_FMT_Q6K), width};
  }

  // fp32 rows (GDN alpha/beta, MoE router) over the bf16 input, optionally through the same RMSNorm.
  static void addFloat(CommandGraph &graph, const Buffer &weights, const Buffer &input, uint32_t inputStride, uint32_t rows,
                       uint32_t outputSize, uint32_t inputSize, const Buffer &output, uint32_t outputStride, Destination d,
                       const Buffer *normWeight) {
    requireBytes(weights, size_t(outputSize) * inputSize * 4, "Linear::addFloat weights");
    requireBytes(input, size_t(rows - 1) * inputStride * 2 + size_t(inputSize) * 2, "Linear::addFloat input");
    requireBytes(output, (size_t(rows - 1) * outputStride + outputSize) * (d == Destination::Float32 ? 4 : 2), "Linear::addFloat output");
    check(sb_linear_f32(graph.stream, weights.as<float>(), input.as(), rows, outputSize, inputSize, inputStride, output.as(),
                        outputStride, d == Destination::Float32, normWeight ? normWeight->as() : nullptr));
    ++graph.launches;
  }
};

}  // namespace splash::b200::ops
