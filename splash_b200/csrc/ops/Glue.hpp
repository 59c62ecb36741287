// ops::Normalization, ops::Embedding and ops::RoPE of the reference (runtime/ops/Normalization.hpp:30-42,
// runtime/ops/Embedding.hpp:13-17, runtime/ops/RoPE.hpp:12-45) on the B200 kernels.
#pragma once
#include "Backend.hpp"

namespace splash::b200::ops {

struct NormWeights {
  Buffer buffer;  // fp32 [width] (a GGUF's F32 norms)
};

class Normalization {
 public:
  static void addRms(CommandGraph &graph, const Buffer &input, const NormWeights &w, const Buffer &output, uint32_t width,
                     uint32_t rows, uint32_t inputStride, uint32_t outputStride) {
    requireBytes(input, (size_t(rows - 1) * inputStride + width) * 2, "Normalization::addRms input");
    requireBytes(output, (size_t(rows - 1) * outputStride + width) * 2, "Normalization::addRms output");
    requireBytes(w.buffer, size_t(width) * 4, "Normalization::addRms weights");
    check(sb_rmsnorm(graph.stream, input.as(), rows, width, inputStride, w.buffer.as(), output.as(), outputStride));
    ++graph.launches;
  }
};

struct EmbeddingWeights {
  Buffer rows;  // [vocabulary] native rows of `width` weights
  uint32_t vocabulary = 0, width = 0, format = SB_FMT_Q6K;
};

class Embedding {
 public:
  static void add(CommandGraph &graph, const Buffer &tokens, const EmbeddingWeights &w, const Buffer &output, uint32_t rows,
                  uint32_t outputStride) {
    requireBytes(tokens, size_t(rows) * 4, "Embedding::add tokens");
    requireBytes(w.rows, size_t(w.vocabulary) * sb_row_bytes(w.format, w.width), "Embedding::add table");
    requireBytes(output, (size_t(rows - 1) * outputStride + w.width) * 2, "Embedding::add output");
    check(sb_embed(graph.stream, w.format, w.rows.as(), w.vocabulary, w.width, tokens.as<uint32_t>(), rows, output.as(), outputStride));
    ++graph.launches;
  }
};

class RoPE {
 public:
  // cos/sin rows of the step's packed rows at positions[row] = anchor + tree depth.
  static void addTreeTables(CommandGraph &graph, const Buffer &positions, const Buffer &invFreq, const Buffer &cosine,
                            const Buffer &sine, uint32_t rows, float scale, uint32_t pairs) {
    requireBytes(positions, size_t(rows) * 4, "RoPE::addTreeTables positions");
    requireBytes(invFreq, size_t(pairs) * 4, "RoPE::addTreeTables frequencies");
    requireBytes(cosine, size_t(rows) * pairs * 4, "RoPE::addTreeTables cosine");
    requireBytes(sine, size_t(rows) * pairs * 4, "RoPE::addTreeTables sine");
    check(sb_rope_tables(graph.stream, positions.as<uint32_t>(), rows, invFreq.as<float>(), pairs, scale, cosine.as<float>(), sine.as<float>()));
    ++graph.launches;
  }
};

}  // namespace splash::b200::ops
