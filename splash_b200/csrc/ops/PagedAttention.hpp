// ops::PagedAttention of the reference (runtime/ops/PagedAttention.hpp:259-366, runtime/ops/PagedKv.hpp:155-232)
// on the B200 kernels: projection (q/k norm, RoPE, INT8 store), attention over the pages, path commit.
#pragma once
#include "Backend.hpp"

namespace splash::b200::ops {

namespace kv {
// Geometry of the INT8 cache of every attention layer (kv::Layout, runtime/ops/PagedKv.hpp:155-178).
struct Layout {
  uint32_t attentionLayers = 0, kvHeads = 0, headDimension = 0, pageTokens = 256;
  bool halfScales = true;  // fp16 per-token-per-head scales; false: the reference's fp32
  size_t dataBytesPerLayerPage() const { return size_t(kvHeads) * pageTokens * headDimension; }
  size_t scaleBytesPerLayerPage() const { return size_t(kvHeads) * pageTokens * (halfScales ? 2 : 4); }
};
// One layer's pages.
struct LayerPages {
  Buffer keys, values, keyScales, valueScales;
  uint32_t pages = 0;
};
}  // namespace kv

class PagedAttention {
 public:
  static SbKvLayer describe(const kv::Layout &l, const kv::LayerPages &p) {
    requireBytes(p.keys, p.pages * l.dataBytesPerLayerPage(), "PagedAttention keys");
    requireBytes(p.values, p.pages * l.dataBytesPerLayerPage(), "PagedAttention values");
    requireBytes(p.keyScales, p.pages * l.scaleBytesPerLayerPage(), "PagedAttention key scales");
    requireBytes(p.valueScales, p.pages * l.scaleBytesPerLayerPage(), "PagedAttention value scales");
    return SbKvLayer{p.keys.as(), p.values.as(), p.keyScales.as(), p.valueScales.as(), l.kvHeads, l.headDimension, l.pageTokens,
                     l.halfScales ? 1u : 0u};
  }

  // q/k RMSNorm, partial RoPE, queries staged, K and V rows of the block stored at committed + row.
  static void addProjection(CommandGraph &graph, const kv::Layout &l, const kv::LayerPages &pages, const Buffer &packed,
                            uint32_t packedStride, const Buffer &qNorm, const Buffer &kNorm, const Buffer &cosine,
                            const Buffer &sine, const Buffer &pageTable, const Buffer &queries, uint32_t rows, uint32_t queryHeads,
                            bool gated, uint32_t pairs, uint32_t committed, const Buffer *committedDevice) {
    const uint32_t D = l.headDimension, width = queryHeads * (gated ? 2 * D : D) + 2 * l.kvHeads * D;
    requireBytes(packed, (size_t(rows - 1) * packedStride + width) * 2, "PagedAttention::addProjection packed rows");
    requireBytes(qNorm, size_t(D) * 4, "PagedAttention::addProjection q norm");
    requireBytes(kNorm, size_t(D) * 4, "PagedAttention::addProjection k norm");
    requireBytes(cosine, size_t(rows) * pairs * 4, "PagedAttention::addProjection cosine");
    requireBytes(sine, size_t(rows) * pairs * 4, "PagedAttention::addProjection sine");
    requireBytes(queries, size_t(rows) * queryHeads * D * 2, "PagedAttention::addProjection queries");
    requireBytes(pageTable, size_t((committed + rows + l.pageTokens - 1) / l.pageTokens) * 4, "PagedAttention::addProjection page table");
    SbAttnStoreArgs a{packed.as(), qNorm.as<float>(), kNorm.as<float>(), cosine.as<float>(), sine.as<float>(), pageTable.as<uint32_t>(),
                      queries.as(), describe(l, pages), committedDevice ? committedDevice->as<uint32_t>() : nullptr,
                      rows, queryHeads, gated ? 1u : 0u, pairs, packedStride, committed};
    check(sb_attn_store(graph.stream, &a));
    ++graph.launches;
  }

  static void addAttention(CommandGraph &graph, const kv::Layout &l, const kv::LayerPages &pages, const Buffer &queries,
                           const Buffer &packed, uint32_t packedStride, const Buffer &pageTable, const Buffer *tree,
                           const Buffer &output, uint32_t outputStride, uint32_t rows, uint32_t queryHeads, bool gated,
                           uint32_t committed, const Buffer *committedDevice) {
    requireBytes(queries, size_t(rows) * queryHeads * l.headDimension * 2, "PagedAttention::addAttention queries");
    requireBytes(output, (size_t(rows - 1) * outputStride + queryHeads * l.headDimension) * 2, "PagedAttention::addAttention output");
    requireBytes(pageTable, size_t((committed + rows + l.pageTokens - 1) / l.pageTokens) * 4, "PagedAttention::addAttention page table");
    SbAttnArgs a{queries.as(), gated ? packed.as() : nullptr, pageTable.as<uint32_t>(), tree ? tree->as() : nullptr, output.as(),
                 describe(l, pages), committedDevice ? committedDevice->as<uint32_t>() : nullptr,
                 rows, queryHeads, gated ? 1u : 0u, packedStride, outputStride, committed};
    check(sb_attn_verify(graph.stream, &a));
    ++graph.launches;
  }

  // Moves an accepted tree path's rows to the slots of their depths; a chain's rows are in place.
  static void addPathCommit(CommandGraph &graph, const kv::Layout &l, const kv::LayerPages &pages, const Buffer &pageTable,
                            uint32_t committed, const Buffer &pathMask, const Buffer *committedDevice = nullptr) {
    requireBytes(pathMask, 4, "PagedAttention::addPathCommit path");
    const SbKvLayer c = describe(l, pages);
    if (committedDevice) check(sb_kv_path_commit_at(graph.stream, &c, pageTable.as<uint32_t>(), committedDevice->as<uint32_t>(), pathMask.as<uint32_t>()));
    else check(sb_kv_path_commit(graph.stream, &c, pageTable.as<uint32_t>(), committed, pathMask.as<uint32_t>()));
    ++graph.launches;
  }
};

}  // namespace splash::b200::ops
