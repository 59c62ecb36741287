// C ABI of the target model's verify step (include/splash_b200.h, "the target model's verify step"):
// creation, tensor access, seeded synthetic weights written on the device, and the step itself, eager
// or replayed as a CUDA graph per step parity.
#include <map>
#include <memory>
#include <tuple>
#include <vector>

#include "model/QwenTarget.hpp"
#include "sb_internal.h"
#include "sb_ptx.cuh"
#include "sb_tp_internal.cuh"

namespace sb {

// ---- step bookkeeping kernels ----
// positions[row] = committed + depth(row) and the chain's tree rows (parent = row - 1).
// With a tree given, the rows stay as the caller wrote them and a row's position is the anchor's plus its depth.
__global__ void step_begin_kernel(const uint32_t *committed, uint2 *tree, uint32_t *positions, uint32_t rows, uint32_t tree_given) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t r = threadIdx.x, lane = blockIdx.x;  // (a block per lane: its 16 row slots, its own position)
  if (r >= rows) return;
  tree += 16 * lane, positions += 16 * lane;
  if (!tree_given) tree[r] = make_uint2((2u << r) - 1u, (r ? r - 1 : 0) | (r << 16));
  positions[r] = committed[lane] + (tree_given ? tree[r].y >> 16 : r);
}
// The lane's commit: the retained rows become history; the next step folds them into the GDN state.
// advance: 0 hold and clear the pending rows, 1 commit what acceptance retained, 2 hold and keep the pending rows,
// 3 | rows << 8 commit every row of the block whatever was selected (a block of prompt tokens).
__global__ void step_end_kernel(uint32_t *results, uint32_t *committed, uint32_t *pending_rows, uint32_t *pending_path, uint32_t advance,
                                uint32_t *tp_epoch, uint32_t tp_exchanges, uint32_t lanes) {
  pdl_wait();
  if (threadIdx.x < lanes) {  // (a thread per lane)
    const uint32_t lane = threadIdx.x, mode = advance & 0xffu, rows = advance >> 8;
    // The next step's exchanges are numbered after this step's. Their kernels read the count when they start, and
    // kernels may start before the ones ahead of them complete: dependents are let go only after the count has moved.
    if (tp_epoch && lane == 0) *tp_epoch += tp_exchanges;
    if (mode == 3) {
      results[4 * lane] = rows, results[4 * lane + 1] = rows - 1, results[4 * lane + 2] = (2u << (rows - 1)) - 1u;
      committed[lane] += rows;
      pending_rows[lane] = rows;
      pending_path[lane] = 0;  // (the tape's first `rows` rows)
    } else if (mode == 1) {
      committed[lane] += results[4 * lane];
      pending_rows[lane] = results[4 * lane];
      pending_path[lane] = results[4 * lane + 2];
    } else if (mode == 0) {
      pending_rows[lane] = 0;
      pending_path[lane] = 0;
    }  // (2: the lane stays where it is and keeps its pending rows: every such step folds the same rows again)
    __threadfence();
  }
  __syncthreads();
  pdl_launch_dependents();
}

// ---- seeded synthetic data ----
__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t i) { return float(mix64(seed ^ mix64(i)) >> 40) * (1.0f / 16777216.0f); }
__device__ __forceinline__ float normal01(uint64_t seed, uint64_t i) {
  const float u1 = fmaxf(uniform01(seed, 2 * i), 1e-7f), u2 = uniform01(seed, 2 * i + 1);
  return sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}
enum FillKind { kBytes, kF32Normal, kF32Uniform, kBf16Normal, kF16Uniform, kF32NegExp, kInt8 };
__global__ void fill_kernel(int kind, void *p, uint64_t count, uint64_t seed, float a, float b) {
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < count; i += uint64_t(gridDim.x) * blockDim.x) {
    switch (kind) {
      case kBytes: static_cast<uint32_t *>(p)[i] = uint32_t(mix64(seed ^ mix64(i))); break;  // count in words
      case kF32Normal: static_cast<float *>(p)[i] = a + b * normal01(seed, i); break;
      case kF32Uniform: static_cast<float *>(p)[i] = a + (b - a) * uniform01(seed, i); break;
      case kBf16Normal: static_cast<uint16_t *>(p)[i] = float_to_bf16_bits(a + b * normal01(seed, i)); break;
      case kF16Uniform: static_cast<__half *>(p)[i] = __float2half_rn(a + (b - a) * uniform01(seed, i)); break;
      case kF32NegExp: static_cast<float *>(p)[i] = -expf(a + (b - a) * uniform01(seed, i)); break;
      case kInt8: static_cast<int8_t *>(p)[i] = int8_t(int(mix64(seed ^ mix64(i)) % 255) - 127); break;
    }
  }
}
// The half scale fields of native blocks whose other bytes are already random: Q4_K d and dmin =
// |N(0,1)| * 1e-3 (the benchmark configuration's recipe); Q6_K d in U(2e-5, 1e-4) and Q8_0 d in
// U(5e-4, 4e-3) (the ranges of the reference's kernel tests, dev/tests/engine/GgufFormatReference.hpp:292-324).
__global__ void scale_fields_kernel(uint32_t format, uint8_t *p, uint64_t blocks, uint64_t seed) {
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < blocks; i += uint64_t(gridDim.x) * blockDim.x) {
    if (format == SB_FMT_Q4K) {
      __half *h = reinterpret_cast<__half *>(p + i * 144);
      h[0] = __float2half_rn(fabsf(normal01(seed, 2 * i)) * 1e-3f);
      h[1] = __float2half_rn(fabsf(normal01(seed, 2 * i + 1)) * 1e-3f);
    } else if (format == SB_FMT_Q6K) {
      *reinterpret_cast<__half *>(p + i * 210 + 208) = __float2half_rn(2e-5f + 8e-5f * uniform01(seed, i));
    } else if (format == SB_FMT_Q80) {
      *reinterpret_cast<__half *>(p + i * 34) = __float2half_rn(5e-4f + 3.5e-3f * uniform01(seed, i));
    } else if (format == SB_FMT_NVFP4) {  // e4m3 scales of exponents 3..10 (the codes stay as filled), one fp32 scale for the tensor
      uint8_t *b = p + i * 148;
      for (int j = 0; j < 16; ++j) b[j] = uint8_t((b[j] & 0x87u) | ((3u + (b[j] >> 3) % 8u) << 3));
      const float g = 2e-4f + 1.8e-3f * uniform01(seed, 0);
      memcpy(b + 16, &g, 4);
    }
  }
}
__global__ void iota_kernel(uint32_t *p, uint32_t n) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = i;
}
__global__ void inv_freq_kernel(float *p, uint32_t pairs, float theta) {
  const uint32_t i = threadIdx.x;
  if (i < pairs) p[i] = powf(theta, -float(i) / float(pairs));
}

static int fill(int kind, const splash::b200::Buffer &b, uint64_t count, uint64_t seed, float a0, float a1) {
  if (!b || !count) return SB_OK;
  const uint32_t blocks = uint32_t(std::min<uint64_t>((count + 255) / 256, 148 * 32));
  fill_kernel<<<blocks, 256>>>(kind, b.as(), count, seed, a0, a1);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
static int fill_rows(const splash::b200::ops::QuantizedSegment &s, uint64_t seed) {
  const uint64_t bytes = uint64_t(s.outputSize) * sb_row_bytes(s.format, s.inputSize);
  int st = fill(kBytes, s.rows, (bytes + 3) / 4, seed, 0, 0);
  if (st != SB_OK) return st;
  FmtInfo fi;
  fmt_info(s.format, fi);
  const uint64_t blocks = bytes / fi.block_bytes;
  scale_fields_kernel<<<uint32_t(std::min<uint64_t>((blocks + 255) / 256, 148 * 32)), 256>>>(s.format, s.rows.as<uint8_t>(), blocks, seed ^ 0x5ca1eull);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

struct Target {
  std::unique_ptr<splash::b200::model::QwenTarget> model;
  std::map<std::tuple<uint32_t, uint32_t, uint32_t, uint32_t, uint32_t>, cudaGraphExec_t> graphs;  // rows, temperature bits, parity, advance, bound
  uint32_t launches = 0;
  uint32_t *results_pinned = nullptr;  // 4 + 16 words
  uint32_t lane_rows_host[64] = {};    // the lanes' row counts of the ragged step in flight
  cudaStream_t own_stream = nullptr;   // used when the caller passes no stream (the default stream cannot be captured)
  cudaStream_t pick(void *s) const { return s ? as_stream(s) : own_stream; }
};

}  // namespace sb

namespace splash::b200::model {
void launchStepBegin(CommandGraph &graph, const Buffer &committed, const Buffer &tree, const Buffer &positions, uint32_t rows, bool treeGiven,
                     uint32_t lanes) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(lanes), cfg.blockDim = dim3(32), cfg.stream = sb::as_stream(graph.stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = graph.pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, sb::step_begin_kernel, static_cast<const uint32_t *>(committed.as<uint32_t>()), tree.as<uint2>(),
                         positions.as<uint32_t>(), rows, treeGiven ? 1u : 0u) != cudaSuccess)
    throw BackendError(SB_ERR_CUDA, "step_begin launch failed");
  ++graph.launches;
}
void launchStepEnd(CommandGraph &graph, const Buffer &results, const Buffer &committed, const Buffer &pendingRows, const Buffer &pendingPath,
                   uint32_t advance, void *tpGroup, uint32_t exchanges, uint32_t lanes) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1), cfg.blockDim = dim3(32), cfg.stream = sb::as_stream(graph.stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = graph.pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, sb::step_end_kernel, results.as<uint32_t>(), committed.as<uint32_t>(),
                         pendingRows.as<uint32_t>(), pendingPath.as<uint32_t>(), advance, sb::tp_epoch_word(tpGroup), exchanges, lanes) != cudaSuccess)
    throw BackendError(SB_ERR_CUDA, "step_end launch failed");
  ++graph.launches;
}
}  // namespace splash::b200::model

using namespace sb;
using splash::b200::Buffer;
using splash::b200::CommandGraph;
using splash::b200::model::QwenTarget;

// Runs `body`, mapping the operator layer's exceptions to status codes.
template <class F> static int guarded(F body) {
  try {
    return body();
  } catch (const std::invalid_argument &e) {
    return fail(SB_ERR_INVALID, "%s", e.what());
  } catch (const splash::b200::BackendError &e) {
    return fail(e.status(), "%s", e.what());
  } catch (const std::exception &e) {
    return fail(SB_ERR_CUDA, "%s", e.what());
  }
}

extern "C" {

// The format of a checkpoint tensor, for a target whose tensors take their formats from a checkpoint (sb_gguf.cu).
using TensorFormat = uint32_t (*)(void *context, uint32_t layer, const char *stem, uint32_t configured);
int sb_target_create_with_formats(const SbTargetConfig *config, TensorFormat format_of, void *context, void **out_target);

int sb_target_create(const SbTargetConfig *config, void **out_target) { return sb_target_create_with_formats(config, nullptr, nullptr, out_target); }

int sb_target_create_with_formats(const SbTargetConfig *config, TensorFormat format_of, void *context, void **out_target) {
  SB_NEED_DEVICE();
  SB_REQUIRE(config && out_target, "sb_target_create: null pointer");
  return guarded([&] {
    auto t = std::make_unique<Target>();
    QwenTarget::FormatOf by_tensor;
    if (format_of) by_tensor = [=](uint32_t layer, const char *stem, uint32_t configured) { return format_of(context, layer, stem, configured); };
    t->model = std::make_unique<QwenTarget>(*config, by_tensor);
    const uint32_t L = std::max(1u, config->lanes);
    SB_CUDA(cudaMallocHost(&t->results_pinned, size_t(20) * L * sizeof(uint32_t)));
    SB_CUDA(cudaStreamCreateWithFlags(&t->own_stream, cudaStreamNonBlocking));
    QwenTarget &m = *t->model;
    Buffer table;
    m.find(-1, "page_table", table);
    const uint32_t pages = uint32_t(table.bytes() / 4);
    iota_kernel<<<(pages + 255) / 256, 256>>>(table.as<uint32_t>(), pages);
    if (config->rotary_pairs) inv_freq_kernel<<<1, 256>>>(m.invFreq.as<float>(), config->rotary_pairs, config->rope_theta);
    SB_CUDA(cudaMemset(m.committed.as(), 0, 4 * L));
    SB_CUDA(cudaMemset(m.tickets.as(), 0, m.tickets.bytes()));
    SB_CUDA(cudaMemset(m.remaining.as(), 0xff, m.remaining.bytes()));  // no bound on what a request may still take
    SB_CUDA(cudaMemset(m.pendingRows.as(), 0, 4 * L));
    SB_CUDA(cudaMemset(m.pendingPath.as(), 0, 4 * L));
    SB_CUDA(cudaMemset(m.penaltyWords.as(), 0, m.penaltyWords.bytes()));
    SB_CUDA(cudaMemset(m.uniforms.as(), 0, 80 * 4 * L));
    SB_CUDA(cudaMemset(m.tokens.as(), 0, 64 * L));
    SB_CUDA(cudaMemset(m.tree.as(), 0, 128 * L));
    SB_CUDA(cudaDeviceSynchronize());
    *out_target = t.release();
    return int(SB_OK);
  });
}

int sb_target_destroy(void *target) {
  SB_NEED_DEVICE();
  Target *t = static_cast<Target *>(target);
  if (!t) return SB_OK;
  cudaDeviceSynchronize();
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);
  if (t->results_pinned) cudaFreeHost(t->results_pinned);
  if (t->own_stream) cudaStreamDestroy(t->own_stream);
  delete t;
  return SB_OK;
}

int sb_target_tp_export(void *target, void *handle_out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && handle_out, "sb_target_tp_export: null pointer");
  auto *tp = static_cast<Target *>(target)->model->tensorParallel();
  auto *ep = static_cast<Target *>(target)->model->expertParallel();
  SB_REQUIRE(tp || ep, "sb_target_tp_export: the target was created without tensor or expert parallelism");
  if (ep) return guarded([&] { return ep->exportHandle(handle_out), int(SB_OK); });
  return guarded([&] { return tp->exportHandle(handle_out), int(SB_OK); });
}

int sb_target_tp_connect(void *target, const void *handles) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && handles, "sb_target_tp_connect: null pointer");
  auto *tp = static_cast<Target *>(target)->model->tensorParallel();
  auto *ep = static_cast<Target *>(target)->model->expertParallel();
  SB_REQUIRE(tp || ep, "sb_target_tp_connect: the target was created without tensor or expert parallelism");
  if (ep) return guarded([&] { return ep->connect(handles), int(SB_OK); });
  return guarded([&] { return tp->connect(handles), int(SB_OK); });
}

int sb_target_share(const SbTargetConfig *config, SbTargetShare *out_share) {
  SB_REQUIRE(config && out_share, "sb_target_share: null pointer");
  return guarded([&] { return *out_share = splash::b200::model::shareOf(*config), int(SB_OK); });
}

int sb_target_set_policy(void *target, float min_p, uint32_t top_k, float top_p) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_policy: null target");
  SB_REQUIRE(min_p >= 0.0f && min_p <= 1.0f && top_p > 0.0f && top_p <= 1.0f, "sb_target_set_policy: min_p %g outside 0..1 or top_p %g outside (0, 1]", double(min_p), double(top_p));
  Target *t = static_cast<Target *>(target);
  SB_CUDA(cudaDeviceSynchronize());
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);  // captured steps carry the old policy
  t->graphs.clear();
  t->model->minP = min_p, t->model->topK = top_k, t->model->topP = top_p;
  return SB_OK;
}

int sb_target_set_lane_policies(void *target, const SbLanePolicy *policies_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_lane_policies: null target");
  Target *t = static_cast<Target *>(target);
  QwenTarget &m = *t->model;
  SB_REQUIRE(m.manyRowStep(), "sb_target_set_lane_policies: a target of one lane takes the step's temperature and sb_target_set_policy");
  if (policies_host)
    for (uint32_t l = 0; l < m.lanes(); ++l) {
      const SbLanePolicy &q = policies_host[l];
      SB_REQUIRE(q.temperature >= 0.0f && q.min_p >= 0.0f && q.min_p <= 1.0f && q.top_p > 0.0f && q.top_p <= 1.0f,
                 "sb_target_set_lane_policies: lane %u: temperature %g, min_p %g, top_p %g", l, double(q.temperature), double(q.min_p), double(q.top_p));
    }
  SB_CUDA(cudaDeviceSynchronize());
  if (m.lanePoliciesSet != (policies_host != nullptr)) {  // (only switching them on or off changes the captured step: the values are read on the device)
    for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);
    t->graphs.clear();
  }
  if (policies_host) SB_CUDA(cudaMemcpy(m.lanePolicies.as(), policies_host, sizeof(SbLanePolicy) * m.lanes(), cudaMemcpyHostToDevice));
  m.lanePoliciesSet = policies_host != nullptr;
  return SB_OK;
}

int sb_target_set_stop_tokens(void *target, const uint32_t *stop_tokens_host, uint32_t n_stop) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_stop_tokens: null target");
  SB_REQUIRE(n_stop <= 16 && (!n_stop || stop_tokens_host), "sb_target_set_stop_tokens: up to 16 stop tokens, with their ids");
  Target *t = static_cast<Target *>(target);
  SB_CUDA(cudaDeviceSynchronize());
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);  // captured steps carry the old count
  t->graphs.clear();
  if (n_stop) SB_CUDA(cudaMemcpy(t->model->stopTokens.as(), stop_tokens_host, n_stop * 4, cudaMemcpyHostToDevice));
  t->model->stopCount = n_stop;
  return SB_OK;
}

int sb_target_set_admission(void *target, int constrained, const uint32_t *excluded_host, uint32_t n_excluded) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_admission: null target");
  SB_REQUIRE(n_excluded <= 16 && (!n_excluded || excluded_host), "sb_target_set_admission: up to 16 excluded tokens, with their ids");
  Target *t = static_cast<Target *>(target);
  SB_CUDA(cudaDeviceSynchronize());
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);  // captured steps carry the old admission
  t->graphs.clear();
  if (n_excluded) SB_CUDA(cudaMemcpy(t->model->excludedTokens.as(), excluded_host, n_excluded * 4, cudaMemcpyHostToDevice));
  t->model->constrained = constrained != 0, t->model->excludedCount = n_excluded;
  return SB_OK;
}

int sb_target_set_penalties(void *target, float repetition, float presence, float frequency) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_penalties: null target");
  SB_REQUIRE(repetition > 0.0f, "sb_target_set_penalties: repetition %g is not positive", double(repetition));
  Target *t = static_cast<Target *>(target);
  SB_CUDA(cudaDeviceSynchronize());
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);  // captured steps carry the old policy
  t->graphs.clear();
  t->model->penalties = {repetition, presence, frequency};
  return SB_OK;
}

int sb_target_set_router_scores(void *target, int given) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_set_router_scores: null target");
  Target *t = static_cast<Target *>(target);
  SB_REQUIRE(t->model->config().moe_experts, "sb_target_set_router_scores: the model has no MoE blocks");
  SB_CUDA(cudaDeviceSynchronize());
  for (auto &g : t->graphs) cudaGraphExecDestroy(g.second);  // captured steps carry the old choice
  t->graphs.clear();
  t->model->routerScoresGiven = given != 0;
  return SB_OK;
}

int sb_target_tensor(void *target, int layer, const char *name, void **out_dev, uint64_t *out_bytes) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && name && out_dev && out_bytes, "sb_target_tensor: null pointer");
  Buffer b;
  SB_REQUIRE(static_cast<Target *>(target)->model->find(layer, name, b), "sb_target_tensor: no tensor '%s' in layer %d", name, layer);
  *out_dev = b.as();
  *out_bytes = b.bytes();
  // The caller may write a projection's rows through this address: their image (Q6_K / NVFP4 on the many-row kernel) is
  // made again before the next step.
  for (const char *w : {"in_proj", "attn_q", "attn_k", "attn_v", "attn_qkv", "attn_gate", "out_proj", "ffn_gate", "ffn_up", "ffn_down", "output"})
    if (!strcmp(name, w)) static_cast<Target *>(target)->model->imagesStale = true;
  return SB_OK;
}

int sb_target_tensor_format(void *target, int layer, const char *name, uint32_t *out_format) {
  SB_REQUIRE(target && name && out_format, "sb_target_tensor_format: null pointer");
  SB_REQUIRE(static_cast<Target *>(target)->model->formatOfTensor(layer, name, *out_format), "sb_target_tensor_format: no weight tensor '%s' in layer %d", name, layer);
  return SB_OK;
}

int sb_target_config(void *target, SbTargetConfig *out_config) {
  SB_REQUIRE(target && out_config, "sb_target_config: null pointer");
  *out_config = static_cast<Target *>(target)->model->config();
  return SB_OK;
}

int sb_target_reset(void *target, uint32_t committed) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_reset: null target");
  QwenTarget &m = *static_cast<Target *>(target)->model;
  SB_REQUIRE(committed <= m.config().max_context, "sb_target_reset: %u tokens exceed the context bound %u", committed, m.config().max_context);
  SB_CUDA(cudaDeviceSynchronize());
  const std::vector<uint32_t> all(m.lanes(), committed);  // every lane at the same position
  SB_CUDA(cudaMemcpy(m.committed.as(), all.data(), 4 * all.size(), cudaMemcpyHostToDevice));
  SB_CUDA(cudaMemset(m.pendingRows.as(), 0, 4 * all.size()));
  SB_CUDA(cudaMemset(m.pendingPath.as(), 0, 4 * all.size()));
  m.committedHost = committed;
  m.step = 0;
  return SB_OK;
}

int sb_target_reset_lanes(void *target, const uint32_t *committed_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && committed_host, "sb_target_reset_lanes: null pointer");
  QwenTarget &m = *static_cast<Target *>(target)->model;
  uint32_t most = 0;
  for (uint32_t l = 0; l < m.lanes(); ++l) {
    SB_REQUIRE(committed_host[l] <= m.config().max_context, "sb_target_reset_lanes: lane %u at %u tokens exceeds the context bound %u", l, committed_host[l],
               m.config().max_context);
    most = std::max(most, committed_host[l]);
  }
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpy(m.committed.as(), committed_host, 4 * m.lanes(), cudaMemcpyHostToDevice));
  SB_CUDA(cudaMemset(m.pendingRows.as(), 0, 4 * m.lanes()));
  SB_CUDA(cudaMemset(m.pendingPath.as(), 0, 4 * m.lanes()));
  m.committedHost = most;
  m.step = 0;
  return SB_OK;
}

int sb_target_randomize(void *target, uint64_t seed, uint32_t committed) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_randomize: null target");
  QwenTarget &m = *static_cast<Target *>(target)->model;
  const SbTargetConfig &c = m.local();  // a rank fills its share; tensors every rank holds whole get the same values on every rank
  return guarded([&] {
    uint64_t s = seed * 1000003ull;
    auto next = [&] { return s += 0x632BE59BD9B4E019ull; };
    int st;
#define SB_TRY(x) if ((st = (x)) != SB_OK) return st
    for (auto &w : m.layers()) {
      SB_TRY(fill(kF32Normal, w.attnNorm.buffer, c.hidden, next(), 1.0f, 0.1f));
      SB_TRY(fill(kF32Normal, w.ffnNorm.buffer, c.hidden, next(), 1.0f, 0.1f));
      for (const splash::b200::ops::QuantizedSegment *part : w.inSegments()) SB_TRY(fill_rows(*part, next()));
      SB_TRY(fill_rows(w.outProj, next()));
      if (c.moe_experts) {
        const uint32_t total = m.expertParallel() ? m.expertParallel()->local().expertsTotal() : c.moe_experts + 1;  // (a rank's experts)
        splash::b200::ops::QuantizedSegment e;
        e.format = c.fmt_proj;
        e.rows = w.moe.gate, e.outputSize = total * c.moe_intermediate, e.inputSize = c.hidden;
        SB_TRY(fill_rows(e, next()));
        e.rows = w.moe.up;
        SB_TRY(fill_rows(e, next()));
        e.rows = w.moe.down, e.outputSize = total * c.hidden, e.inputSize = c.moe_intermediate;
        SB_TRY(fill_rows(e, next()));
        SB_TRY(fill(kF32Normal, w.moe.router, w.moe.router.bytes() / 4, next(), 0.0f, 0.05f));
        SB_TRY(fill(kF32Normal, w.moe.sharedGate, c.hidden, next(), 0.0f, 0.02f));
      } else {
        SB_TRY(fill_rows(w.ffnGate, next()));
        SB_TRY(fill_rows(w.ffnUp, next()));
        SB_TRY(fill_rows(w.ffnDown, next()));
      }
      if (w.attention) {
        SB_TRY(fill(kF32Normal, w.qNorm, c.head_dim, next(), 1.0f, 0.1f));
        SB_TRY(fill(kF32Normal, w.kNorm, c.head_dim, next(), 1.0f, 0.1f));
        SB_TRY(fill(kInt8, w.pages.keys, w.pages.keys.bytes(), next(), 0, 0));
        SB_TRY(fill(kInt8, w.pages.values, w.pages.values.bytes(), next(), 0, 0));
        const uint64_t scales = w.pages.keyScales.bytes() / (c.kv_scale_f16 ? 2 : 4);
        SB_TRY(fill(c.kv_scale_f16 ? kF16Uniform : kF32Uniform, w.pages.keyScales, scales, next(), 0.005f, 0.03f));
        SB_TRY(fill(c.kv_scale_f16 ? kF16Uniform : kF32Uniform, w.pages.valueScales, scales, next(), 0.005f, 0.03f));
      } else {
        SB_TRY(fill(kF32Normal, w.ssmAb, w.ssmAb.bytes() / 4, next(), 0.0f, 0.02f));
        SB_TRY(fill(kBf16Normal, w.ssmConv, w.ssmConv.bytes() / 2, next(), 0.0f, 0.4f));
        SB_TRY(fill(kF32NegExp, w.ssmA, c.gdn_value_heads, next(), -3.0f, 0.5f));
        SB_TRY(fill(kBf16Normal, w.ssmDtBias, c.gdn_value_heads, next(), 0.0f, 0.5f));
        SB_TRY(fill(kF32Normal, w.ssmNorm, 128, next(), 1.0f, 0.1f));
        for (int i = 0; i < 2; ++i) {
          SB_TRY(fill(kF32Normal, w.cells[i].state, w.cells[i].state.bytes() / 4, next(), 0.0f, 0.05f));
          SB_TRY(fill(kBf16Normal, w.cells[i].convolution, w.cells[i].convolution.bytes() / 2, next(), 0.0f, 1.0f));
        }
      }
    }
    Buffer b;
    m.find(-1, "output_norm", b);
    SB_TRY(fill(kF32Normal, b, c.hidden, next(), 1.0f, 0.1f));
    splash::b200::ops::QuantizedSegment seg;
    m.find(-1, "token_embd", seg.rows);
    seg.outputSize = c.vocab, seg.inputSize = c.hidden, seg.format = c.fmt_embed;
    SB_TRY(fill_rows(seg, next()));
    m.find(-1, "output", seg.rows);
    seg.format = c.fmt_head, seg.outputSize = m.share().vocab;
    SB_TRY(fill_rows(seg, next()));
    m.imagesStale = true;
#undef SB_TRY
    SB_CUDA(cudaDeviceSynchronize());
    return sb_target_reset(target, committed);
  });
}

constexpr uint32_t kRaggedStep = 1u << 30;  // (internal: the step reads the lanes' own row counts)

static int run_step(Target *t, cudaStream_t stream, uint32_t rows, float temperature, uint32_t flags) {
  QwenTarget &m = *t->model;
  const bool advance = (flags & SB_TARGET_ADVANCE) != 0, tree = (flags & SB_TARGET_TREE) != 0;
  const bool keep = !advance && (flags & SB_TARGET_KEEP_PENDING) != 0, draws = (flags & SB_TARGET_DRAWS) != 0;
  const bool prompt = (flags & SB_TARGET_PROMPT) != 0;
  SB_REQUIRE(!prompt || (advance && !tree), "sb_target_step: SB_TARGET_PROMPT commits a chain: it needs SB_TARGET_ADVANCE and excludes SB_TARGET_TREE");
  const bool ragged = (flags & kRaggedStep) != 0;
  SB_REQUIRE(!ragged || (m.manyRowStep() && !tree), "sb_target_verify_lanes_ragged: blocks of different lengths are chains of a target of several lanes");
  const uint32_t parity = m.step & 1;
  m.promptBlock = prompt;
  m.raggedStep = ragged;
  return guarded([&] {
    if (m.imagesStale) m.buildImages(stream);
    if (flags & SB_TARGET_GRAPH) {
      // The attention plan and the page-table extents are made for a bound of the lane's position; a graph
      // serves until the lane passes its bound.
      const uint32_t bound = std::min(m.config().max_context, (m.committedHost / 1024 + 2) * 1024);
      uint32_t tbits;
      memcpy(&tbits, &temperature, 4);
      const auto key = std::make_tuple(rows, tbits, parity, uint32_t(advance) | (uint32_t(tree) << 1) | (uint32_t(keep) << 2) | (uint32_t(draws) << 3) | (uint32_t(prompt) << 4) | (uint32_t(ragged) << 5), bound);
      auto it = t->graphs.find(key);
      if (it == t->graphs.end()) {
        const uint32_t saved = m.committedHost;
        m.committedHost = bound;
        CommandGraph g{stream, true, 0};
        SB_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        int status = SB_OK;
        try {
          m.encodeVerify(g, rows, temperature, parity, advance, tree, keep, draws);
        } catch (...) {
          cudaGraph_t dead = nullptr;
          cudaStreamEndCapture(stream, &dead);
          if (dead) cudaGraphDestroy(dead);
          m.committedHost = saved;
          throw;
        }
        m.committedHost = saved;
        cudaGraph_t graph = nullptr;
        SB_CUDA(cudaStreamEndCapture(stream, &graph));
        cudaGraphExec_t exec = nullptr;
        const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
        t->launches = g.launches;
        it = t->graphs.emplace(key, exec).first;
        (void)status;
      }
      SB_CUDA(cudaGraphLaunch(it->second, stream));
    } else {
      CommandGraph g{stream, ctx().pdl, 0};
      m.encodeVerify(g, rows, temperature, parity, advance, tree, keep, draws);
      t->launches = g.launches;
    }
    ++m.step;
    if (advance) m.committedHost = std::min(m.config().max_context, m.committedHost + rows);
    return int(SB_OK);
  });
}

int sb_target_step(void *target, void *stream, uint32_t rows, float temperature, uint32_t flags) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_step: null target");
  return run_step(static_cast<Target *>(target), static_cast<Target *>(target)->pick(stream), rows, temperature, flags);
}

// What a step's results must satisfy before a host acts on them (the reference's finalizeDecode,
// runtime/model/Runtime.cpp:2943-2977): 1 <= retained <= rows, the retained rows a mask of that many rows with the anchor among
// them and none past the block, accepted < rows and <= retained, and every retained token one of the vocabulary (a row without
// a selectable logit selects the sentinel 0xFFFFFFFF, which must not be retained as a token).
static int check_lane_results(const uint32_t *results, const uint32_t *tokens, uint32_t rows, uint32_t vocab, uint32_t lane) {
  const uint32_t retained = results[0], accepted = results[1], mask = results[2];
  if (!rows) return retained || accepted || mask ? fail(SB_ERR_DEVICE, "lane %u: a lane without rows retained %u tokens", lane, retained) : int(SB_OK);
  if (!retained || retained > rows || uint32_t(__builtin_popcount(mask)) != retained || !(mask & 1u) || (mask >> (rows - 1)) > 1u)
    return fail(SB_ERR_DEVICE, "lane %u: invalid retention (retained %u of %u rows, rows 0x%x)", lane, retained, rows, mask);
  if (accepted >= rows || accepted > retained) return fail(SB_ERR_DEVICE, "lane %u: accepted %u of %u rows, retained %u", lane, accepted, rows, retained);
  for (uint32_t i = 0; i < retained; ++i)
    if (tokens[i] >= vocab) return fail(SB_ERR_DEVICE, "lane %u: retained token %u is 0x%x, not one of the vocabulary's %u (a row without a selectable logit)", lane, i, tokens[i], vocab);
  return SB_OK;
}

int sb_target_verify(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host, uint32_t rows, float temperature,
                     uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && tokens_host && out_tokens_host && out_results_host, "sb_target_verify: null pointer");
  SB_REQUIRE(rows >= 1 && rows <= splash::b200::model::kVerifyRows, "sb_target_verify: rows = %u outside 1..16", rows);
  SB_REQUIRE(temperature == 0.0f || uniforms_host, "sb_target_verify: a sampled policy needs uniforms");
  Target *t = static_cast<Target *>(target);
  QwenTarget &m = *t->model;
  SB_REQUIRE(m.lanes() == 1, "sb_target_verify: the target steps %u lanes; use sb_target_verify_lanes", m.lanes());
  cudaStream_t s = t->pick(stream);
  const uint32_t before = m.committedHost;
  SB_CUDA(cudaMemcpyAsync(m.tokens.as(), tokens_host, rows * 4, cudaMemcpyHostToDevice, s));
  if (uniforms_host) SB_CUDA(cudaMemcpyAsync(m.uniforms.as(), uniforms_host, 80 * 4, cudaMemcpyHostToDevice, s));
  const int st = run_step(t, s, rows, temperature, flags);
  if (st != SB_OK) return st;
  SB_CUDA(cudaMemcpyAsync(t->results_pinned, m.results.as(), 16, cudaMemcpyDeviceToHost, s));
  SB_CUDA(cudaMemcpyAsync(t->results_pinned + 4, m.selected.as(), rows * 4, cudaMemcpyDeviceToHost, s));
  SB_CUDA(cudaStreamSynchronize(s));
  memcpy(out_results_host, t->results_pinned, 16);
  memcpy(out_tokens_host, t->results_pinned + 4, rows * 4);
  if (flags & SB_TARGET_ADVANCE) m.committedHost = before + std::min(t->results_pinned[0], rows);  // the exact position again
  return check_lane_results(t->results_pinned, t->results_pinned + 4, rows, m.config().vocab, 0);
}

int sb_target_verify_lanes(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host, uint32_t rows, float temperature,
                           uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && tokens_host && out_tokens_host && out_results_host, "sb_target_verify_lanes: null pointer");
  SB_REQUIRE(rows >= 1 && rows <= splash::b200::model::kVerifyRows, "sb_target_verify_lanes: rows = %u outside 1..16", rows);
  SB_REQUIRE((temperature == 0.0f && !static_cast<Target *>(target)->model->lanePoliciesSet) || uniforms_host, "sb_target_verify_lanes: a sampled policy (or policies a lane) needs uniforms");
  Target *t = static_cast<Target *>(target);
  QwenTarget &m = *t->model;
  const uint32_t L = m.lanes();
  cudaStream_t s = t->pick(stream);
  const uint32_t before = m.committedHost;
  SB_CUDA(cudaMemcpyAsync(m.tokens.as(), tokens_host, size_t(16) * L * 4, cudaMemcpyHostToDevice, s));
  if (uniforms_host) SB_CUDA(cudaMemcpyAsync(m.uniforms.as(), uniforms_host, size_t(80) * L * 4, cudaMemcpyHostToDevice, s));
  const int st = run_step(t, s, rows, temperature, flags);
  if (st != SB_OK) return st;
  SB_CUDA(cudaMemcpyAsync(t->results_pinned, m.results.as(), size_t(16) * L, cudaMemcpyDeviceToHost, s));
  SB_CUDA(cudaMemcpyAsync(t->results_pinned + 4 * L, m.selected.as(), size_t(16) * L * 4, cudaMemcpyDeviceToHost, s));
  SB_CUDA(cudaStreamSynchronize(s));
  memcpy(out_results_host, t->results_pinned, size_t(16) * L);
  memcpy(out_tokens_host, t->results_pinned + 4 * L, size_t(16) * L * 4);
  if (flags & SB_TARGET_ADVANCE) {  // the exact bound again: the furthest lane
    uint32_t most = 0;
    for (uint32_t l = 0; l < L; ++l) most = std::max(most, std::min(t->results_pinned[4 * l], rows));
    m.committedHost = std::min(m.config().max_context, before + most);
  }
  for (uint32_t l = 0; l < L; ++l) {
    const uint32_t lane_rows = (flags & kRaggedStep) ? std::min(t->lane_rows_host[l], rows) : rows;
    const int st = check_lane_results(t->results_pinned + 4 * l, t->results_pinned + 4 * L + 16 * l, lane_rows, m.config().vocab, l);
    if (st != SB_OK) return st;
  }
  return SB_OK;
}

int sb_target_verify_lanes_ragged(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host, const uint32_t *lane_rows_host,
                                  float temperature, uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && lane_rows_host, "sb_target_verify_lanes_ragged: null pointer");
  SB_REQUIRE(!(flags & (SB_TARGET_TREE | kRaggedStep)), "sb_target_verify_lanes_ragged: chains only");
  Target *t = static_cast<Target *>(target);
  QwenTarget &m = *t->model;
  uint32_t most = 0;
  for (uint32_t l = 0; l < m.lanes(); ++l) {
    SB_REQUIRE(lane_rows_host[l] <= splash::b200::model::kVerifyRows, "sb_target_verify_lanes_ragged: lane %u has %u rows (up to 16)", l, lane_rows_host[l]);
    most = std::max(most, lane_rows_host[l]);
  }
  SB_REQUIRE(most >= 1, "sb_target_verify_lanes_ragged: no lane has a row");
  memcpy(t->lane_rows_host, lane_rows_host, size_t(4) * m.lanes());
  SB_CUDA(cudaMemcpyAsync(m.laneRows.as(), t->lane_rows_host, size_t(4) * m.lanes(), cudaMemcpyHostToDevice, t->pick(stream)));
  return sb_target_verify_lanes(target, stream, tokens_host, uniforms_host, most, temperature, flags | kRaggedStep, out_tokens_host, out_results_host);
}

int sb_target_verify_tree(void *target, void *stream, const uint32_t *tokens_host, const void *tree_host, const float *uniforms_host, uint32_t rows,
                          float temperature, uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target && tree_host, "sb_target_verify_tree: null pointer");
  SB_REQUIRE(rows >= 1 && rows <= splash::b200::model::kVerifyRows, "sb_target_verify_tree: rows = %u outside 1..16", rows);
  // Parents come before their children and a row's ancestors are rows before it: what the kernels index by.
  const uint32_t *t = static_cast<const uint32_t *>(tree_host);
  for (uint32_t r = 0; r < rows; ++r) {
    const uint32_t ancestors = t[2 * r], parent = t[2 * r + 1] & 0xffffu, depth = t[2 * r + 1] >> 16;
    SB_REQUIRE((ancestors >> r & 1u) && (ancestors & 1u) && !(ancestors >> (r + 1)) && parent <= r && depth + 1 == uint32_t(__builtin_popcount(ancestors)) &&
                   (r == 0 || (parent < r && ancestors == (t[2 * parent] | (1u << r)))),
               "sb_target_verify_tree: row %u is not a tree row (ancestors 0x%x, parent %u, depth %u)", r, ancestors, parent, depth);
  }
  Target *tg = static_cast<Target *>(target);
  SB_CUDA(cudaMemcpyAsync(tg->model->tree.as(), tree_host, rows * 8, cudaMemcpyHostToDevice, tg->pick(stream)));
  return sb_target_verify(target, stream, tokens_host, uniforms_host, rows, temperature, flags | SB_TARGET_TREE, out_tokens_host, out_results_host);
}

int sb_target_stats(void *target, uint32_t rows, uint32_t *out_launches, uint64_t *out_weight_bytes, uint64_t *out_kv_bytes,
                    uint64_t *out_state_bytes) {
  SB_NEED_DEVICE();
  SB_REQUIRE(target, "sb_target_stats: null target");
  Target *t = static_cast<Target *>(target);
  if (out_launches) *out_launches = t->launches;
  if (out_weight_bytes) *out_weight_bytes = t->model->weightBytes(rows);
  if (out_kv_bytes) *out_kv_bytes = t->model->kvBytes(t->model->committedHost + rows);
  if (out_state_bytes) *out_state_bytes = t->model->stateBytes();
  return SB_OK;
}

}  // extern "C"
