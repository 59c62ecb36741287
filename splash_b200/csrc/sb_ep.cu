// Expert parallelism between the GPUs of one node (one process per GPU): every rank steps its own lanes and holds a
// share of the experts of the MoE blocks. A block's routed rows meet their experts in two exchanges through peer-mapped
// memory (CUDA IPC windows over NVLink, plain stores and loads, as the tensor-parallel exchange of sb_tp.cu: no TMA, no
// multicast):
//   dispatch  every rank's normalised rows, routes and route weights are stored into every rank's `gathered` arrays (rows
//             [world][rows][hidden] bf16, selected and weights [world][rows][routes]); each rank then runs the routes that
//             name its experts, over all ranks' rows (sb_moe_experts_partial)
//   combine   a rank's weighted sums for the rows of rank d (fp32 [rows][hidden]) are stored into d's inbox [source];
//             d adds the world's contributions in rank order onto its residual and rounds once
// The reference runs on one GPU; its MoE::addRouted gathers rows per expert and combines per row inside one device
// (runtime/ops/MoE.cpp:122-187,260-270). Both exchanges are dense: a row travels to every rank whether or not one of its
// routes lives there (top 8 of 256 experts over 8 ranks reach 5.3 ranks on average, so a sparse dispatch would move two
// thirds of this).
//
// Ordering: exchanges are numbered by a device word the exchange kernels advance themselves when their last CTA is done
// (every kernel of the stream waits for the kernel ahead before it reads the word). CTA j of a kernel stores its part into
// the peers, publishes the number in the peers' flag [source][j] (system-scope release) and waits for the peers' flag of
// its own index (acquire), bounded by the clock like every wait here. One slot per array suffices: a rank writes
// `gathered` again only after its combine has seen the peers' contributions, which they send after their last read of
// `gathered`; it writes an inbox again only after the next dispatch has seen the peers' rows, which they send after their
// combine has read its inbox.
#include <string.h>

#include "sb_ptx.cuh"
#include "sb_tp_internal.cuh"

namespace sb {

constexpr uint32_t kEpCtas = 64, kEpThreads = 256;

struct EpGroup {
  uint32_t world = 0, rank = 0, rows = 0, hidden = 0, routes = 0;
  uint8_t *window = nullptr;
  size_t window_bytes = 0, rows_off = 0, selected_off = 0, weights_off = 0, inbox_off = 0, flags_off = 0;
  uint8_t *peer[kTpMaxWorld] = {};
  uint32_t *words = nullptr;  // [0] exchanges completed, [1] CTAs of the running exchange that are done
  bool connected = false;
};

struct EpParams {
  uint32_t world, rank, rows, hidden, routes;
  uint32_t *words, *status;
  uint64_t wait_ns;
  uint8_t *peer[kTpMaxWorld];
  size_t rows_off, selected_off, weights_off, inbox_off, flags_off;
};

__device__ __forceinline__ void ep_signal_and_wait(const EpParams &p, uint32_t epoch, bool healthy) {
  __syncthreads();
  const uint32_t t = threadIdx.x;
  if (t < p.world && t != p.rank) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t *>(p.peer[t] + p.flags_off) + p.rank * kEpCtas + blockIdx.x, epoch);
    if (healthy) tp_wait_flag(reinterpret_cast<const uint32_t *>(p.peer[p.rank] + p.flags_off) + t * kEpCtas + blockIdx.x, epoch, p.status, p.wait_ns);
  }
  __syncthreads();
}
// The kernel's last CTA moves the exchange count on (the next exchange kernel reads it after this kernel has completed).
__device__ __forceinline__ void ep_finish(const EpParams &p) {
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.words + 1, 1u) == gridDim.x - 1) {
      p.words[1] = 0;
      p.words[0] += 1;
      __threadfence();
    }
  }
}

__global__ void __launch_bounds__(kEpThreads) ep_gather_kernel(const EpParams p, const uint4 *rows, const uint32_t *selected, const float *weights) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t *>(p.words) + 1u;
  const bool healthy = *reinterpret_cast<const volatile uint32_t *>(p.status) == SB_DEV_OK;
  const uint32_t units = p.rows * p.hidden / 8, routes = p.rows * p.routes;
  const uint32_t tid = blockIdx.x * kEpThreads + threadIdx.x, stride = kEpCtas * kEpThreads;
  for (uint32_t i = tid; i < units; i += stride) {
    const uint4 v = __ldcg(rows + i);
    for (uint32_t d = 0; d < p.world; ++d) reinterpret_cast<uint4 *>(p.peer[d] + p.rows_off)[size_t(p.rank) * units + i] = v;
  }
  for (uint32_t i = tid; i < routes; i += stride) {
    const uint32_t s = __ldcg(selected + i);
    const float w = __ldcg(weights + i);
    for (uint32_t d = 0; d < p.world; ++d) {
      reinterpret_cast<uint32_t *>(p.peer[d] + p.selected_off)[size_t(p.rank) * routes + i] = s;
      reinterpret_cast<float *>(p.peer[d] + p.weights_off)[size_t(p.rank) * routes + i] = w;
    }
  }
  ep_signal_and_wait(p, epoch, healthy);
  ep_finish(p);
}

// partial: fp32 [world][rows][hidden], this rank's weighted sums for every rank's rows. out = bf16(residual + the ranks'
// sums for this rank's rows, added in rank order).
__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const EpParams p, const float4 *partial, const uint2 *residual, uint2 *out) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t *>(p.words) + 1u;
  const bool healthy = *reinterpret_cast<const volatile uint32_t *>(p.status) == SB_DEV_OK;
  const uint32_t quads = p.rows * p.hidden / 4;
  const uint32_t tid = blockIdx.x * kEpThreads + threadIdx.x, stride = kEpCtas * kEpThreads;
  for (uint32_t d = 0; d < p.world; ++d) {
    if (d == p.rank) continue;
    float4 *inbox = reinterpret_cast<float4 *>(p.peer[d] + p.inbox_off) + size_t(p.rank) * quads;
    for (uint32_t i = tid; i < quads; i += stride) inbox[i] = __ldcg(partial + size_t(d) * quads + i);
  }
  ep_signal_and_wait(p, epoch, healthy);
  const float4 *own_inbox = reinterpret_cast<const float4 *>(p.peer[p.rank] + p.inbox_off);
  for (uint32_t i = tid; i < quads; i += stride) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (uint32_t s = 0; s < p.world; ++s) {
      const float4 v = s == p.rank ? __ldcg(partial + size_t(p.rank) * quads + i) : __ldcv(own_inbox + size_t(s) * quads + i);
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    const uint2 r = residual ? residual[i] : make_uint2(0, 0);
    const uint32_t lo = uint32_t(float_to_bf16_bits(bf16_bits_to_float(r.x & 0xffffu) + acc.x)) | (uint32_t(float_to_bf16_bits(bf16_bits_to_float(r.x >> 16) + acc.y)) << 16);
    const uint32_t hi = uint32_t(float_to_bf16_bits(bf16_bits_to_float(r.y & 0xffffu) + acc.z)) | (uint32_t(float_to_bf16_bits(bf16_bits_to_float(r.y >> 16) + acc.w)) << 16);
    out[i] = make_uint2(lo, hi);
  }
  ep_finish(p);
}

static size_t ep_align(size_t v) { return (v + 255) / 256 * 256; }

static int ep_params(void *group, EpParams &p) {
  EpGroup *g = static_cast<EpGroup *>(group);
  if (!g || !g->connected) return fail(SB_ERR_INVALID, "expert-parallel group is not connected (sb_ep_connect)");
  p = EpParams{};
  p.world = g->world, p.rank = g->rank, p.rows = g->rows, p.hidden = g->hidden, p.routes = g->routes;
  p.words = g->words, p.status = ctx().status_dev, p.wait_ns = ctx().wait_ns;
  for (uint32_t r = 0; r < g->world; ++r) p.peer[r] = g->peer[r];
  p.rows_off = g->rows_off, p.selected_off = g->selected_off, p.weights_off = g->weights_off, p.inbox_off = g->inbox_off, p.flags_off = g->flags_off;
  return SB_OK;
}

template <class K, class... A> static int ep_launch(K kernel, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kEpCtas), cfg.blockDim = dim3(kEpThreads), cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = ctx().pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_ep_create(uint32_t world, uint32_t rank, uint32_t rows, uint32_t hidden, uint32_t routes, void **out_group) {
  SB_NEED_DEVICE();
  SB_REQUIRE(out_group, "sb_ep_create: null group");
  SB_REQUIRE(world >= 2 && world <= uint32_t(kTpMaxWorld) && rank < world, "sb_ep_create: rank %u of %u ranks (2 to %d ranks)", rank, world, kTpMaxWorld);
  SB_REQUIRE(rows && hidden && hidden % 8 == 0 && routes, "sb_ep_create: %u rows of width %u (a multiple of 8) with %u routes", rows, hidden, routes);
  EpGroup *g = new EpGroup;
  g->world = world, g->rank = rank, g->rows = rows, g->hidden = hidden, g->routes = routes;
  size_t at = 0;
  auto take = [&](size_t bytes) { const size_t here = at; at += ep_align(bytes); return here; };
  g->rows_off = take(size_t(world) * rows * hidden * 2);
  g->selected_off = take(size_t(world) * rows * routes * 4), g->weights_off = take(size_t(world) * rows * routes * 4);
  g->inbox_off = take(size_t(world) * rows * hidden * 4);
  g->flags_off = take(size_t(world) * kEpCtas * 4);
  g->window_bytes = at;
  cudaError_t e = cudaMalloc(&g->window, g->window_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&g->words, 8);
  if (e == cudaSuccess) e = cudaMemset(g->window, 0, g->window_bytes);
  if (e == cudaSuccess) e = cudaMemset(g->words, 0, 8);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(g->window), cudaFree(g->words);
    delete g;
    return e == cudaErrorMemoryAllocation ? fail(SB_ERR_OOM, "sb_ep_create: out of device memory") : cuda_fail(e, "sb_ep_create");
  }
  g->peer[rank] = g->window;
  *out_group = g;
  return SB_OK;
}

int sb_ep_destroy(void *group) {
  EpGroup *g = static_cast<EpGroup *>(group);
  if (!g) return SB_OK;
  cudaDeviceSynchronize();
  for (uint32_t p = 0; p < g->world; ++p)
    if (p != g->rank && g->peer[p]) cudaIpcCloseMemHandle(g->peer[p]);
  cudaFree(g->window), cudaFree(g->words);
  delete g;
  return SB_OK;
}

int sb_ep_export(void *group, void *handle_out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(group && handle_out, "sb_ep_export: null pointer");
  cudaIpcMemHandle_t h;
  SB_CUDA(cudaIpcGetMemHandle(&h, static_cast<EpGroup *>(group)->window));
  memcpy(handle_out, &h, sizeof h);
  return SB_OK;
}

int sb_ep_connect(void *group, const void *handles) {
  SB_NEED_DEVICE();
  SB_REQUIRE(group && handles, "sb_ep_connect: null pointer");
  EpGroup *g = static_cast<EpGroup *>(group);
  SB_REQUIRE(!g->connected, "sb_ep_connect: the group is connected already");
  for (uint32_t p = 0; p < g->world; ++p) {
    if (p == g->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t *>(handles) + size_t(p) * SB_TP_HANDLE_BYTES, sizeof h);
    void *mapped = nullptr;
    SB_CUDA(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess));
    g->peer[p] = static_cast<uint8_t *>(mapped);
  }
  g->connected = true;
  return SB_OK;
}

int sb_ep_gathered(void *group, void **out_rows, uint32_t **out_selected, float **out_weights) {
  SB_REQUIRE(group && out_rows && out_selected && out_weights, "sb_ep_gathered: null pointer");
  EpGroup *g = static_cast<EpGroup *>(group);
  *out_rows = g->window + g->rows_off;
  *out_selected = reinterpret_cast<uint32_t *>(g->window + g->selected_off);
  *out_weights = reinterpret_cast<float *>(g->window + g->weights_off);
  return SB_OK;
}

int sb_ep_dispatch(void *stream, void *group, const void *rows, const uint32_t *selected, const float *weights) {
  SB_NEED_DEVICE();
  SB_REQUIRE(rows && selected && weights, "sb_ep_dispatch: null pointer");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(rows) & 15) == 0, "sb_ep_dispatch: rows must be 16-byte aligned");
  EpParams p;
  const int st = ep_params(group, p);
  if (st != SB_OK) return st;
  return ep_launch(ep_gather_kernel, as_stream(stream), p, static_cast<const uint4 *>(rows), selected, weights);
}

int sb_ep_combine(void *stream, void *group, const float *partial, const void *residual, void *out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(partial && out, "sb_ep_combine: null pointer");
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
             "sb_ep_combine: pointers must be 16-byte aligned");
  EpParams p;
  const int st = ep_params(group, p);
  if (st != SB_OK) return st;
  return ep_launch(ep_combine_kernel, as_stream(stream), p, reinterpret_cast<const float4 *>(partial), static_cast<const uint2 *>(residual),
                   static_cast<uint2 *>(out));
}

}  // extern "C"
