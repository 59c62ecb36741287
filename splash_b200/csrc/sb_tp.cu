// Tensor parallelism between the GPUs of one node (one process per GPU): the group's window of peer-mapped
// memory, its rendezvous through CUDA IPC handles, and the all-gather kernel. The reference runs on one GPU
// and has no counterpart; the split it would take is the one its projections admit (column split of the input,
// gate and up projections and of the vocabulary, split of the reduction dimension of out_proj and down), whose
// partial sums are what ops::Linear's split-K reduction (runtime/metal/kernels/common/split_reduce.h:24-55)
// already adds. Layout and protocol: sb_tp_internal.cuh.
#include <string.h>

#include "sb_ptx.cuh"
#include "sb_tp_internal.cuh"

namespace sb {

struct TpGroup {
  uint32_t world = 0, rank = 0, width = 0, gather_width = 0;
  uint8_t *window = nullptr;  // this rank's
  size_t window_bytes = 0, inbox_off = 0, sums_off = 0, flags_off = 0, gather_off = 0;
  uint8_t *peer[kTpMaxWorld] = {};  // every rank's window as mapped here (peer[rank] == window)
  uint32_t *epoch = nullptr;  // two words: the exchange count, and `ready`
  bool connected = false;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int tp_exchange(void *group, uint32_t index, bool gather, TpExchange &out) {
  TpGroup *g = static_cast<TpGroup *>(group);
  if (!g || !g->connected) return fail(SB_ERR_INVALID, "tensor-parallel group is not connected (sb_tp_connect)");
  out = TpExchange{};
  out.world = g->world, out.rank = g->rank, out.index = index, out.width = gather ? g->gather_width : g->width;
  out.epoch_base = g->epoch, out.ready = g->epoch + 1, out.status = ctx().status_dev;
  out.two_shot = ctx().tp_exchange_shots ? ctx().tp_exchange_shots == 2 : g->world > 2;
  out.wait_ns = ctx().wait_ns;
  for (uint32_t p = 0; p < g->world; ++p) {
    out.sums[p] = reinterpret_cast<uint4 *>(g->peer[p] + g->sums_off);
    out.data[p] = reinterpret_cast<float *>(g->peer[p] + (gather ? g->gather_off : g->inbox_off));
    out.flags[p] = reinterpret_cast<uint32_t *>(g->peer[p] + g->flags_off);
  }
  return SB_OK;
}
uint32_t *tp_epoch_word(void *group) { return group ? static_cast<TpGroup *>(group)->epoch : nullptr; }

// Every rank's columns [column0, column0 + columns) of the gather matrix go to the same place in every peer's
// matrix; the kernel returns when all peers' columns have arrived here.
__global__ void __launch_bounds__(256) tp_gather_kernel(const TpExchange x, uint32_t rows, uint32_t column0, uint32_t columns) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t epoch = tp_epoch(x);
  const bool healthy = tp_healthy(x);
  const uint32_t quads = columns / 4, total = rows * quads;
  const float *own = x.data[x.rank];
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const size_t at = size_t(i / quads) * x.width + column0 + 4 * (i % quads);
    const float4 v = __ldcg(reinterpret_cast<const float4 *>(own + at));
    for (uint32_t p = 0; p < x.world; ++p)
      if (p != x.rank) *reinterpret_cast<float4 *>(x.data[p] + at) = v;
  }
  tp_signal_and_wait(x, epoch, blockIdx.x, gridDim.x, healthy);
}

// Later kernels may start before the kernels ahead of them complete, and the exchanges' kernels read the count
// when they start: so this kernel lets its dependents start only after the count has moved.
__global__ void tp_advance_kernel(uint32_t *epoch, uint32_t exchanges) {
  pdl_wait();
  if (threadIdx.x == 0) {
    *epoch += exchanges;
    __threadfence();
  }
  __syncthreads();
  pdl_launch_dependents();
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_tp_create(uint32_t world, uint32_t rank, uint32_t width, uint32_t gather_width, void **out_group) {
  SB_NEED_DEVICE();
  SB_REQUIRE(out_group, "sb_tp_create: null group");
  SB_REQUIRE(world >= 2 && world <= uint32_t(kTpMaxWorld) && rank < world, "sb_tp_create: rank %u of %u ranks (2 to %d ranks)", rank, world, kTpMaxWorld);
  SB_REQUIRE(width && width % 256 == 0, "sb_tp_create: width %u is not a multiple of 256", width);
  SB_REQUIRE(gather_width % 4 == 0, "sb_tp_create: gather width %u is not a multiple of 4", gather_width);
  TpGroup *g = new TpGroup;
  g->world = world, g->rank = rank, g->width = width, g->gather_width = gather_width;
  g->inbox_off = 0;
  g->sums_off = align_up(size_t(2) * world * 16 * width * 8, 256);   // (inbox: units of 16 bytes hold two values)
  g->flags_off = g->sums_off + align_up(size_t(2) * 16 * width * 4, 256);  // (finished sums: units of 16 bytes hold four bf16)
  g->gather_off = g->flags_off + align_up(size_t(world) * kTpGatherCtas * 4, 256);
  g->window_bytes = g->gather_off + align_up(size_t(16) * gather_width * 4, 256) + 256;
  cudaError_t e = cudaMalloc(&g->window, g->window_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&g->epoch, 8);
  if (e == cudaSuccess) e = cudaMemset(g->window, 0, g->window_bytes);
  if (e == cudaSuccess) e = cudaMemset(g->epoch, 0, 8);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(g->window), cudaFree(g->epoch);
    delete g;
    return e == cudaErrorMemoryAllocation ? fail(SB_ERR_OOM, "sb_tp_create: out of device memory") : cuda_fail(e, "sb_tp_create");
  }
  g->peer[rank] = g->window;
  *out_group = g;
  return SB_OK;
}

int sb_tp_destroy(void *group) {
  TpGroup *g = static_cast<TpGroup *>(group);
  if (!g) return SB_OK;
  cudaDeviceSynchronize();
  for (uint32_t p = 0; p < g->world; ++p)
    if (p != g->rank && g->peer[p]) cudaIpcCloseMemHandle(g->peer[p]);
  cudaFree(g->window), cudaFree(g->epoch);
  delete g;
  return SB_OK;
}

int sb_tp_export(void *group, void *handle_out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(group && handle_out, "sb_tp_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == SB_TP_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  SB_CUDA(cudaIpcGetMemHandle(&h, static_cast<TpGroup *>(group)->window));
  memcpy(handle_out, &h, sizeof h);
  return SB_OK;
}

int sb_tp_connect(void *group, const void *handles) {
  SB_NEED_DEVICE();
  SB_REQUIRE(group && handles, "sb_tp_connect: null pointer");
  TpGroup *g = static_cast<TpGroup *>(group);
  SB_REQUIRE(!g->connected, "sb_tp_connect: the group is connected already");
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

int sb_tp_gather_matrix(void *group, void **out_dev, uint64_t *out_bytes) {
  SB_REQUIRE(group && out_dev && out_bytes, "sb_tp_gather_matrix: null pointer");
  TpGroup *g = static_cast<TpGroup *>(group);
  *out_dev = g->window + g->gather_off;
  *out_bytes = uint64_t(16) * g->gather_width * 4;
  return SB_OK;
}

int sb_tp_all_gather(void *stream, void *group, uint32_t index, uint32_t rows, uint32_t column0, uint32_t columns) {
  SB_NEED_DEVICE();
  TpExchange x;
  const int st = tp_exchange(group, index, true, x);
  if (st != SB_OK) return st;
  SB_REQUIRE(rows >= 1 && rows <= 16, "sb_tp_all_gather: rows = %u outside 1..16", rows);
  SB_REQUIRE(column0 % 4 == 0 && columns % 4 == 0 && column0 + columns <= x.width, "sb_tp_all_gather: columns [%u, %u) of %u, in fours", column0,
             column0 + columns, x.width);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kTpGatherCtas), cfg.blockDim = dim3(256), cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = ctx().pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, tp_gather_kernel, x, rows, column0, columns));
  return SB_OK;
}

int sb_tp_set_exchange(int shots) {
  SB_REQUIRE(shots >= 0 && shots <= 2, "sb_tp_set_exchange: %d shots (0: by the number of ranks, 1 or 2)", shots);
  ctx().tp_exchange_shots = shots;
  return SB_OK;
}

int sb_set_wait_limit_ns(uint64_t ns) {
  ctx().wait_ns = ns ? ns : kTpWaitNs;
  return SB_OK;
}

int sb_tp_advance(void *stream, void *group, uint32_t exchanges) {
  SB_NEED_DEVICE();
  SB_REQUIRE(group, "sb_tp_advance: null group");
  tp_advance_kernel<<<1, 32, 0, as_stream(stream)>>>(static_cast<TpGroup *>(group)->epoch, exchanges);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // extern "C"
