// Context, memory, streams, events and graph capture of the C ABI (include/splash_b200.h):
// the part of the reference's MetalBackend the verify step needs (buffers, one command stream,
// completion events; runtime/metal/MetalBackend.hpp:375-547), on the CUDA runtime.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <map>
#include <mutex>
#include <thread>

#include "sb_internal.h"

namespace sb {

static thread_local char g_error[512] = "";

Context &ctx() {
  static Context c;
  return c;
}

int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return status;
}

int cuda_fail(cudaError_t e, const char *what) {
  const int status = e == cudaErrorMemoryAllocation ? SB_ERR_OOM
                     : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? SB_ERR_NO_DEVICE
                                                                                   : SB_ERR_CUDA;
  return fail(status, "%s: %s", what, cudaGetErrorString(e));
}

// Allocations by base address with a holder count: the allocation itself holds one, every live view one more, and the
// memory goes back to the driver when the last holder lets go (the reference's buffers are ref-counted handles whose
// views keep the base alive, runtime/metal/MetalBackend.hpp:42-78).
struct Allocation {
  size_t bytes = 0;
  uint32_t holders = 0;
};
static std::mutex g_alloc_mutex;
static std::map<uintptr_t, Allocation> g_allocs;       // base -> allocation
static std::map<uintptr_t, std::pair<uintptr_t, uint32_t>> g_views;  // view address (not a base) -> {base, live views there}

// The allocation that holds `p`, or end().
static std::map<uintptr_t, Allocation>::iterator owner_of(uintptr_t p) {
  auto it = g_allocs.upper_bound(p);
  if (it == g_allocs.begin()) return g_allocs.end();
  --it;
  return p < it->first + it->second.bytes ? it : g_allocs.end();
}

// The one command the boundary lets be in flight (sb_submit): its completion event and whether a ticket is out.
static std::mutex g_ticket_mutex;
static cudaEvent_t g_ticket_event = nullptr;
static uint64_t g_ticket_serial = 0;
static bool g_ticket_out = false;

}  // namespace sb

using namespace sb;

extern "C" {

int sb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

const char *sb_last_error(void) { return g_error; }

int sb_init(int device) {
  Context &c = ctx();
  if (sb_device_count() <= device || device < 0) return fail(SB_ERR_NO_DEVICE, "no CUDA device %d", device);
  SB_CUDA(cudaSetDevice(device));
  if (c.ready && c.device == device) return SB_OK;
  cudaDeviceProp prop;
  SB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(SB_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                                    device, prop.major, prop.minor);
  c.device = device;
  c.sm_count = prop.multiProcessorCount;
  SB_CUDA(cudaMalloc(&c.status_dev, sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.status_dev, 0, sizeof(uint32_t)));
  // Split-K scratch: 8 slices x 16 rows x 2 x 17408 gate/up columns in fp32 covers every dense
  // projection of the supported shapes; the vocabulary projection runs with at most 2 slices.
  c.linear_partials_bytes = size_t(64) << 20;
  SB_CUDA(cudaMalloc(&c.linear_partials, c.linear_partials_bytes));
  c.prepared_bytes = 64 + size_t(72) * 8704;  // k up to 18432
  SB_CUDA(cudaMalloc(&c.prepared, c.prepared_bytes));
  c.wide_prepared_bytes = 4 * (1024 + size_t(128) * 18432 * 2);
  SB_CUDA(cudaMalloc(&c.wide_prepared, c.wide_prepared_bytes));
  c.linear_counter_count = 1u << 16;
  SB_CUDA(cudaMalloc(&c.linear_counters, c.linear_counter_count * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.linear_counters, 0, c.linear_counter_count * sizeof(uint32_t)));
  c.attn_workspace_bytes = size_t(32) << 20;
  SB_CUDA(cudaMalloc(&c.attn_workspace, c.attn_workspace_bytes));
  // (per lane of a step of several lanes: 128 attention counters; the GDN scratch and counters hold kGdnScratchHeads heads over all lanes)
  SB_CUDA(cudaMalloc(&c.attn_counters, kAttnCounterWords * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.attn_counters, 0, kAttnCounterWords * sizeof(uint32_t)));
  SB_CUDA(cudaMalloc(&c.gdn_scratch, size_t(kGdnScratchHeads) * 16 * 128 * 2));
  SB_CUDA(cudaMalloc(&c.gdn_counters, kGdnScratchHeads * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.gdn_counters, 0, kGdnScratchHeads * sizeof(uint32_t)));
  c.ready = true;
  return SB_OK;
}

uint64_t sb_struct_bytes(const char *name) {
  if (!name) return 0;
#define SB_SIZE_OF(T) if (!strcmp(name, #T)) return sizeof(T)
  SB_SIZE_OF(SbLinearArgs);
  SB_SIZE_OF(SbLinearPlan);
  SB_SIZE_OF(SbKvLayer);
  SB_SIZE_OF(SbAttnStoreArgs);
  SB_SIZE_OF(SbAttnArgs);
  SB_SIZE_OF(SbGdnTape);
  SB_SIZE_OF(SbGdnArgs);
  SB_SIZE_OF(SbSampleArgs);
  SB_SIZE_OF(SbPenaltyArgs);
  SB_SIZE_OF(SbAcceptArgs);
  SB_SIZE_OF(SbSelectAcceptArgs);
  SB_SIZE_OF(SbAdmitArgs);
  SB_SIZE_OF(SbLanePolicy);
  SB_SIZE_OF(SbGgufTensor);
  SB_SIZE_OF(SbMoeRouteArgs);
  SB_SIZE_OF(SbMoeExpertArgs);
  SB_SIZE_OF(SbTargetConfig);
  SB_SIZE_OF(SbTargetShare);
#undef SB_SIZE_OF
  return 0;
}

int sb_sm_count(void) { return ctx().ready ? ctx().sm_count : 0; }

int sb_device_status(uint32_t *status) {
  SB_NEED_DEVICE();
  SB_REQUIRE(status, "status is null");
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpy(status, ctx().status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*status) {
    // A kernel that gave up may have left its arrival counters part-way: the next launch must find them at zero, or its
    // own wait would pass early on a stale count.
    Context &c = ctx();
    SB_CUDA(cudaMemset(c.status_dev, 0, sizeof(uint32_t)));
    SB_CUDA(cudaMemset(c.linear_counters, 0, c.linear_counter_count * sizeof(uint32_t)));
    SB_CUDA(cudaMemset(c.attn_counters, 0, kAttnCounterWords * sizeof(uint32_t)));
    SB_CUDA(cudaMemset(c.gdn_counters, 0, kGdnScratchHeads * sizeof(uint32_t)));
  }
  return SB_OK;
}

int sb_alloc(size_t bytes, void **out_dev) {
  SB_NEED_DEVICE();
  SB_REQUIRE(out_dev && bytes, "sb_alloc: null result or zero bytes");
  *out_dev = nullptr;
  SB_CUDA(cudaMalloc(out_dev, bytes));
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  g_allocs[reinterpret_cast<uintptr_t>(*out_dev)] = Allocation{bytes, 1};
  return SB_OK;
}
int sb_view(void *base_dev, size_t offset, size_t bytes, void **out_view) {
  SB_NEED_DEVICE();
  SB_REQUIRE(base_dev && out_view && bytes, "sb_view: null pointer or zero bytes");
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  const uintptr_t from = reinterpret_cast<uintptr_t>(base_dev);
  auto it = owner_of(from);
  SB_REQUIRE(it != g_allocs.end(), "sb_view: %p is not inside a live sb_alloc allocation", base_dev);
  const size_t at = from - it->first;
  SB_REQUIRE(offset <= it->second.bytes - at && bytes <= it->second.bytes - at - offset,
             "sb_view: [%zu, %zu) runs past the allocation's %zu bytes", at + offset, at + offset + bytes, it->second.bytes);
  const uintptr_t view = from + offset;
  ++it->second.holders;
  if (view != it->first) {
    auto &v = g_views[view];
    v.first = it->first;
    ++v.second;
  }
  *out_view = reinterpret_cast<void *>(view);
  return SB_OK;
}
int sb_free(void *dev) {
  SB_NEED_DEVICE();
  if (!dev) return SB_OK;
  uintptr_t base = reinterpret_cast<uintptr_t>(dev);
  {
    std::lock_guard<std::mutex> lock(g_alloc_mutex);
    auto v = g_views.find(base);
    if (v != g_views.end()) {  // a view: its base loses a holder
      const uintptr_t of = v->second.first;
      if (--v->second.second == 0) g_views.erase(v);
      base = of;
    }
    auto it = g_allocs.find(base);
    SB_REQUIRE(it != g_allocs.end(), "sb_free: %p is neither a live allocation nor a live view", dev);
    if (--it->second.holders > 0) return SB_OK;
    g_allocs.erase(it);
  }
  SB_CUDA(cudaFree(reinterpret_cast<void *>(base)));
  return SB_OK;
}
int sb_memset(void *dev, int value, size_t bytes, void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaMemsetAsync(dev, value, bytes, as_stream(stream)));
  return SB_OK;
}
int sb_upload(void *dst_dev, const void *src_host, size_t bytes, void *stream) {
  SB_NEED_DEVICE();
  SB_REQUIRE(dst_dev && src_host, "sb_upload: null pointer");
  SB_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return SB_OK;
}
int sb_download(void *dst_host, const void *src_dev, size_t bytes, void *stream) {
  SB_NEED_DEVICE();
  SB_REQUIRE(dst_host && src_dev, "sb_download: null pointer");
  SB_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return SB_OK;
}
int sb_host_alloc(size_t bytes, void **out_host) {
  SB_NEED_DEVICE();
  SB_REQUIRE(out_host && bytes, "sb_host_alloc: null result or zero bytes");
  SB_CUDA(cudaMallocHost(out_host, bytes));
  return SB_OK;
}
int sb_host_free(void *host) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaFreeHost(host));
  return SB_OK;
}

int sb_stream_create(void **out_stream) {
  SB_NEED_DEVICE();
  cudaStream_t s;
  SB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out_stream = s;
  return SB_OK;
}
int sb_stream_destroy(void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaStreamDestroy(as_stream(stream)));
  return SB_OK;
}
int sb_stream_sync(void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return SB_OK;
}
int sb_event_create(void **out_event) {
  SB_NEED_DEVICE();
  cudaEvent_t e;
  SB_CUDA(cudaEventCreate(&e));
  *out_event = e;
  return SB_OK;
}
int sb_event_destroy(void *event) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return SB_OK;
}
int sb_event_record(void *event, void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
  return SB_OK;
}
int sb_event_sync(void *event) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
  return SB_OK;
}
int sb_event_query(void *event, int *out_done) {
  SB_NEED_DEVICE();
  SB_REQUIRE(event && out_done, "sb_event_query: null pointer");
  const cudaError_t e = cudaEventQuery(reinterpret_cast<cudaEvent_t>(event));
  if (e != cudaSuccess && e != cudaErrorNotReady) return cuda_fail(e, "cudaEventQuery");
  *out_done = e == cudaSuccess;
  return SB_OK;
}
int sb_event_wait_bounded(void *event, uint32_t timeout_ms) {
  SB_NEED_DEVICE();
  SB_REQUIRE(event, "sb_event_wait_bounded: null event");
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (uint32_t polls = 0;; ++polls) {
    const cudaError_t e = cudaEventQuery(reinterpret_cast<cudaEvent_t>(event));
    if (e == cudaSuccess) return SB_OK;
    if (e != cudaErrorNotReady) return cuda_fail(e, "cudaEventQuery");
    if (std::chrono::steady_clock::now() >= deadline) return fail(SB_ERR_BUSY, "sb_event_wait_bounded: not complete after %u ms", timeout_ms);
    if (polls < 64) std::this_thread::yield();
    else std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}
int sb_event_elapsed_ms(void *start, void *stop, float *out_ms) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaEventElapsedTime(out_ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(stop)));
  return SB_OK;
}

int sb_graph_begin(void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal));
  return SB_OK;
}
int sb_graph_end(void *stream, void **out_graph) {
  SB_NEED_DEVICE();
  cudaGraph_t g = nullptr;
  SB_CUDA(cudaStreamEndCapture(as_stream(stream), &g));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
  *out_graph = exec;
  return SB_OK;
}
int sb_graph_launch(void *graph, void *stream) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph), as_stream(stream)));
  return SB_OK;
}
int sb_submit(void *graph, void *stream, uint64_t *out_ticket) {
  SB_NEED_DEVICE();
  SB_REQUIRE(graph && out_ticket, "sb_submit: null graph or ticket");
  std::lock_guard<std::mutex> lock(g_ticket_mutex);
  if (g_ticket_out) return fail(SB_ERR_BUSY, "sb_submit: command %llu is still in flight; consume its ticket first", (unsigned long long)g_ticket_serial);
  if (!g_ticket_event) SB_CUDA(cudaEventCreateWithFlags(&g_ticket_event, cudaEventDisableTiming));
  SB_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph), as_stream(stream)));
  SB_CUDA(cudaEventRecord(g_ticket_event, as_stream(stream)));
  g_ticket_out = true;
  *out_ticket = ++g_ticket_serial;
  return SB_OK;
}
int sb_ticket_wait(uint64_t ticket, uint32_t timeout_ms) {
  SB_NEED_DEVICE();
  {
    std::lock_guard<std::mutex> lock(g_ticket_mutex);
    SB_REQUIRE(g_ticket_out && ticket == g_ticket_serial, "sb_ticket_wait: ticket %llu is not the command in flight", (unsigned long long)ticket);
  }
  const int st = sb_event_wait_bounded(g_ticket_event, timeout_ms);
  if (st != SB_OK) return st;  // still in flight: the ticket stays out
  std::lock_guard<std::mutex> lock(g_ticket_mutex);
  g_ticket_out = false;
  return SB_OK;
}
int sb_graph_destroy(void *graph) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(graph)));
  return SB_OK;
}

uint64_t sb_row_bytes(uint32_t format, uint32_t k) {
  FmtInfo i;
  if (!fmt_info(format, i) || k % i.block_elements) return 0;
  return uint64_t(k / i.block_elements) * i.block_bytes;
}

}  // extern "C"
