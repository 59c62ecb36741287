// Context, memory, streams, events and graph capture of the C ABI (include/splash_b200.h):
// the part of the reference's MetalBackend the verify step needs (buffers, one command stream,
// completion events; runtime/metal/MetalBackend.hpp:375-547), on the CUDA runtime.
#include <stdarg.h>
#include <string.h>

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
  c.linear_counter_count = 1u << 16;
  SB_CUDA(cudaMalloc(&c.linear_counters, c.linear_counter_count * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.linear_counters, 0, c.linear_counter_count * sizeof(uint32_t)));
  c.attn_workspace_bytes = size_t(32) << 20;
  SB_CUDA(cudaMalloc(&c.attn_workspace, c.attn_workspace_bytes));
  SB_CUDA(cudaMalloc(&c.attn_counters, 128 * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.attn_counters, 0, 128 * sizeof(uint32_t)));
  SB_CUDA(cudaMalloc(&c.gdn_scratch, size_t(256) * 16 * 128 * 2));
  SB_CUDA(cudaMalloc(&c.gdn_counters, 256 * sizeof(uint32_t)));
  SB_CUDA(cudaMemset(c.gdn_counters, 0, 256 * sizeof(uint32_t)));
  c.ready = true;
  return SB_OK;
}

int sb_sm_count(void) { return ctx().ready ? ctx().sm_count : 0; }

int sb_device_status(uint32_t *status) {
  SB_NEED_DEVICE();
  SB_REQUIRE(status, "status is null");
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpy(status, ctx().status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (*status) SB_CUDA(cudaMemset(ctx().status_dev, 0, sizeof(uint32_t)));
  return SB_OK;
}

int sb_alloc(size_t bytes, void **out_dev) {
  SB_NEED_DEVICE();
  SB_REQUIRE(out_dev && bytes, "sb_alloc: null result or zero bytes");
  *out_dev = nullptr;
  SB_CUDA(cudaMalloc(out_dev, bytes));
  return SB_OK;
}
int sb_free(void *dev) {
  SB_NEED_DEVICE();
  SB_CUDA(cudaFree(dev));
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
