// Internal declarations shared by the translation units of libsplash_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/splash_b200.h"

namespace sb {

struct Context {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  uint32_t *status_dev = nullptr;        // device status word: 0 healthy, else SB_DEV_* of the first failure
  float *linear_partials = nullptr;      // split-K partials [slice][16][columns]
  uint32_t *linear_counters = nullptr;   // one arrival counter per tile, zero between launches
  size_t linear_partials_bytes = 0;
  uint8_t *prepared = nullptr;           // sb_linear's own prepared-input scratch
  size_t prepared_bytes = 0;
  uint32_t linear_counter_count = 0;
  uint8_t *wide_prepared = nullptr;      // sb_linear_wide's own converted-input scratch (up to 512 rows of k up to 18432)
  size_t wide_prepared_bytes = 0;
  float *attn_workspace = nullptr;       // split partials and (max, sum) of sb_attn_verify
  size_t attn_workspace_bytes = 0;
  uint32_t *attn_counters = nullptr;     // one arrival counter per KV head, zero between launches
  uint16_t *gdn_scratch = nullptr;       // recurrent outputs before the gate [value_heads][16][128]
  uint32_t *gdn_counters = nullptr;      // one arrival counter per value head
  bool pdl = true;                       // launch glue kernels with programmatic stream serialization
  int tp_exchange_shots = 0;             // 0: by the number of ranks, 1: one shot, 2: two shots (sb_tp_set_exchange)
  uint64_t wait_ns = 2000000000ull;      // how long a kernel waits for a peer GPU before it gives up (sb_set_wait_limit_ns)
  int attention_kernel = 0;              // 0: tcgen05 kernel, 1: warp-level MMA kernel (sb_set_attention_kernel)
};
Context &ctx();

int fail(int status, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define SB_CUDA(call)                                          \
  do {                                                         \
    cudaError_t e_ = (call);                                   \
    if (e_ != cudaSuccess) return ::sb::cuda_fail(e_, #call);  \
  } while (0)

#define SB_REQUIRE(cond, ...)                                        \
  do {                                                               \
    if (!(cond)) return ::sb::fail(SB_ERR_INVALID, __VA_ARGS__);     \
  } while (0)

#define SB_NEED_DEVICE()                                                                   \
  do {                                                                                     \
    if (!::sb::ctx().ready) return ::sb::fail(SB_ERR_NO_DEVICE, "sb_init has not succeeded: no CUDA device"); \
  } while (0)

constexpr uint32_t kAttnCounterWords = 64 * 128;  // 128 arrival / merge counters per lane, up to 64 lanes
constexpr uint32_t kGdnScratchHeads = 2048;       // value heads x lanes of one sb_gdn_verify launch

// Device status word values.
enum : uint32_t {
  SB_DEV_OK = 0,
  SB_DEV_WAIT_EXPIRED = 1,  // a bounded mbarrier / flag wait gave up
  SB_DEV_CONTRACT = 2       // a kernel met arguments outside its contract and returned early
};

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

struct FmtInfo {
  uint32_t block_elements, block_bytes;
};
inline bool fmt_info(uint32_t f, FmtInfo &i) {
  switch (f) {
    case SB_FMT_Q4K: i = {256, 144}; return true;
    case SB_FMT_Q6K: i = {256, 210}; return true;
    case SB_FMT_Q80: i = {32, 34}; return true;
    case SB_FMT_NVFP4: i = {256, 148}; return true;
    case SB_FMT_BF16: case SB_FMT_F16: i = {1, 2}; return true;
    case SB_FMT_F32: i = {1, 4}; return true;
  }
  return false;
}

}  // namespace sb
