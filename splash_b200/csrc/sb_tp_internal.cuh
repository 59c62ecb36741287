// Tensor-parallel exchange between the GPUs of one node, shared by the kernels that take part in it
// (prepare_kernel of sb_linear.cu, tp_gather_kernel of sb_tp.cu).
//
// Every rank owns a window of device memory that its peers map (CUDA IPC) and write with plain stores
// over NVLink:
//   inbox   fp32 [2 slots][world][16 rows][width]   slot = exchange number mod 2, one matrix per source rank
//   flags A u32  [world][128]                        per source rank and CTA of the converting kernel
//   flags B u32  [world][kTpGatherCtas]              per source rank and CTA of the gather kernel
//   gather  fp32 [16 rows][gather_width]             a matrix every rank holds whole (the logits)
// An exchange is numbered: epoch = *epoch_base + index + 1, where epoch_base counts the exchanges of the steps
// already completed (advanced by the step's last kernel) and index is the exchange's place in the step. The
// ranks run the same steps, so they agree on the numbers. CTA j of rank s stores its elements into every
// peer's window, then publishes `epoch` in that peer's flag [s][j] (system-scope release); CTA j of the peer
// waits for that flag (system-scope acquire) before it reads what arrived. A CTA owns the same elements on
// every rank, so the hand-shake is between pairs of CTAs and nothing is broadcast.
// Two slots suffice: rank s writes slot e mod 2 again at exchange e + 2, after its exchange e + 1 completed,
// which needed the peer's flags of e + 1, which the peer publishes after its kernel of exchange e (the last
// reader of that slot) has completed.
// Every wait is bounded by the clock: after kTpWaitNs the kernel records SB_DEV_WAIT_EXPIRED in the context's
// status word and carries on with what it has; kernels that find the status word set do not wait at all.
#pragma once
#include <stdint.h>

#include "sb_internal.h"

namespace sb {

constexpr int kTpMaxWorld = 8;
constexpr int kTpConvertCtas = 128;  // grid of the converting kernel: 16 rows x a cluster of 8
constexpr int kTpGatherCtas = 64;
constexpr uint64_t kTpWaitNs = 2000000000ull;  // 2 s

// By value in kernel parameters; world == 0: no exchange.
struct TpExchange {
  uint32_t world, rank, index, width;
  const uint32_t *epoch_base;
  uint32_t *status;
  float *data[kTpMaxWorld];      // rank p's inbox (or gather matrix) as mapped here; data[rank] is this rank's own
  uint32_t *flags[kTpMaxWorld];  // rank p's flag words of the kernel in question
};

// The exchange's parameters for a group (sb_tp_create), `gather` selecting the gather matrix and its flags.
int tp_exchange(void *group, uint32_t index, bool gather, TpExchange &out);
// The group's exchange counter, for the kernel that ends a step to advance.
uint32_t *tp_epoch_word(void *group);

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t tp_epoch(const TpExchange &x) {
  return *reinterpret_cast<const volatile uint32_t *>(x.epoch_base) + x.index + 1u;
}
__device__ __forceinline__ bool tp_healthy(const TpExchange &x) { return *reinterpret_cast<const volatile uint32_t *>(x.status) == SB_DEV_OK; }

// Waits until the flag has reached `epoch`. Gives up after kTpWaitNs (or 2^30 polls, should the clock stand
// still), records the failure and returns false.
__device__ __forceinline__ bool tp_wait_flag(const uint32_t *flag, uint32_t epoch, uint32_t *status) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (int32_t(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((polls & 63u) == 0) {
      if (global_timer_ns() - t0 > kTpWaitNs || polls >= (1u << 30)) {
        atomicCAS(status, uint32_t(SB_DEV_OK), uint32_t(SB_DEV_WAIT_EXPIRED));
        return false;
      }
      __nanosleep(100);
    }
  }
}

// After the CTA's stores into the peers' windows: publishes `epoch` to every peer and waits for every peer's.
// Called by all threads of the CTA; `cta` is the CTA's index in its grid, `ctas` the grid's size.
__device__ __forceinline__ void tp_signal_and_wait(const TpExchange &x, uint32_t epoch, uint32_t cta, uint32_t ctas, bool healthy) {
  __syncthreads();
  const uint32_t t = threadIdx.x;
  if (t < x.world && t != x.rank) {
    __threadfence_system();
    st_release_sys(x.flags[t] + x.rank * ctas + cta, epoch);
    if (healthy) tp_wait_flag(x.flags[x.rank] + t * ctas + cta, epoch, x.status);
  }
  __syncthreads();
}
#endif

}  // namespace sb
