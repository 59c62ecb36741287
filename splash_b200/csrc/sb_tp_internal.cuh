// Tensor-parallel exchange between the GPUs of one node, shared by the kernels that take part in it
// (prepare_kernel of sb_linear.cu, tp_gather_kernel of sb_tp.cu).
//
// Every rank owns a window of device memory that its peers map (CUDA IPC) and write with plain stores
// over NVLink:
//   inbox   [2 slots][world][16 rows][width / 2] units of 16 bytes {value, epoch, value, epoch}
//                                                    slot = exchange number mod 2, one matrix per source rank
//   flags   u32  [world][kTpGatherCtas]              per source rank and CTA of the gather kernel
//   gather  fp32 [16 rows][gather_width]             a matrix every rank holds whole (the logits)
// An exchange is numbered: epoch = *epoch_base + index + 1, where epoch_base counts the exchanges of the steps
// already completed (advanced by the step's last kernel) and index is the exchange's place in the step. The
// ranks run the same steps, so they agree on the numbers.
//
// Shares of a sum take two kernels with the same thread-to-element map on every rank.
//   tp_push_kernel     after the projection that left the k-slices' sums has completed: announces that in this
//                      rank's `ready` word, adds the slices in order and stores the result into every peer's inbox,
//                      as units that carry the exchange's number beside each value.
//   prepare_kernel     (the input conversion) does not wait for the push kernel to complete: it waits for `ready`,
//                      adds the slices itself, and polls its own inbox until every peer's units show the exchange's
//                      number. A unit announces itself (8 bytes arrive whole), so no fence or flag is needed and
//                      the values are usable one trip over NVLink (1.3 us) after they were stored.
// With more than two ranks the shares do not go to everybody (W - 1 copies of 8 bytes a value: 4.6 MB a rank and
// exchange at 8 ranks, 6.5 us of NVLink time) but to the owner of their columns (super-blocks are dealt to the ranks in
// contiguous ranges): the push kernel's threads of owned columns wait for the W - 1 shares, add all W in rank order,
// add the residual, round to bf16 and send the finished values to every rank (themselves included) as units
// {2 x bf16, epoch, 2 x bf16, epoch} in a second inbox [2 slots][16 rows][width / 4]; the conversion then only polls
// that inbox. 0.9 MB a rank and exchange at 8 ranks, two trips over NVLink instead of one.
// Why two kernels: a kernel that has stored into a peer's memory completes only after those stores are flushed
// to the peer, measured at 4.5 us on top of the kernel. That cost now falls on the push kernel, which nothing
// waits for; the conversion, which the next projection waits for, touches local memory only.
//
// Columns of the gather matrix (the gather kernel) land as plain values where their readers expect them, so
// they are announced by flags: CTA j of rank s stores its part into every peer's matrix, then publishes `epoch`
// in that peer's flag [s][j] (system-scope release); CTA j of the peer waits for it (system-scope acquire).
// Two slots suffice: rank s writes slot e mod 2 again at exchange e + 2, after its exchange e + 1 completed,
// which needed the peer's values of e + 1, which the peer sends after its conversion of exchange e (the last
// reader of that slot) has completed.
// Every wait is bounded by the clock: after kTpWaitNs the kernel records SB_DEV_WAIT_EXPIRED in the context's
// status word and carries on with what it has; kernels that find the status word set do not wait at all.
#pragma once
#include <stdint.h>

#include "sb_internal.h"

namespace sb {

constexpr int kTpMaxWorld = 8;
constexpr int kTpGatherCtas = 64;
constexpr uint64_t kTpWaitNs = 2000000000ull;  // 2 s: the default of the context's limit (sb_set_wait_limit_ns)

// By value in kernel parameters; world == 0: no exchange.
struct TpExchange {
  uint32_t world, rank, index, width;
  const uint32_t *epoch_base;
  uint32_t *status;
  uint32_t *ready;               // this rank's word: the number of the last exchange whose slices' sums are complete
  uint32_t two_shot;             // shares go to the columns' owner only, which adds them and sends the sum to everybody
  uint64_t wait_ns;              // how long a wait for a peer may last
  uint4 *sums[kTpMaxWorld];      // rank p's inbox of finished sums (two_shot), as mapped here
  float *data[kTpMaxWorld];      // rank p's inbox (or gather matrix) as mapped here; data[rank] is this rank's own
  uint32_t *flags[kTpMaxWorld];  // rank p's flag words (the gather kernel's)
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
// A unit of the inbox: two values, each beside the exchange's number.
__device__ __forceinline__ void tp_store_unit(uint4 *p, float a, float b, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(epoch), "r"(__float_as_uint(b)), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ uint4 tp_load_unit(const uint4 *p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
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
__device__ __forceinline__ bool tp_wait_flag(const uint32_t *flag, uint32_t epoch, uint32_t *status, uint64_t wait_ns) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (int32_t(ld_relaxed_sys(flag) - epoch) >= 0) {
      (void)ld_acquire_sys(flag);  // one acquire once the flag is there, not one per poll
      return true;
    }
    if ((polls & 63u) == 0) {
      if (global_timer_ns() - t0 > wait_ns || polls >= (1u << 30)) {
        atomicCAS(status, uint32_t(SB_DEV_OK), uint32_t(SB_DEV_WAIT_EXPIRED));
        return false;
      }
      __nanosleep(100);
    }
  }
}

// The conversion's wait for this rank's `ready` word (written by the push kernel on the same GPU).
__device__ __forceinline__ bool tp_wait_ready(const TpExchange &x, uint32_t epoch) {
  const uint64_t t0 = global_timer_ns();
  for (uint32_t polls = 1;; ++polls) {
    if (int32_t(ld_acquire_gpu(x.ready) - epoch) >= 0) return true;
    if ((polls & 63u) == 0 && (global_timer_ns() - t0 > x.wait_ns || polls >= (1u << 30))) {
      atomicCAS(x.status, uint32_t(SB_DEV_OK), uint32_t(SB_DEV_WAIT_EXPIRED));
      return false;
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
    if (healthy) tp_wait_flag(x.flags[x.rank] + t * ctas + cta, epoch, x.status, x.wait_ns);
  }
  __syncthreads();
}
#endif

}  // namespace sb
