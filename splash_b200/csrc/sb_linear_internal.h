// Shared between the two quantized-linear kernels (warp-MMA in sb_linear.cu, tcgen05 in
// sb_linear_tc.cu): the prepared-activation sizes and the host helpers both launchers use.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/splash_b200.h"

namespace sb {

constexpr uint32_t kPrepHeader = 64;    // scale_back[16] floats
constexpr uint32_t kPrepSbBytes = 8704; // 16 tokens x 256 fp16 inputs + 512 bytes of split sub-block sums


// A 2-D map over `rows` rows of `stride` bytes starting at the 16-byte aligned `base`: u32 elements,
// box = box_rows x box_bytes. Rows past the end and bytes past a row read as zero.
int encode_weight_map(CUtensorMap *map, uintptr_t base, uint32_t stride, uint32_t rows, uint32_t box_bytes, uint32_t box_rows);

// The tcgen05 Q4_K kernel: plan for a shape, and launch with prepared activations (UMMA layout).
int tc_plan(uint32_t n, uint32_t k, uint32_t epilogue, SbLinearPlan &plan);
int launch_linear_tc(cudaStream_t stream, const SbLinearArgs *a, const void *prepared, bool pdl);

// ---- the many-row kernel over groups of rows with their own weights (the experts of an MoE block) ----
// groups: device uint4 {expert, first row slot, rows (up to max_rows), rows padded to 16}; group_count: device word. A group's
// inputs are converted into a block of their own (launch_wide_prepare_grouped), its outputs are rows [slot0, slot0 + rows)
// of `out`.
struct WideGroupedArgs {
  const void *weights, *weights2;  // stacked native Q4_K rows [experts][expert_rows][k]; weights2: the up tensor (one-pass gate/up)
  uint32_t experts, expert_rows, k;
  const void *prepared;            // the groups' converted inputs
  const float *scales;             // a scale per row slot
  const uint4 *groups;
  const uint32_t *group_count;
  uint32_t max_groups;             // bounds the grid
  uint32_t max_rows;               // the most rows a group holds (a multiple of 16 up to 128; up to 64: double-buffered sums)
  void *out;                       // bf16 [row slots][out_stride]
  uint32_t out_stride;
  bool pdl;
};
int launch_linear_wide_grouped(cudaStream_t stream, const WideGroupedArgs &a);
// Converts row slot s of every group from row slot_src[s] of x (bf16 [.., x_stride]; ~0: zeros) into the groups' blocks.
struct WidePrepareGroupedArgs {
  const void *x;
  uint32_t x_stride, k;
  const uint32_t *slot_src, *slot_group, *slot_count;
  uint32_t max_slots;  // the grid
  const uint4 *groups;
  void *prepared;
  float *scales;
  bool pdl;
};
int launch_wide_prepare_grouped(cudaStream_t stream, const WidePrepareGroupedArgs &a);

}  // namespace sb
