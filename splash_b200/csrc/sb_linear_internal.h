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

}  // namespace sb
