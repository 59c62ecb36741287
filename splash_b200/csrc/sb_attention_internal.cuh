// Shared by the two INT8 paged-attention kernels (warp-level MMA in sb_attention.cu, tcgen05 in
// sb_attention_tc.cu): launch parameters, the exact int8 -> fp16 conversion, and the split merge that both
// kernels end with.
#pragma once
#include "sb_internal.h"
#include "sb_ptx.cuh"

namespace sb {

constexpr int kMaxFused = 128;   // rows x query heads of one KV head

struct AttnParams {
  const uint16_t *queries, *qkv;
  const uint32_t *page_table;
  const uint2 *tree;
  uint16_t *out;
  SbKvLayer cache;
  float *partials;     // [kv_head][split][fused][D]
  float *stats;        // [kv_head][split][fused][2]
  uint32_t *counters;  // [kv_head] arrivals, [64 + kv_head] merges done
  uint32_t *status;
  const uint32_t *committed_dev;
  uint32_t rows, q_heads, group, gated, qkv_stride, out_stride, committed, splits, chunks_per_split, fused;
  uint32_t page_table_stride;  // lanes (blockIdx.z): page-table entries between consecutive lanes' tables
};

// Lane blockIdx.z's view of a launch over several lanes: its 16 row slots of the row-indexed buffers, its page table and
// position, its share of the workspace and counters.
__device__ __forceinline__ AttnParams attn_lane_view(AttnParams p) {
  const uint32_t z = blockIdx.z;
  if (z == 0 && gridDim.z == 1) return p;
  const size_t D = p.cache.head_dim;
  p.queries += size_t(16) * z * p.q_heads * D;
  if (p.qkv) p.qkv += size_t(16) * z * p.qkv_stride;
  p.page_table += size_t(z) * p.page_table_stride;
  if (p.tree) p.tree += 16 * z;
  p.out += size_t(16) * z * p.out_stride;
  const size_t per_lane = size_t(p.cache.kv_heads) * p.splits * kMaxFused;
  p.partials += size_t(z) * per_lane * D;
  p.stats += size_t(z) * per_lane * 2;
  p.counters += 128 * z;
  if (p.committed_dev) p.committed_dev += z;
  return p;
}

// 16 int8 (one uint4) -> 16 fp16, exactly: (q ^ 0x80) | 0x6400 is 1024 + q + 128.
__device__ __forceinline__ void int8x16_to_half(const uint4 v, uint4 &lo, uint4 &hi) {
  const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = hsub2_u32(__byte_perm(w[i], 0x64646464u, 0x4140), 0x64806480u);      // bytes 0, 1
    o[2 * i + 1] = hsub2_u32(__byte_perm(w[i], 0x64646464u, 0x4342), 0x64806480u);  // bytes 2, 3
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// The end of both kernels, called by every thread of the CTA after its split's partials (fp32 O rows and
// (max, sum) in log2 units) are stored. Every split of this KV head publishes its partials, then all of the
// head's CTAs (co-resident: the launch is cooperative and the grid has at most one CTA per SM) share the
// merge: CTA `split` merges fused rows split, split + splits, ... in split order with weights
// exp2(max_s - max), divides, rounds to bf16 and multiplies by sigmoid(gate)
// (runtime/metal/kernels/common/paged_attention_tile.h:498-535, attention_gate.h:19-45). The wait for the
// other splits is bounded: if they never arrive the kernel sets the status word and leaves.
template <int D>
__device__ __forceinline__ void attention_merge(const AttnParams &p, uint32_t split, uint32_t kvh, uint32_t *s_last) {
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  const uint32_t F = p.fused, G = p.group;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    atomicAdd(&p.counters[kvh], 1u);
    uint32_t spins = 0;
    while (atomicAdd(&p.counters[kvh], 0u) < p.splits && ++spins < (1u << 22)) __nanosleep(100);
    *s_last = spins < (1u << 22);
    if (!*s_last) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  // A warp per (fused row, 128 dimensions): lane -> dimensions 128 part + 4 lane .. + 3, one 16-byte load a split, 16
  // splits' loads in flight; the CTA's few rows so spread over all its warps. Every element is summed in split order.
  constexpr uint32_t kParts = D / 128;
  static_assert(D % 128 == 0, "merge tasks take 128 dimensions");
  const uint32_t my_rows = split < F ? (F - split + p.splits - 1) / p.splits : 0;
  for (uint32_t task = warp; task < my_rows * kParts; task += warps) {
    const uint32_t f = split + (task / kParts) * p.splits, d0 = 128 * (task % kParts) + 4 * lane;
    const float *stats = p.stats + (size_t(kvh) * p.splits * kMaxFused + f) * 2;
    const float *parts = p.partials + (size_t(kvh) * p.splits * kMaxFused + f) * D + d0;
    const size_t sstride = size_t(kMaxFused) * 2, pstride = size_t(kMaxFused) * D;
    float mall = -INFINITY;
    for (uint32_t s = lane; s < p.splits; s += 32) mall = fmaxf(mall, __ldcg(stats + s * sstride));
#pragma unroll
    for (int o = 16; o; o >>= 1) mall = fmaxf(mall, __shfl_xor_sync(0xffffffffu, mall, o));
    float num[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float den = 0.0f;
    for (uint32_t s0 = 0; s0 < p.splits; s0 += 16) {
      float ms[16], ls[16];
      float4 v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t s = min(s0 + j, p.splits - 1);
        ms[j] = __ldcg(stats + s * sstride);
        ls[j] = __ldcg(stats + s * sstride + 1);
        v[j] = __ldcg(reinterpret_cast<const float4 *>(parts + s * pstride));
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (s0 + j >= p.splits || ms[j] == -INFINITY) continue;
        const float w = exp2f(ms[j] - mall);
        num[0] += w * v[j].x, num[1] += w * v[j].y, num[2] += w * v[j].z, num[3] += w * v[j].w;
        den += w * ls[j];
      }
    }
    const uint32_t row = f / G, qh = kvh * G + f % G;
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = round_bf16(den > 0.0f ? num[i] / den : 0.0f);
    if (p.gated) {
      const uint2 g2 = *reinterpret_cast<const uint2 *>(p.qkv + size_t(row) * p.qkv_stride + qh * 2 * D + D + d0);
      o[0] *= sigmoid_f(bf16_bits_to_float(g2.x & 0xffffu)), o[1] *= sigmoid_f(bf16_bits_to_float(g2.x >> 16));
      o[2] *= sigmoid_f(bf16_bits_to_float(g2.y & 0xffffu)), o[3] *= sigmoid_f(bf16_bits_to_float(g2.y >> 16));
    }
    uint2 packed;
    packed.x = uint32_t(float_to_bf16_bits(o[0])) | (uint32_t(float_to_bf16_bits(o[1])) << 16);
    packed.y = uint32_t(float_to_bf16_bits(o[2])) | (uint32_t(float_to_bf16_bits(o[3])) << 16);
    *reinterpret_cast<uint2 *>(p.out + size_t(row) * p.out_stride + qh * D + d0) = packed;
  }
  // The last CTA to finish its share returns both counters to zero for the next launch.
  __syncthreads();
  if (tid == 0 && atomicAdd(&p.counters[64 + kvh], 1u) == p.splits - 1) {
    p.counters[kvh] = 0;
    p.counters[64 + kvh] = 0;
  }
}

// The tcgen05 kernel's launcher (sb_attention_tc.cu); `p` comes filled except for the split geometry.
int launch_attention_tc(cudaStream_t stream, AttnParams &p, uint32_t visible, uint32_t lanes);

}  // namespace sb
