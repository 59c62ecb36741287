// Dot products of fp32 weight rows with bf16 activation rows in one fixed order, shared by the fp32 projection
// kernel and by the GDN kernel's fused gate projection so that both produce the same bits.
//
// The order: inputs are cut into chunks of 8; chunk j belongs to lane j % 32 and round j / 32, rounds to group
// round % 8. A group's partial sum is, per lane, a chain of fused multiply-adds over the lane's chunks of that
// group in index order (8 inputs of a chunk in order), then a butterfly over the lanes. The dot product is the 8
// groups' partial sums added in group order. One warp can take all groups (sb_linear_f32), or 8 warps one each.
#pragma once
#include "sb_ptx.cuh"

namespace sb {

constexpr int kDotGroups = 8;

// acc[a][b] = group `group`'s partial sum of x[a] . w[b] (all lanes hold it).
template <int NW, int NX>
__device__ __forceinline__ void warp_dot_group_f32_bf16(const float *const (&w)[NW], const uint16_t *const (&x)[NX], uint32_t k, uint32_t lane,
                                                        uint32_t group, float (&acc)[NX][NW]) {
#pragma unroll
  for (int a = 0; a < NX; ++a)
#pragma unroll
    for (int b = 0; b < NW; ++b) acc[a][b] = 0.0f;
#pragma unroll 1
  for (uint32_t c = 8 * lane + 256 * group; c < k; c += 256 * kDotGroups) {
    float wv[NW][8];
#pragma unroll
    for (int b = 0; b < NW; ++b) {
      const float4 w0 = *reinterpret_cast<const float4 *>(w[b] + c), w1 = *reinterpret_cast<const float4 *>(w[b] + c + 4);
      wv[b][0] = w0.x, wv[b][1] = w0.y, wv[b][2] = w0.z, wv[b][3] = w0.w, wv[b][4] = w1.x, wv[b][5] = w1.y, wv[b][6] = w1.z, wv[b][7] = w1.w;
    }
    uint4 xv[NX];
#pragma unroll
    for (int a = 0; a < NX; ++a) xv[a] = *reinterpret_cast<const uint4 *>(x[a] + c);
#pragma unroll
    for (int a = 0; a < NX; ++a) {
      const uint32_t u[4] = {xv[a].x, xv[a].y, xv[a].z, xv[a].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = bf16_bits_to_float((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xffffu));
#pragma unroll
        for (int b = 0; b < NW; ++b) acc[a][b] = fmaf(v, wv[b][j], acc[a][b]);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < NX; ++a)
#pragma unroll
    for (int b = 0; b < NW; ++b)
#pragma unroll
      for (int o = 16; o; o >>= 1) acc[a][b] += __shfl_xor_sync(0xffffffffu, acc[a][b], o);
}

// The whole dot product by one warp.
__device__ __forceinline__ float warp_dot_f32_bf16(const float *w, const uint16_t *x, uint32_t k, uint32_t lane) {
  const float *const wr[1] = {w};
  const uint16_t *const xr[1] = {x};
  float total = 0.0f;
#pragma unroll
  for (int g = 0; g < kDotGroups; ++g) {
    float p[1][1];
    warp_dot_group_f32_bf16<1, 1>(wr, xr, k, lane, g, p);
    total = g == 0 ? p[0][0] : total + p[0][0];
  }
  return total;
}

}  // namespace sb
