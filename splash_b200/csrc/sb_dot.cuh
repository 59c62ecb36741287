// Dot products of fp32 weight rows with bf16 activation rows in one fixed order, shared by the fp32 projection
// kernel and by the GDN kernel's fused gate projection so that both produce the same bits: lane l adds
// inputs 8 l + 256 i .. + 7 in index order with fused multiply-adds, then the lanes' sums meet in a butterfly.
#pragma once
#include "sb_ptx.cuh"

namespace sb {

template <int NW, int NX>
__device__ __forceinline__ void warp_dots_f32_bf16(const float *const (&w)[NW], const uint16_t *const (&x)[NX], uint32_t k, uint32_t lane,
                                                   float (&acc)[NX][NW]) {
#pragma unroll
  for (int a = 0; a < NX; ++a)
#pragma unroll
    for (int b = 0; b < NW; ++b) acc[a][b] = 0.0f;
#pragma unroll 5
  for (uint32_t c = 8 * lane; c < k; c += 256) {
    float wv[NW][8];
#pragma unroll
    for (int b = 0; b < NW; ++b) {
      const float4 w0 = *reinterpret_cast<const float4 *>(w[b] + c), w1 = *reinterpret_cast<const float4 *>(w[b] + c + 4);
      wv[b][0] = w0.x, wv[b][1] = w0.y, wv[b][2] = w0.z, wv[b][3] = w0.w, wv[b][4] = w1.x, wv[b][5] = w1.y, wv[b][6] = w1.z, wv[b][7] = w1.w;
    }
#pragma unroll
    for (int a = 0; a < NX; ++a) {
      const uint4 v = *reinterpret_cast<const uint4 *>(x[a] + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xv = bf16_bits_to_float((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xffffu));
#pragma unroll
        for (int b = 0; b < NW; ++b) acc[a][b] = fmaf(xv, wv[b][j], acc[a][b]);
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

}  // namespace sb
