// Quantized linear for many rows (17 .. 128 per pass; more rows run as passes of 128): Y[M,N] = X[M,K] W[N,K]^T with the
// weights dequantized in registers to fp16 and multiplied on the tcgen05 tensor cores, A operand and accumulators in
// tensor memory.
//
// Takes the place of the reference's many-row projection tile (the 128-row prefill entry points gguf_prefill_<fmt>_{a,r,g}
// of runtime/metal/kernels/shared/gguf_linear.metal with the geometry of runtime/metal/abi/Gguf.h:31-35, and the 64-row
// decode tiles of runtime/ops/Linear.hpp:94-97). Its arithmetic is that tile's: the weight is rounded to half once it is
// dequantized (the staged tile, runtime/metal/kernels/common/gguf_staged.h:11-57), products and sums run in fp32, one
// rounding to the destination after the epilogue (runtime/metal/kernels/common/gguf_tile.h:8-14). Here the half weight of
// Q4_K is fl16(q * fl16(d sc) + fl16(-dmin mn)): the two floating factors are rounded to half before the one fused
// multiply-add, which keeps the expansion at three instructions per two weights; the projection stays inside the
// reference's bound for half-rounded weights with room to spare (tests/test_linear_wide_gpu.py states the bound used).
//
//   item      256 weight rows (two 128-row halves, or 128 gate rows and the 128 up rows of the same columns; one half where
//             whole items would leave SMs idle) x all of K x one pass of up to 128 rows of X; persistent CTAs walk the items
//   weights   tiled TMA: one box of 128 rows x 144 bytes per (half, super-block) into a ring of four; never re-read
//   X         converted once by wide_prepare_kernel to fp16 with a per-row power-of-two scale, laid out as the K-major
//             core matrices the MMA reads (8 rows x 16 bytes), and streamed super-block by super-block from the L2 into a
//             second ring (128 KB) by a warp of its own
//   dequant   16 warps: warp (half of the item, inputs' half h, quadrant q) expands sub-blocks 4h .. 4h+3 of rows
//             32q .. 32q+31 (a thread owns a row) and writes the 128 halves with tcgen05.st into its A buffer of tensor
//             memory (64 columns; four buffers, one per (half of the item, inputs' half))
//   mma       two threads in two warps, one per half of the item, each with its own accumulator (128 lanes x N fp32
//             columns), so the order of a sum is fixed. Measured here: one thread issues a tcgen05.mma of this shape every
//             100 to 125 cycles whatever N <= 128 is, two threads together one per 62 to 70, four one per 31 to 36; the
//             tensor pipe needs 64 at N = 128. Per A buffer 8 MMAs (M 128, N = rows rounded up to 16, K 16), A from tensor
//             memory, B from the X ring; tcgen05.commit frees the A buffer, the X group and, after the item's last step,
//             hands the accumulators to the epilogue
//   epilogue  4 warps, a thread per weight row: tcgen05.ld 16 columns at a time, scale back, the epilogue on all 16
//             without a branch, then the stores
// Every wait is bounded and reports through the status word; tensor memory is always returned.
#include <algorithm>

#include <cuda.h>

#include "sb_internal.h"
#include "sb_linear_internal.h"
#include "sb_ptx.cuh"
#include "sb_tcgen05.cuh"

namespace sb {

constexpr uint32_t kWideMaxRows = 128;             // rows of X one pass multiplies (the accumulators' columns)
constexpr uint32_t kWideHeader = 1024;             // scale_back[256] floats (a pass reads its 128)
constexpr uint32_t kWideDequantWarps = 16, kWideEpilogueWarps = 4;  // dequant: (half of the item, inputs' half, quadrant)
constexpr uint32_t kWideRawWarp = kWideDequantWarps + kWideEpilogueWarps, kWideXWarp = kWideRawWarp + 1, kWideMmaWarp0 = kWideXWarp + 1;
constexpr uint32_t kWideThreads = 32 * (kWideMmaWarp0 + 2);  // 768
// A super-block of a weight row as the kernel reads it, and the ring of 128-row stages it fits in shared memory.
//   Q4_K   the native 144 bytes (4 stages of 18 KB)
//   Q6_K   the image of sb_linear_wide_image, 224 bytes: low nibbles paired as Q4_K pairs them, the two high bits in a plane
//          of their own, the sixteen scales as halves d * sc / row scale (3 stages of 28 KB)
//   NVFP4  the image, 160 bytes: the nibbles in expansion order, the sixteen scales as halves e4m3 * g * 2^14 / row scale
//          (4 stages of 20 KB)
//   Q8_0   the image, 272 bytes for eight blocks of 32: the codes + 128 as bytes, the eight scales as halves d / row scale
//          (2 stages of 34 KB: a stream of the item has one stage to itself)
template <uint32_t FMT> struct WideFmt;
template <> struct WideFmt<SB_FMT_Q4K> { static constexpr uint32_t kSb = 144, kStages = 4; };
template <> struct WideFmt<SB_FMT_Q6K> { static constexpr uint32_t kSb = 224, kStages = 3; };
template <> struct WideFmt<SB_FMT_NVFP4> { static constexpr uint32_t kSb = 160, kStages = 4; };
template <> struct WideFmt<SB_FMT_Q80> { static constexpr uint32_t kSb = 272, kStages = 2; };
constexpr uint32_t kWideMaxRawStages = 4;
constexpr uint32_t kWideXBytes = 128 * 1024, kWideMaxXStages = 8;   // the X ring; a stage holds 64 inputs of every row
constexpr uint32_t kWideABufs = 4, kWideACols = 64, kWideACol0 = 256, kWideDCols = 128, kWideTmemCols = 512;
constexpr uint32_t kWideBarBytes = 3072;           // barriers, tensor-memory slot, scale_back[128] at 512, then an epilogue warp's own [128] x 4
constexpr uint32_t kWideXOff = kWideBarBytes, kWideRawOff = kWideXOff + kWideXBytes;
template <uint32_t FMT> constexpr uint32_t wide_smem() { return kWideRawOff + WideFmt<FMT>::kStages * 128 * WideFmt<FMT>::kSb; }  // 205,824 bytes for Q4_K

struct WideParams {
  const uint8_t *prepared;  // header + units of 64 inputs: [k-step 4][row / 8][input / 8 (2)][row % 8][8 halves]
  const uint16_t *aux;
  void *out;
  uint32_t *status;
  uint32_t n, rows, rows_padded, aux_stride, out_stride, epilogue, out_f32;
  uint32_t nsb, items, x_groups, x_stage_bytes, gate_up;
  uint32_t halves;  // 128-row halves per item: 2, or 1 when whole items would leave SMs idle  // x_groups: super-blocks of X the ring holds
  // Split K (SB_EPILOGUE_PARTIALS): an item is (tile, split), items = tiles x splits; a split's sums over its range of
  // super-blocks go to out as fp32 [split][rows_total][out_stride], for the next input conversion to add in split order.
  uint32_t splits, rows_total, row0;
  const float *row_scale[2];  // images: a power of two per weight row taken out of its scales (NULL for native Q4_K rows)
  // Grouped (the experts of an MoE block): the launch's items are (group, tile) pairs over a device table of groups, each
  // group the rows routed to one expert (up to 128 of them, padded to 16), its inputs a block of `prepared` of its own at
  // row slot `slot0`, its weights the expert's rows of the stacked tensor, its outputs rows slot0 .. of `out`.
  const uint4 *groups;         // {expert, slot0, rows, rows padded to 16}
  const uint32_t *group_count;
  const float *group_scales;   // scale_back of every row slot
  uint32_t tiles_per_group, expert_rows;  // weight rows per expert in the stacked tensor
  // Up to 64 rows of X in every item: the accumulators are double-buffered inside their 128 columns (an item's sums at
  // columns 64 (i & 1) .., i the CTA's count of items), so the epilogue of an item overlaps the next item's MMAs.
  uint32_t dbuf;
};
// An item's tile, its range of super-blocks, its rows of X and where its weights, inputs and outputs are.
struct WideItem {
  uint32_t tile, split, sb0, sb1;
  uint32_t rows, rows_padded, slot0, wrow0;
  const uint8_t *x;  // the item's converted inputs: super-block sb at x + sb * 512 * rows_padded
};
__device__ __forceinline__ uint32_t wide_items(const WideParams &p) { return p.groups ? __ldg(p.group_count) * p.tiles_per_group : p.items; }
__device__ __forceinline__ WideItem wide_item(const WideParams &p, uint32_t item) {
  WideItem w;
  if (p.groups) {
    const uint32_t g = item / p.tiles_per_group;
    const uint4 rec = __ldg(p.groups + g);
    w.tile = item - g * p.tiles_per_group, w.split = 0, w.sb0 = 0, w.sb1 = p.nsb;
    w.rows = rec.z, w.rows_padded = rec.w, w.slot0 = rec.y, w.wrow0 = rec.x * p.expert_rows;
    w.x = p.prepared + size_t(rec.y) * p.nsb * 512;
    return w;
  }
  w.tile = item / p.splits, w.split = item - w.tile * p.splits;
  w.sb0 = w.split * p.nsb / p.splits, w.sb1 = (w.split + 1) * p.nsb / p.splits;
  w.rows = p.rows, w.rows_padded = p.rows_padded, w.slot0 = 0, w.wrow0 = 0;
  w.x = p.prepared + kWideHeader;
  return w;
}
#ifdef SB_DIAG
// Cycle counters of the roles of CTA 0 (diagnostic builds only): [role][what], read back through sb_linear_wide_timing.
__device__ unsigned long long g_wide_timing[8][8];
#define WIDE_T0() const long long t_begin_ = clock64()
#define WIDE_TADD(role, what) do { wt_[what] += (unsigned long long)(clock64() - t_begin_); wt_role_ = role; } while (0)
#define WIDE_EVENT(i) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) g_wide_timing[7][i] = (unsigned long long)(clock64() - t_kernel_); } while (0)
#define WIDE_KERNEL_T0() const long long t_kernel_ = clock64(); unsigned long long wt_[4] = {0, 0, 0, 0}; int wt_role_ = -1
#define WIDE_FLUSH() do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && wt_role_ >= 0) for (int i_ = 0; i_ < 4; ++i_) g_wide_timing[wt_role_][i_] = wt_[i_]; } while (0)
#else
#define WIDE_FLUSH() do {} while (0)
#define WIDE_T0() do {} while (0)
#define WIDE_TADD(role, what) do {} while (0)
#define WIDE_EVENT(i) do {} while (0)
#define WIDE_KERNEL_T0() do {} while (0)
#endif
struct WideMaps {
  CUtensorMap m[2];  // the item's first half (or gate rows), its second half (or up rows)
};

__device__ __forceinline__ void wide_expired(uint32_t *status, uint32_t site) {
  atomicCAS(status, 0u, uint32_t(SB_DEV_WAIT_EXPIRED) | (site << 8));
}
__device__ __forceinline__ bool wide_warp_wait(uint64_t *bar, uint32_t parity, bool backoff = false) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = backoff ? mbar_wait_backoff(bar, parity) : mbar_wait(bar, parity);
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- the conversion of X ----
// One CTA per row slot (rows past `rows` are written as zeros): optional RMSNorm, the row's largest magnitude, a
// power-of-two scale that keeps the values below 2^10, fp16, stored in the MMA's core-matrix order. Within every four
// consecutive inputs the order is [0, 2, 1, 3]: the order in which the weight expansion produces its halves.
constexpr int kWidePrepThreads = 256;
struct WidePrepParams {
  const uint16_t *x;
  const float *norm_w;
  uint8_t *out;
  uint32_t rows, rows_padded, k, x_stride;
  // With `partials`: x = bf16(residual + the splits' sums added in split order), written to x (the new hidden rows) first.
  const float *partials;  // fp32 [splits][rows_total][partial_stride], this pass's first row at row0
  const uint16_t *residual;
  uint32_t splits, rows_total, row0, partial_stride, residual_stride;
  // Grouped (an MoE block's routed rows; wide_prepare_slots_kernel): slot_src[s] is the row of x that row slot s of the
  // groups' blocks holds (~0: a padding slot, zeros), slot_group[s] = group << 8 | its row inside the group, groups as
  // WideParams has them; the blocks start at out (a group's at slot0 * k * 2), the slots' scales go to `scales`.
  const uint32_t *slot_src, *slot_group, *slot_count;
  const uint4 *groups;
  float *scales;
  uint16_t *normed_out;  // optional bf16 [rows][k]: the normalised rows (with norm_w), for the fp32 side projections of the same input
};
__global__ void __launch_bounds__(kWidePrepThreads) wide_prepare_kernel(const WidePrepParams p) {
  __shared__ float red_s[2 * (kWidePrepThreads / 32)];
  const uint32_t tok = blockIdx.x, tid = threadIdx.x;  // the row slot inside its block
  pdl_launch_dependents();
  pdl_wait();
  const bool live = tok < p.rows;
  const uint32_t rows_padded = p.rows_padded;
  const uint16_t *xrow = p.x + size_t(tok) * p.x_stride;
  uint8_t *block = p.out + kWideHeader;
  float *scale_dst = reinterpret_cast<float *>(p.out) + tok;
  const uint32_t chunks = p.k / 8;  // 8 inputs each
  // A thread's chunks (tid, tid + 256, ...) stay in its registers from the pass that forms or first reads them to the
  // conversion (up to kKeep of them: k <= 18432); a longer row is read again from memory, where this thread wrote it.
  constexpr int kKeep = 9;
  uint4 keep[kKeep];
  const bool kept = chunks <= uint32_t(kKeep) * kWidePrepThreads;
  if (p.partials && live) {
    // The projection ahead left its k-splits' sums: add them in split order onto the residual, round once, and keep the
    // rows (the new hidden state).
    uint16_t *xw = const_cast<uint16_t *>(xrow);
    auto sum_chunk = [&](uint32_t c) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(p.residual + size_t(tok) * p.residual_stride + 8 * c);
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (uint32_t sp = 0; sp < p.splits; ++sp) {
        const float4 *src = reinterpret_cast<const float4 *>(p.partials + (size_t(sp) * p.rows_total + p.row0 + tok) * p.partial_stride + 8 * c);
        const float4 a = __ldcg(src), b = __ldcg(src + 1);
        acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w, acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t lo = float_to_bf16_bits(acc[2 * j] + bf16_bits_to_float(u[j] & 0xffffu));
        const uint32_t hi = float_to_bf16_bits(acc[2 * j + 1] + bf16_bits_to_float(u[j] >> 16));
        o[j] = lo | (hi << 16);
      }
      const uint4 out = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4 *>(xw + 8 * c) = out;
      return out;
    };
    if (kept) {
#pragma unroll
      for (int i = 0; i < kKeep; ++i) {
        const uint32_t c = tid + uint32_t(i) * kWidePrepThreads;
        if (c < chunks) keep[i] = sum_chunk(c);
      }
    } else {
      for (uint32_t c = tid; c < chunks; c += kWidePrepThreads) (void)sum_chunk(c);
    }
  } else if (kept && live) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const uint32_t c = tid + uint32_t(i) * kWidePrepThreads;
      if (c < chunks) keep[i] = *reinterpret_cast<const uint4 *>(xrow + 8 * c);
    }
  }
  float ss = 0.0f, mx = 0.0f;
  auto measure = [&](uint32_t c, const uint4 raw) {
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = bf16_bits_to_float(u[j] & 0xffffu), b = bf16_bits_to_float(u[j] >> 16);
      ss = fmaf(a, a, ss), ss = fmaf(b, b, ss);
      const float wa = p.norm_w ? p.norm_w[8 * c + 2 * j] : 1.0f, wb = p.norm_w ? p.norm_w[8 * c + 2 * j + 1] : 1.0f;
      mx = fmaxf(mx, fmaxf(fabsf(a * wa), fabsf(b * wb)));
    }
  };
  if (kept) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const uint32_t c = tid + uint32_t(i) * kWidePrepThreads;
      if (c < chunks && live) measure(c, keep[i]);
    }
  } else {
    for (uint32_t c = tid; c < chunks && live; c += kWidePrepThreads) measure(c, *reinterpret_cast<const uint4 *>(xrow + 8 * c));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((tid & 31) == 0) red_s[2 * (tid >> 5)] = ss, red_s[2 * (tid >> 5) + 1] = mx;
  __syncthreads();
  ss = red_s[0], mx = red_s[1];
  for (int w = 1; w < kWidePrepThreads / 32; ++w) ss += red_s[2 * w], mx = fmaxf(mx, red_s[2 * w + 1]);
  float inv = 1.0f;
  if (p.norm_w) {
    inv = rsqrtf(ss / float(p.k) + 1e-6f);
    mx = mx * inv * 1.0625f;  // (x inv) w against x w inv and the rounding to bf16: well inside 6 %
  }
  int e = 0;
  if (mx > 0.0f && mx <= 3.0e38f) {
    (void)frexpf(mx, &e);
    e -= 10;
  }
  const float down = ldexpf(1.0f, -e);
  if (tid == 0) *scale_dst = live ? ldexpf(1.0f, e) : 0.0f;
  const size_t unit_bytes = size_t(rows_padded) * 128;  // 64 inputs of every row slot
  auto convert = [&](uint32_t c, const uint4 raw) {
    uint32_t h[4] = {0, 0, 0, 0};
    if (live) {
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
      float v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[2 * j] = bf16_bits_to_float(u[j] & 0xffffu), v[2 * j + 1] = bf16_bits_to_float(u[j] >> 16);
      if (p.norm_w) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = round_bf16((v[j] * inv) * p.norm_w[8 * c + j]);
        if (p.normed_out) {
          uint32_t n[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) n[j] = float_to_bf16_bits(v[2 * j]) | (float_to_bf16_bits(v[2 * j + 1]) << 16);
          *reinterpret_cast<uint4 *>(p.normed_out + size_t(tok) * p.k + 8 * c) = make_uint4(n[0], n[1], n[2], n[3]);
        }
      }
      __half hv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(v[j] * down);
      const __half2 p0 = __halves2half2(hv[0], hv[2]), p1 = __halves2half2(hv[1], hv[3]);
      const __half2 p2 = __halves2half2(hv[4], hv[6]), p3 = __halves2half2(hv[5], hv[7]);
      h[0] = *reinterpret_cast<const uint32_t *>(&p0), h[1] = *reinterpret_cast<const uint32_t *>(&p1);
      h[2] = *reinterpret_cast<const uint32_t *>(&p2), h[3] = *reinterpret_cast<const uint32_t *>(&p3);
    }
    const uint32_t k0 = 8 * c, unit = k0 / 64, step = (k0 % 64) / 16, half = (k0 % 16) / 8;
    uint8_t *dst = block + unit * unit_bytes + size_t(step) * rows_padded * 32 + (tok >> 3) * 256 + half * 128 + (tok & 7) * 16;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
  };
  if (kept) {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const uint32_t c = tid + uint32_t(i) * kWidePrepThreads;
      if (c < chunks) convert(c, live ? keep[i] : make_uint4(0, 0, 0, 0));
    }
  } else {
    for (uint32_t c = tid; c < chunks; c += kWidePrepThreads) convert(c, live ? *reinterpret_cast<const uint4 *>(xrow + 8 * c) : make_uint4(0, 0, 0, 0));
  }
}

// The conversion of the groups' row slots with a warp per slot (no norm, no sums to add): a slot's table look-ups and its row
// are a short chain, so many slots a CTA and few CTAs beat a CTA per slot (an MoE block's 6700 slots were 27 us as a CTA each).
constexpr int kWideSlotWarps = 8;
__global__ void __launch_bounds__(32 * kWideSlotWarps) wide_prepare_slots_kernel(const WidePrepParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t slot = blockIdx.x * kWideSlotWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (slot >= __ldg(p.slot_count)) return;
  const uint32_t src = __ldg(p.slot_src + slot), sg = __ldg(p.slot_group + slot);
  const uint4 rec = __ldg(p.groups + (sg >> 8));
  const bool live = src != 0xffffffffu;
  const uint32_t tok = sg & 0xffu, rows_padded = rec.w, chunks = p.k / 8;
  const uint16_t *xrow = p.x + size_t(live ? src : 0) * p.x_stride;
  uint8_t *block = p.out + size_t(rec.y) * p.k * 2;
  float mx = 0.0f;
  for (uint32_t c = lane; c < chunks && live; c += 32) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(xrow + 8 * c);
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) mx = fmaxf(mx, fmaxf(fabsf(bf16_bits_to_float(u[j] & 0xffffu)), fabsf(bf16_bits_to_float(u[j] >> 16))));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  int e = 0;
  if (mx > 0.0f && mx <= 3.0e38f) {
    (void)frexpf(mx, &e);
    e -= 10;
  }
  const float down = ldexpf(1.0f, -e);
  if (lane == 0) p.scales[slot] = live ? ldexpf(1.0f, e) : 0.0f;
  const size_t unit_bytes = size_t(rows_padded) * 128;
  for (uint32_t c = lane; c < chunks; c += 32) {
    uint32_t h[4] = {0, 0, 0, 0};
    if (live) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(xrow + 8 * c);
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
      __half hv[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hv[2 * j] = __float2half_rn(bf16_bits_to_float(u[j] & 0xffffu) * down);
        hv[2 * j + 1] = __float2half_rn(bf16_bits_to_float(u[j] >> 16) * down);
      }
      const __half2 p0 = __halves2half2(hv[0], hv[2]), p1 = __halves2half2(hv[1], hv[3]);
      const __half2 p2 = __halves2half2(hv[4], hv[6]), p3 = __halves2half2(hv[5], hv[7]);
      h[0] = *reinterpret_cast<const uint32_t *>(&p0), h[1] = *reinterpret_cast<const uint32_t *>(&p1);
      h[2] = *reinterpret_cast<const uint32_t *>(&p2), h[3] = *reinterpret_cast<const uint32_t *>(&p3);
    }
    const uint32_t k0 = 8 * c, unit = k0 / 64, step = (k0 % 64) / 16, half = (k0 % 16) / 8;
    uint8_t *dst = block + unit * unit_bytes + size_t(step) * rows_padded * 32 + (tok >> 3) * 256 + half * 128 + (tok & 7) * 16;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
  }
}

// The four sub-blocks 4h .. 4h+3 of a Q4_K row's super-block as 128 halves in 64 packed columns:
// fl16(q * fl16(d sc) + fl16(-dmin mn)); a high nibble enters as 16 q against fl16(d sc / 16).
__device__ __forceinline__ void wide_expand_q4k(const uint8_t *row, uint32_t h, uint32_t (&r)[64]) {
  const uint4 hdr = *reinterpret_cast<const uint4 *>(row);
  const __half2 dd = *reinterpret_cast<const __half2 *>(&hdr.x);
  const float d = __low2float(dd), ndmin = -__high2float(dd);
  // 6-bit scales and mins of sub-blocks 0..3 (h = 0) or 4..7 (h = 1) as bytes
  const uint32_t sc4 = h ? ((hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u)) : (hdr.y & 0x3f3f3f3fu);
  const uint32_t mn4 = h ? (((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u)) : (hdr.z & 0x3f3f3f3fu);
  const uint32_t k1024 = 0x64006400u;
#pragma unroll
  for (uint32_t pr = 0; pr < 2; ++pr) {  // pair pr of this half: sub-blocks 2 pr (low nibbles) and 2 pr + 1 (high nibbles)
    const float sc0 = float((sc4 >> (16 * pr)) & 0xffu), sc1 = float((sc4 >> (16 * pr + 8)) & 0xffu);
    const float mn0 = float((mn4 >> (16 * pr)) & 0xffu), mn1 = float((mn4 >> (16 * pr + 8)) & 0xffu);
    const __half2 a0 = __float2half2_rn(d * sc0), a1 = __float2half2_rn(d * sc1 * 0.0625f);
    const __half2 b0 = __float2half2_rn(ndmin * mn0), b1 = __float2half2_rn(ndmin * mn1);
    const uint32_t ua0 = *reinterpret_cast<const uint32_t *>(&a0), ua1 = *reinterpret_cast<const uint32_t *>(&a1);
    const uint32_t ub0 = *reinterpret_cast<const uint32_t *>(&b0), ub1 = *reinterpret_cast<const uint32_t *>(&b1);
    const uint8_t *qs = row + 16 + 32 * (2 * h + pr);
    const uint4 qa = *reinterpret_cast<const uint4 *>(qs), qb = *reinterpret_cast<const uint4 *>(qs + 16);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t hi8 = w[c] >> 8;
      // {1024 + q} - 1024 = q exactly, then one fused multiply-add per two weights
      r[32 * pr + 2 * c] = hfma2_u32(hsub2_u32(and_or(w[c], 0x000f000fu, k1024), k1024), ua0, ub0);
      r[32 * pr + 2 * c + 1] = hfma2_u32(hsub2_u32(and_or(hi8, 0x000f000fu, k1024), k1024), ua0, ub0);
      r[32 * pr + 16 + 2 * c] = hfma2_u32(hsub2_u32(and_or(w[c], 0x00f000f0u, k1024), k1024), ua1, ub1);
      r[32 * pr + 16 + 2 * c + 1] = hfma2_u32(hsub2_u32(and_or(hi8, 0x00f000f0u, k1024), k1024), ua1, ub1);
    }
  }
}

__device__ __forceinline__ uint32_t wide_shift(uint32_t q, int from, int to) { return to >= from ? q << (to - from) : q >> (from - to); }

// Inputs' half h of a Q6_K image row's super-block: half = fl16((u - 32) * s), u - 32 exact. The low nibbles of a pair of
// 32-element groups share bytes as in Q4_K; a group in the high nibbles enters as 16 (u - 32) against s / 16.
__device__ __forceinline__ void wide_expand_q6k(const uint8_t *row, uint32_t h, uint32_t (&r)[64]) {
  const uint4 sc = *reinterpret_cast<const uint4 *>(row + 192 + 16 * h);  // 8 halves: the scales of elements 128 h ..
  const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
  const uint32_t k1024 = 0x64006400u;
#pragma unroll
  for (uint32_t pr = 0; pr < 2; ++pr) {
    const uint8_t *ql = row + 32 * (2 * h + pr);
    const uint4 qa = *reinterpret_cast<const uint4 *>(ql), qb = *reinterpret_cast<const uint4 *>(ql + 16);
    const uint4 qh = *reinterpret_cast<const uint4 *>(row + 128 + 16 * (2 * h + pr));
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w}, hw[4] = {qh.x, qh.y, qh.z, qh.w};
    // the pair's four scales: low group's elements 0..15, 16..31, high group's 0..15, 16..31
    const uint32_t sa = scw[2 * pr], sb = scw[2 * pr + 1];
    const uint32_t s_lo[2] = {__byte_perm(sa, sa, 0x1010), __byte_perm(sa, sa, 0x3232)};
    const uint32_t t0 = __byte_perm(sb, sb, 0x1010), t1 = __byte_perm(sb, sb, 0x3232);
    const uint32_t s_hi[2] = {hmul2_u32(t0, 0x2c002c00u), hmul2_u32(t1, 0x2c002c00u)};  // / 16
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint32_t hi8 = w[c] >> 8, q = hw[c >> 1];
      // Output j's two high bits sit at bits b + 2 j (and 16 higher) of the plane's word, b = 8 (c & 1). They go to
      // [5:4] of each half beside a low nibble, to [9:8] beside a high nibble (16 u).
      const int b = 8 * (c & 1);
      const uint32_t f0 = wide_shift(q, b, 4), f1 = wide_shift(q, b + 2, 4), f2 = wide_shift(q, b + 4, 8), f3 = wide_shift(q, b + 6, 8);
      const uint32_t v0 = and_or(f0, 0x00300030u, and_or(w[c], 0x000f000fu, k1024));
      const uint32_t v1 = and_or(f1, 0x00300030u, and_or(hi8, 0x000f000fu, k1024));
      const uint32_t v2 = and_or(f2, 0x03000300u, and_or(w[c], 0x00f000f0u, k1024));
      const uint32_t v3 = and_or(f3, 0x03000300u, and_or(hi8, 0x00f000f0u, k1024));
      r[32 * pr + 2 * c] = hmul2_u32(hsub2_u32(v0, 0x64206420u), s_lo[c >> 2]);           // 1024 + 32
      r[32 * pr + 2 * c + 1] = hmul2_u32(hsub2_u32(v1, 0x64206420u), s_lo[c >> 2]);
      r[32 * pr + 16 + 2 * c] = hmul2_u32(hsub2_u32(v2, 0x66006600u), s_hi[c >> 2]);      // 1024 + 512
      r[32 * pr + 16 + 2 * c + 1] = hmul2_u32(hsub2_u32(v3, 0x66006600u), s_hi[c >> 2]);
    }
  }
}

// Inputs' half h of an NVFP4 image row's super-block. An e2m1 code's three magnitude bits at bits 11..9 of a half are
// |value| * 2^-14 exactly (the subnormal 0.5 included), the sign goes to bit 15; the 2^14 is in the image's scales.
__device__ __forceinline__ void wide_expand_nvfp4(const uint8_t *row, uint32_t h, uint32_t (&r)[64]) {
  const uint4 sc = *reinterpret_cast<const uint4 *>(row + 128 + 16 * h);
  const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint4 qv = *reinterpret_cast<const uint4 *>(row + 64 * h + 16 * g);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = 4 * g + i;  // word c of this half: elements 8 c .. 8 c + 7, scale c / 2
      const uint32_t s2 = (c >> 1) & 1 ? __byte_perm(scw[c >> 2], 0, 0x3232) : __byte_perm(scw[c >> 2], 0, 0x1010);
      const uint32_t x = w[i];
      r[4 * c] = hmul2_u32(and_or(x << 9, 0x0e000e00u, (x << 12) & 0x80008000u), s2);
      r[4 * c + 1] = hmul2_u32(and_or(x << 5, 0x0e000e00u, (x << 8) & 0x80008000u), s2);
      r[4 * c + 2] = hmul2_u32(and_or(x << 1, 0x0e000e00u, (x << 4) & 0x80008000u), s2);
      r[4 * c + 3] = hmul2_u32(and_or(x >> 3, 0x0e000e00u, x & 0x80008000u), s2);
    }
  }
}

// Inputs' half h of a Q8_0 image row's super-block (four blocks of 32): half = fl16(c * s), c exact: the image's byte is c + 128,
// beside 0x64 it reads 1024 + 128 + c.
__device__ __forceinline__ void wide_expand_q80(const uint8_t *row, uint32_t h, uint32_t (&r)[64]) {
  const uint2 sc = *reinterpret_cast<const uint2 *>(row + 256 + 8 * h);  // 4 halves: the scales of blocks 4 h ..
  const uint32_t scw[2] = {sc.x, sc.y};
#pragma unroll
  for (int g = 0; g < 8; ++g) {  // 16 codes a load; two loads a block
    const uint4 qv = *reinterpret_cast<const uint4 *>(row + 128 * h + 16 * g);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
    const uint32_t s2 = (g >> 1) & 1 ? __byte_perm(scw[g >> 2], 0, 0x3232) : __byte_perm(scw[g >> 2], 0, 0x1010);
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // elements 4 i .. 4 i + 3 of the load: halves (e0, e2) and (e1, e3)
      r[8 * g + 2 * i] = hmul2_u32(hsub2_u32(__byte_perm(w[i], 0x64646464u, 0x4240), 0x64806480u), s2);
      r[8 * g + 2 * i + 1] = hmul2_u32(hsub2_u32(__byte_perm(w[i], 0x64646464u, 0x4341), 0x64806480u), s2);
    }
  }
}

template <uint32_t FMT>
__device__ __forceinline__ void wide_expand(const uint8_t *row, uint32_t h, uint32_t (&r)[64]) {
  if (FMT == SB_FMT_Q4K) wide_expand_q4k(row, h, r);
  else if (FMT == SB_FMT_Q6K) wide_expand_q6k(row, h, r);
  else if (FMT == SB_FMT_Q80) wide_expand_q80(row, h, r);
  else wide_expand_nvfp4(row, h, r);
}

template <uint32_t FMT>
__global__ void __launch_bounds__(kWideThreads, 1) linear_wide_kernel(const WideParams p, const __grid_constant__ WideMaps maps) {
  constexpr uint32_t kWideRawStages = WideFmt<FMT>::kStages, kWideRawStage = 128 * WideFmt<FMT>::kSb;
  extern __shared__ __align__(128) uint8_t smem[];
  WIDE_KERNEL_T0();
  uint64_t *raw_full = reinterpret_cast<uint64_t *>(smem);        // [kWideRawStages]
  uint64_t *raw_empty = raw_full + kWideMaxRawStages;
  uint64_t *x_full = raw_empty + kWideMaxRawStages;                   // [kWideMaxXStages]
  uint64_t *x_empty = x_full + kWideMaxXStages;
  uint64_t *a_full = x_empty + kWideMaxXStages;                    // [kWideABufs]
  uint64_t *a_empty = a_full + kWideABufs;
  uint64_t *d_full = a_empty + kWideABufs;                         // [2]: per accumulator buffer (the second with p.dbuf)
  uint64_t *d_empty = d_full + 2;                                  // [2]
  uint64_t *h_full = d_empty + 2;                                  // the header (scale_back) has landed
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 496);
  float *scale_back_all = reinterpret_cast<float *>(smem + 512);   // [128], the launch's rows (not grouped)
  uint8_t *x_ring = smem + kWideXOff, *raw_ring = smem + kWideRawOff;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kWideRawStages; ++s) mbar_init(&raw_full[s], 1), mbar_init(&raw_empty[s], 8);
    for (uint32_t s = 0; s < kWideMaxXStages; ++s) mbar_init(&x_full[s], 1), mbar_init(&x_empty[s], p.halves);
    for (uint32_t s = 0; s < kWideABufs; ++s) mbar_init(&a_full[s], 4), mbar_init(&a_empty[s], 1);
    for (uint32_t s = 0; s < 2; ++s) mbar_init(&d_full[s], p.halves), mbar_init(&d_empty[s], kWideEpilogueWarps);
    mbar_init(h_full, 1);
    fence_mbar_init();
  }
  if (warp == kWideMmaWarp0) tmem_alloc(tmem_slot, kWideTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  const bool grouped = p.groups != nullptr;
  if (warp == 0) WIDE_EVENT(0);  // set-up done

  if (warp == kWideRawWarp) {
    // ---- weights: they do not depend on the kernel ahead, so the ring fills at once ----
    const uint64_t policy = policy_evict_first();
    uint32_t rs = 0, rphase = 0, rcount = 0;
    bool ok = true;
    if (grouped) pdl_wait();  // the table of groups comes from the kernels ahead
    const uint32_t n_items = wide_items(p);
    for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const WideItem w = wide_item(p, item);
      for (uint32_t sb = w.sb0; sb < w.sb1 && ok; ++sb)
        for (uint32_t tn = 0; tn < p.halves && ok; ++tn, ++rcount) {
          if (rcount >= kWideRawStages && !wide_warp_wait(&raw_empty[rs], rphase ^ 1, true)) {
            if (lane == 0) wide_expired(p.status, 1);
            ok = false;
            break;
          }
          if (lane == 0) {
            mbar_arrive_expect_tx(&raw_full[rs], kWideRawStage);
            tma_load_2d(raw_ring + rs * kWideRawStage, &maps.m[tn], int(sb * (WideFmt<FMT>::kSb / 4)), int(w.wrow0 + (p.gate_up ? w.tile * 128 : w.tile * 128 * p.halves + tn * 128)), &raw_full[rs], policy, true);
          }
          if (++rs == kWideRawStages) rs = 0, rphase ^= 1;
        }
    }
    // Do not leave while copies are in flight: every stage issued is waited for (bounded) before the warp returns.
    for (uint32_t f = rcount > kWideRawStages ? rcount - kWideRawStages : 0; f < rcount; ++f)
      if (!wide_warp_wait(&raw_empty[f % kWideRawStages], (f / kWideRawStages) & 1, true)) break;
  } else if (warp == kWideXWarp) {
    // ---- X: a group is the four stages (64 inputs each) of one super-block; the ring holds x_groups of them ----
    pdl_wait();  // X comes from the kernel ahead
    if (lane == 0 && !grouped) {
      mbar_arrive_expect_tx(h_full, 512);
      bulk_g2s(scale_back_all, p.prepared, 512, h_full);
    }
    uint32_t xg = 0, xphase = 0, xcount = 0;
    bool ok = true;
    const uint32_t group_bytes = 4 * p.x_stage_bytes;  // a ring slot (sized for the launch's most rows)
    const uint32_t n_items = wide_items(p);
    for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const WideItem w = wide_item(p, item);
      for (uint32_t sb = w.sb0; sb < w.sb1 && ok; ++sb, ++xcount) {
        if (xcount >= p.x_groups && !wide_warp_wait(&x_empty[xg], xphase ^ 1, true)) {
          if (lane == 0) wide_expired(p.status, 2);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t bytes = 512 * w.rows_padded;  // a super-block of the item's rows
          mbar_arrive_expect_tx(&x_full[xg], bytes);
          bulk_g2s(x_ring + xg * group_bytes, w.x + size_t(sb) * bytes, bytes, &x_full[xg]);
        }
        if (++xg == p.x_groups) xg = 0, xphase ^= 1;
      }
    }
    for (uint32_t f = xcount > p.x_groups ? xcount - p.x_groups : 0; f < xcount; ++f)
      if (!wide_warp_wait(&x_empty[f % p.x_groups], (f / p.x_groups) & 1, true)) break;
  } else if (warp >= kWideMmaWarp0) {
    // ---- MMA issuers: one thread per half of the item (its own accumulator, so the sums' order is fixed). A single
    // thread issues one tcgen05.mma of this shape per 100 to 125 cycles whatever N is; two threads keep the tensor pipe
    // busy at N = 128 (measured: 62 to 70 cycles per MMA overall). ----
    if (lane == 0 && warp - kWideMmaWarp0 < p.halves) {
      const uint32_t tn = warp - kWideMmaWarp0;
      if (grouped) pdl_wait();
      const uint32_t n_items = wide_items(p);
      bool ok = true;
      uint32_t ucount = 0, xg = 0, xphase = 0, done_items = 0;
      for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++done_items) {
        const uint32_t buf = p.dbuf ? done_items & 1 : 0, uses = p.dbuf ? done_items >> 1 : done_items;  // uses of this buffer so far
        const uint32_t d0 = tmem + tn * kWideDCols + buf * (kWideDCols / 2);
        if (uses > 0) {  // the buffer's sums of its item before must have been read
          ok = mbar_wait(&d_empty[buf], (uses - 1) & 1);
          if (!ok) { wide_expired(p.status, 3); break; }
        }
        const WideItem w = wide_item(p, item);
        const uint32_t idesc = umma_idesc_f16(128, w.rows_padded);
        for (uint32_t sb = w.sb0; sb < w.sb1 && ok; ++sb) {
          {
            WIDE_T0();
            ok = mbar_wait(&x_full[xg], xphase);
            if (tn == 0) WIDE_TADD(1, 2);
          }
          if (!ok) { wide_expired(p.status, 5); break; }
          const uint32_t xbase = smem_u32(x_ring + xg * 4 * p.x_stage_bytes);
          for (uint32_t hh = 0; hh < 2 && ok; ++hh, ++ucount) {
            const uint32_t ab = 2 * tn + hh;  // this half's A buffer for inputs' half hh
            {
              WIDE_T0();
              ok = mbar_wait(&a_full[ab], ucount >> 1 & 1);
              if (tn == 0) WIDE_TADD(1, 0);
            }
            if (!ok) { wide_expired(p.status, 4); break; }
            if (tn == 0 && ucount == 0) WIDE_EVENT(2);  // first MMA
            WIDE_T0();
            tc_fence_after_sync();
            const uint32_t a0 = tmem + kWideACol0 + ab * kWideACols;
#pragma unroll
            for (uint32_t i = 0; i < 8; ++i) {  // K-step i of this half of the super-block
              const uint64_t b = umma_smem_desc(xbase + (8 * hh + i) * w.rows_padded * 32, 128, 256);
              umma_f16_ts(d0, a0 + i * 8, b, idesc, !(sb == w.sb0 && hh == 0 && i == 0));
            }
            umma_commit(&a_empty[ab]);
            if (tn == 0) WIDE_TADD(1, 1);
          }
          if (ok) umma_commit(&x_empty[xg]);  // this half of the item has read the group (the barrier counts both halves)
          if (++xg == p.x_groups) xg = 0, xphase ^= 1;
        }
        if (ok) umma_commit(&d_full[buf]);
        if (tn == 0) WIDE_EVENT(3);  // last MMA issued
      }
    }
    __syncwarp();
  } else if (warp < kWideDequantWarps) {
    // ---- dequant: warp (tn, h, q) expands inputs' half h of rows 32 q .. 32 q + 31 of half tn of the item, super-block by
    // super-block: its raw stages are every other one of the ring, its A buffer is 2 tn + h ----
    const uint32_t q = warp & 3, h = (warp >> 2) & 1, tn = warp >> 3, row = 32 * q + lane;
    const uint32_t ab = 2 * tn + h;
    uint32_t rs = tn, rphase = 0, scount = 0;  // super-blocks this warp has expanded
    bool ok = tn < p.halves;
    if (grouped) pdl_wait();
    const uint32_t n_items = wide_items(p);
    for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const WideItem w = wide_item(p, item);
      for (uint32_t sb = w.sb0; sb < w.sb1 && ok; ++sb, ++scount) {
        {
          WIDE_T0();
          if (!wide_warp_wait(&raw_full[rs], rphase)) {
            if (lane == 0) wide_expired(p.status, 6);
            ok = false;
            break;
          }
          if (warp == 0) WIDE_TADD(0, 0);
          if (warp == 0 && scount == 0) WIDE_EVENT(1);  // first weights landed
        }
        uint32_t r[64];
        {
          WIDE_T0();
          wide_expand<FMT>(raw_ring + rs * kWideRawStage + row * WideFmt<FMT>::kSb, h, r);
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[rs]);  // the row's bytes are in registers
          if (warp == 0) WIDE_TADD(0, 1);
        }
        rs += p.halves;
        if (rs >= kWideRawStages) rs -= kWideRawStages, rphase ^= 1;
        {
          WIDE_T0();
          if (scount > 0 && !wide_warp_wait(&a_empty[ab], (scount - 1) & 1)) {
            if (lane == 0) wide_expired(p.status, 7);
            ok = false;
            break;
          }
          if (warp == 0) WIDE_TADD(0, 2);
        }
        {
          WIDE_T0();
          tc_fence_after_sync();
          const uint32_t ta = tmem_addr(tmem, 32 * q, kWideACol0 + ab * kWideACols);
          tmem_st16(ta, r), tmem_st16(ta + 16, r + 16), tmem_st16(ta + 32, r + 32), tmem_st16(ta + 48, r + 48);
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[ab]);
          if (warp == 0) WIDE_TADD(0, 3);
        }
      }
    }
  } else {
    // ---- epilogue: a thread per weight row of each half of the item ----
    const uint32_t q = warp & 3, row = 32 * q + lane;
    pdl_wait();  // aux / out belong to the stream's earlier kernels until they finish
    bool ok = grouped || wide_warp_wait(h_full, 0);
    if (!ok && lane == 0) wide_expired(p.status, 8);
    uint32_t done_items = 0;
    const uint32_t n_items = wide_items(p);
    float *own_scales = reinterpret_cast<float *>(smem + 1024 + 512 * q);
    for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++done_items) {
      const WideItem w = wide_item(p, item);
      const uint32_t buf = p.dbuf ? done_items & 1 : 0, uses = p.dbuf ? done_items >> 1 : done_items;
      const float *scale_back = grouped ? own_scales : reinterpret_cast<const float *>(smem + 512);
      if (grouped) {  // the rows' scales, a copy per warp
        __syncwarp();
        for (uint32_t i = lane; i < w.rows_padded; i += 32) own_scales[i] = __ldg(p.group_scales + w.slot0 + i);
        __syncwarp();
      }
      {
        WIDE_T0();
        if (!wide_warp_wait(&d_full[buf], uses & 1)) {
          if (lane == 0) wide_expired(p.status, 9);
          ok = false;
          break;
        }
        if (q == 0) WIDE_TADD(2, 0);
      }
      tc_fence_after_sync();
      if (q == 0) WIDE_EVENT(4);  // sums complete
      WIDE_T0();
      const uint32_t t0 = tmem_addr(tmem, 32 * q, buf * (kWideDCols / 2));
      // Per 16 rows of X: the sums out of tensor memory, the epilogue on all 16 without a branch (the chains of the
      // activation overlap), then the stores of the rows that exist.
      if (p.gate_up) {
        const uint32_t col = w.tile * 128 + row;
        const float rg = p.row_scale[0] && col < p.n ? p.row_scale[0][col] : 1.0f, ru = p.row_scale[1] && col < p.n ? p.row_scale[1][col] : 1.0f;
        uint16_t *dst = static_cast<uint16_t *>(p.out) + size_t(w.slot0) * p.out_stride + col;
        for (uint32_t c = 0; c < w.rows_padded; c += 16) {
          float g[16], u[16];
          tmem_ld16_wait(t0 + c, g);
          tmem_ld16_wait(t0 + kWideDCols + c, u);
          uint16_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float s = scale_back[c + j];
            o[j] = float_to_bf16_bits(round_bf16(u[j] * (s * ru)) * silu_f(round_bf16(g[j] * (s * rg))));
          }
          if (col < p.n) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < w.rows) dst[size_t(c + j) * p.out_stride] = o[j];
          }
        }
      } else if (p.epilogue == SB_EPILOGUE_PARTIALS) {
        for (uint32_t half = 0; half < p.halves; ++half) {
          const uint32_t col = w.tile * 128 * p.halves + half * 128 + row;
          const float rw = p.row_scale[0] && col < p.n ? p.row_scale[0][col] : 1.0f;
          float *dst = static_cast<float *>(p.out) + (size_t(w.split) * p.rows_total + p.row0) * p.out_stride + col;
          for (uint32_t c = 0; c < w.rows_padded; c += 16) {
            float v[16];
            tmem_ld16_wait(t0 + half * kWideDCols + c, v);
            if (col < p.n) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < w.rows) dst[size_t(c + j) * p.out_stride] = v[j] * (scale_back[c + j] * rw);
            }
          }
        }
      } else {
        for (uint32_t half = 0; half < p.halves; ++half) {
          const uint32_t col = w.tile * 128 * p.halves + half * 128 + row;
          const bool live = col < p.n;
          const float rw = p.row_scale[0] && live ? p.row_scale[0][col] : 1.0f;
          for (uint32_t c = 0; c < w.rows_padded; c += 16) {
            float v[16];
            tmem_ld16_wait(t0 + half * kWideDCols + c, v);
            float a[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) a[j] = 0.0f;
            if (p.aux && live) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < w.rows) a[j] = bf16_bits_to_float(p.aux[size_t(w.slot0 + c + j) * p.aux_stride + col]);
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] *= scale_back[c + j] * rw;
              if (p.epilogue == SB_EPILOGUE_RESIDUAL) v[j] += a[j];
              else if (p.epilogue == SB_EPILOGUE_UP_WITH_GATE) v[j] = round_bf16(v[j]) * silu_f(a[j]);
            }
            if (!live) continue;
            if (p.out_f32) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < w.rows) static_cast<float *>(p.out)[size_t(w.slot0 + c + j) * p.out_stride + col] = v[j];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < w.rows) static_cast<uint16_t *>(p.out)[size_t(w.slot0 + c + j) * p.out_stride + col] = float_to_bf16_bits(v[j]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&d_empty[buf]);
      if (q == 0) WIDE_TADD(2, 1);
      if (q == 0) WIDE_EVENT(5);  // stored
    }
  }

  WIDE_FLUSH();
  // Everyone meets here, also after a wait that gave up, so tensor memory is always returned.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWideMmaWarp0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kWideTmemCols);
  }
}

static int wide_check(const SbLinearArgs *a, const char *who) {
  SB_REQUIRE(a, "%s: null arguments", who);
  SB_REQUIRE(a->format == SB_FMT_Q4K || a->format == SB_FMT_Q6K || a->format == SB_FMT_NVFP4 || a->format == SB_FMT_Q80,
             "%s: format %u (the many-row kernel multiplies Q4_K rows, and Q6_K, Q8_0 and NVFP4 images)", who, a->format);
  SB_REQUIRE((a->format == SB_FMT_Q4K) != ((a->flags & SB_LINEAR_WIDE_IMAGE) != 0),
             "%s: Q6_K, Q8_0 and NVFP4 weights are given as their image (sb_linear_wide_image, SB_LINEAR_WIDE_IMAGE); Q4_K rows as they are", who);
  SB_REQUIRE(a->rows >= 1, "%s: no rows", who);
  SB_REQUIRE(a->k && a->k % 256 == 0 && a->n && a->n % 8 == 0, "%s: k = %u is not a multiple of 256 or n = %u not a multiple of 8", who, a->k, a->n);
  SB_REQUIRE(a->weights && a->out && (a->x || a->prepared), "%s: null weights, out, or neither x nor prepared", who);
  SB_REQUIRE(a->epilogue <= SB_EPILOGUE_PARTIALS, "%s: epilogue %u (none, residual, up-with-gate, one-pass gate/up or k-split sums)", who, a->epilogue);
  SB_REQUIRE(a->epilogue != SB_EPILOGUE_PARTIALS || a->out_f32, "%s: k-split sums are fp32", who);
  SB_REQUIRE((a->epilogue == SB_EPILOGUE_GATE_UP) == (a->weights2 != nullptr), "%s: weights2 is given exactly with the gate/up epilogue", who);
  SB_REQUIRE((a->epilogue == SB_EPILOGUE_RESIDUAL || a->epilogue == SB_EPILOGUE_UP_WITH_GATE) == (a->aux != nullptr),
             "%s: aux is given exactly with the residual and up-with-gate epilogues", who);
  SB_REQUIRE(a->out_stride >= a->n && (!a->aux || a->aux_stride >= a->n), "%s: a stride is below n", who);
  SB_REQUIRE(!(a->out_f32 && a->epilogue != SB_EPILOGUE_NONE && a->epilogue != SB_EPILOGUE_PARTIALS), "%s: an fp32 destination takes no epilogue", who);
  SB_REQUIRE((reinterpret_cast<uintptr_t>(a->weights) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->weights2) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a->prepared) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->x) & 15) == 0,
             "%s: weights, x and prepared must be 16-byte aligned", who);
  return SB_OK;
}

static int wide_set_attributes() {
  static bool attr_set[64] = {};  // a function attribute is per device
  Context &c = ctx();
  const int dev = c.device >= 0 && c.device < 64 ? c.device : 0;
  if (!attr_set[dev]) {
    SB_CUDA(cudaFuncSetAttribute(linear_wide_kernel<SB_FMT_Q4K>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(wide_smem<SB_FMT_Q4K>())));
    SB_CUDA(cudaFuncSetAttribute(linear_wide_kernel<SB_FMT_Q6K>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(wide_smem<SB_FMT_Q6K>())));
    SB_CUDA(cudaFuncSetAttribute(linear_wide_kernel<SB_FMT_NVFP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(wide_smem<SB_FMT_NVFP4>())));
    SB_CUDA(cudaFuncSetAttribute(linear_wide_kernel<SB_FMT_Q80>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(wide_smem<SB_FMT_Q80>())));
    attr_set[dev] = true;
  }
  return SB_OK;
}

int launch_wide_prepare_grouped(cudaStream_t stream, const WidePrepareGroupedArgs &a) {
  SB_REQUIRE(a.x && a.prepared && a.scales && a.slot_src && a.slot_group && a.slot_count && a.groups && a.max_slots,
             "grouped conversion: null pointer or no slots");
  SB_REQUIRE(a.k && a.k % 256 == 0 && a.x_stride >= a.k && a.x_stride % 8 == 0, "grouped conversion: k = %u is not a multiple of 256, or x_stride %u", a.k, a.x_stride);
  WidePrepParams pp{};
  pp.x = static_cast<const uint16_t *>(a.x), pp.out = static_cast<uint8_t *>(a.prepared), pp.k = a.k, pp.x_stride = a.x_stride;
  pp.slot_src = a.slot_src, pp.slot_group = a.slot_group, pp.slot_count = a.slot_count, pp.groups = a.groups, pp.scales = a.scales;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.max_slots + kWideSlotWarps - 1) / kWideSlotWarps), cfg.blockDim = dim3(32 * kWideSlotWarps), cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = a.pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, wide_prepare_slots_kernel, pp));
  return SB_OK;
}

int launch_linear_wide_grouped(cudaStream_t stream, const WideGroupedArgs &a) {
  SB_REQUIRE(a.weights && a.prepared && a.scales && a.groups && a.group_count && a.out && a.max_groups, "grouped projection: null pointer or no groups");
  SB_REQUIRE(a.k && a.k % 256 == 0, "grouped projection: k = %u is not a multiple of 256", a.k);
  SB_REQUIRE(a.max_rows >= 16 && a.max_rows <= kWideMaxRows && a.max_rows % 16 == 0, "grouped projection: groups of up to %u rows (16 .. 128 in sixteens)", a.max_rows);
  const bool gate_up = a.weights2 != nullptr;
  SB_REQUIRE(a.expert_rows % (gate_up ? 128 : 256) == 0, "grouped projection: %u rows an expert (whole tiles of %u)", a.expert_rows, gate_up ? 128 : 256);
  Context &c = ctx();
  int st = wide_set_attributes();
  if (st != SB_OK) return st;
  WideMaps maps;
  const uint32_t row_bytes = (a.k / 256) * 144, total_rows = a.experts * a.expert_rows;
  st = encode_weight_map(&maps.m[0], reinterpret_cast<uintptr_t>(a.weights), row_bytes, total_rows, 144, 128);
  if (st == SB_OK && gate_up) st = encode_weight_map(&maps.m[1], reinterpret_cast<uintptr_t>(a.weights2), row_bytes, total_rows, 144, 128);
  if (st != SB_OK) return st;
  if (!gate_up) maps.m[1] = maps.m[0];
  WideParams p{};
  p.prepared = static_cast<const uint8_t *>(a.prepared), p.out = a.out, p.status = c.status_dev;
  p.n = a.expert_rows, p.out_stride = a.out_stride, p.epilogue = gate_up ? SB_EPILOGUE_GATE_UP : SB_EPILOGUE_NONE;
  p.nsb = a.k / 256, p.gate_up = gate_up, p.halves = 2, p.splits = 1;
  p.rows = p.rows_padded = a.max_rows;  // (a group's own rows come from the table)
  p.x_stage_bytes = a.max_rows * 128, p.x_groups = std::min(kWideMaxXStages, kWideXBytes / (4 * p.x_stage_bytes));
  p.dbuf = a.max_rows <= kWideDCols / 2 ? 1 : 0;
  p.groups = a.groups, p.group_count = a.group_count, p.group_scales = a.scales;
  p.tiles_per_group = gate_up ? a.expert_rows / 128 : a.expert_rows / 256, p.expert_rows = a.expert_rows;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(std::min<uint32_t>(a.max_groups * p.tiles_per_group, uint32_t(c.sm_count)));
  cfg.blockDim = dim3(kWideThreads), cfg.dynamicSmemBytes = wide_smem<SB_FMT_Q4K>(), cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = a.pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, linear_wide_kernel<SB_FMT_Q4K>, p, maps));
  return SB_OK;
}

}  // namespace sb

using namespace sb;

#ifdef SB_DIAG
extern "C" __attribute__((visibility("default"))) int sb_linear_wide_timing(unsigned long long *out64, int reset) {
  if (out64) cudaMemcpyFromSymbol(out64, g_wide_timing, sizeof(g_wide_timing));
  if (reset) {
    static unsigned long long zero[64] = {};
    cudaMemcpyToSymbol(g_wide_timing, zero, sizeof(zero));
  }
  return 0;
}
#endif

// ---- the images of Q6_K and NVFP4 rows ----
// One CTA per weight row: the row's largest scale magnitude, the power of two that brings it to [256, 512) (Q6_K) or
// [2^13, 2^14) (NVFP4, whose halves carry 2^-14), then every super-block rewritten (layouts at WideFmt).
__device__ __forceinline__ float wide_e4m3(uint32_t b) {  // bias 7, subnormals below exponent 1
  const int e = (b >> 3) & 15, m = b & 7;
  const float mag = e ? ldexpf(1.0f + float(m) * 0.125f, e - 7) : ldexpf(float(m) * 0.125f, -6);
  return (b & 0x80) ? -mag : mag;
}
__device__ __forceinline__ uint32_t wide_q6k_code(const uint8_t *blk, uint32_t e) {  // element e of a native super-block
  const uint32_t j = e >> 5, k = e & 31, n = j >> 2, r = j & 3;
  const uint8_t *ql = blk + 64 * n, *qh = blk + 128 + 32 * n;
  return ((ql[k + 32 * (r & 1)] >> (4 * (r >> 1))) & 15u) | (((qh[k] >> (2 * r)) & 3u) << 4);
}
template <uint32_t FMT>
__global__ void __launch_bounds__(128) wide_image_kernel(const uint8_t *native, uint32_t n, uint32_t nsb, uint8_t *image, float *row_scale) {
  constexpr uint32_t kNative = FMT == SB_FMT_Q6K ? 210 : FMT == SB_FMT_Q80 ? 272 : 148, kSb = WideFmt<FMT>::kSb;  // (Q8_0: eight blocks of 34)
  constexpr uint32_t kScales = FMT == SB_FMT_Q80 ? 8 : 16;  // scales a super-block
  __shared__ float red_s[4];
  const uint32_t row = blockIdx.x, tid = threadIdx.x;
  const uint8_t *src = native + size_t(row) * nsb * kNative;
  auto scale_of = [&](const uint8_t *blk, uint32_t i) -> float {  // scale i of the super-block, fp32 as the format defines it
    if (FMT == SB_FMT_Q80) return __half2float(*reinterpret_cast<const __half *>(blk + 34 * i));
    if (FMT == SB_FMT_Q6K) {
      const __half d = *reinterpret_cast<const __half *>(blk + 208);
      return __half2float(d) * float(reinterpret_cast<const int8_t *>(blk + 192)[i]);
    }
    float g;
    memcpy(&g, blk + 16, 4);
    return wide_e4m3(blk[i]) * g;
  };
  float mx = 0.0f;
  for (uint32_t u = tid; u < nsb * kScales; u += 128) {
    const float v = fabsf(scale_of(src + (u / kScales) * kNative, u % kScales));
    if (v <= 3.0e38f) mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red_s[tid >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
  int e = 0;
  if (mx > 0.0f) {
    (void)frexpf(mx, &e);  // mx = m 2^e, m in [0.5, 1)
    e -= FMT == SB_FMT_Q6K ? 9 : FMT == SB_FMT_Q80 ? 7 : 0;  // largest scale to [256, 512) / [64, 128) / [2^13, 2^14) after the 2^14 below
  }
  if (tid == 0) row_scale[row] = ldexpf(1.0f, e);
  const float down = ldexpf(1.0f, (FMT == SB_FMT_NVFP4 ? 14 : 0) - e);
  uint8_t *dst_row = image + size_t(row) * nsb * kSb;
  for (uint32_t sb = 0; sb < nsb; ++sb) {
    const uint8_t *blk = src + sb * kNative;
    uint8_t *dst = dst_row + sb * kSb;
    if (FMT == SB_FMT_Q80) {
      // codes + 128 in element order, then the eight blocks' scales
      for (uint32_t el = tid; el < 256; el += 128) dst[el] = uint8_t(reinterpret_cast<const int8_t *>(blk + 34 * (el >> 5) + 2)[el & 31] + 128);
      if (tid < 8) reinterpret_cast<__half *>(dst + 256)[tid] = __float2half_rn(scale_of(blk, tid) * down);
    } else if (FMT == SB_FMT_Q6K) {
      // ql': byte i of pair-block pb (64 elements from 64 pb) = low nibbles of its first 32 elements | of its next 32 << 4
      {
        const uint32_t pb = tid >> 5, i = tid & 31;
        const uint32_t a = wide_q6k_code(blk, 64 * pb + i), bb = wide_q6k_code(blk, 64 * pb + 32 + i);
        dst[32 * pb + i] = uint8_t((a & 15u) | ((bb & 15u) << 4));
      }
      // qh': word w of pair-block pb serves ql' words c = 2 w, 2 w + 1; output j of word c at bits 8 (c & 1) + 2 j (+16)
      if (tid < 16) {
        const uint32_t pb = tid >> 2, w = tid & 3;
        uint32_t word = 0;
        for (uint32_t cc = 0; cc < 2; ++cc)
          for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t c = 2 * w + cc, base = 64 * pb + (j >= 2 ? 32 : 0) + 4 * c + (j & 1);
            const uint32_t lo = wide_q6k_code(blk, base) >> 4, hi = wide_q6k_code(blk, base + 2) >> 4;
            word |= (lo << (8 * cc + 2 * j)) | (hi << (8 * cc + 2 * j + 16));
          }
        reinterpret_cast<uint32_t *>(dst + 128)[4 * pb + w] = word;
      }
      if (tid >= 32 && tid < 48) reinterpret_cast<__half *>(dst + 192)[tid - 32] = __float2half_rn(scale_of(blk, tid - 32) * down);
    } else {
      // nibbles of every 8 elements in the order [0, 1, 4, 5, 2, 3, 6, 7]: nibbles k and k + 4 of a word are neighbours in
      // the order the inputs are laid out in ([0, 2, 1, 3] within every four)
      if (tid < 32) {
        const uint32_t order[8] = {0, 1, 4, 5, 2, 3, 6, 7};
        uint32_t word = 0;
        for (uint32_t k = 0; k < 8; ++k) {
          const uint32_t el = 8 * tid + order[k];
          word |= uint32_t((blk[20 + el / 2] >> (4 * (el & 1))) & 15u) << (4 * k);
        }
        reinterpret_cast<uint32_t *>(dst)[tid] = word;
      }
      if (tid >= 32 && tid < 48) reinterpret_cast<__half *>(dst + 128)[tid - 32] = __float2half_rn(scale_of(blk, tid - 32) * down);
    }
  }
}

// k-splits of a projection left as SB_EPILOGUE_PARTIALS: as many as fill the SMs with two-half items, three super-blocks
// each at least.
static uint32_t wide_splits(uint32_t n, uint32_t k, int sm_count) {
  const uint32_t tiles = (n + 255) / 256, nsb = k / 256;
  if (!tiles || !nsb) return 1;
  return std::max(1u, std::min(uint32_t(sm_count) / tiles, nsb / 3));
}
extern "C" uint32_t sb_linear_wide_splits(uint32_t n, uint32_t k) { return ctx().ready ? wide_splits(n, k, ctx().sm_count) : 0; }

static uint32_t wide_sb_bytes(uint32_t format) {
  return format == SB_FMT_Q4K ? WideFmt<SB_FMT_Q4K>::kSb : format == SB_FMT_Q6K ? WideFmt<SB_FMT_Q6K>::kSb : format == SB_FMT_NVFP4 ? WideFmt<SB_FMT_NVFP4>::kSb
       : format == SB_FMT_Q80 ? WideFmt<SB_FMT_Q80>::kSb : 0;
}
extern "C" uint64_t sb_linear_wide_image_bytes(uint32_t format, uint32_t n, uint32_t k) {
  if ((format != SB_FMT_Q6K && format != SB_FMT_NVFP4 && format != SB_FMT_Q80) || !n || !k || k % 256) return 0;
  return uint64_t(n) * (k / 256) * wide_sb_bytes(format) + uint64_t(n) * 4;  // the rows, then a scale per row
}
extern "C" int sb_linear_wide_image(void *stream, uint32_t format, const void *weights, uint32_t n, uint32_t k, void *image_out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(format == SB_FMT_Q6K || format == SB_FMT_NVFP4 || format == SB_FMT_Q80, "sb_linear_wide_image: format %u (Q6_K, Q8_0 and NVFP4 rows have images; Q4_K rows are read as they are)", format);
  SB_REQUIRE(weights && image_out && n && k && k % 256 == 0, "sb_linear_wide_image: null pointer, no rows or k = %u not a multiple of 256", k);
  SB_REQUIRE((reinterpret_cast<uintptr_t>(image_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(weights) & 1) == 0, "sb_linear_wide_image: the image must be 16-byte aligned, the rows 2-byte");
  const uint32_t nsb = k / 256;
  uint8_t *image = static_cast<uint8_t *>(image_out);
  float *row_scale = reinterpret_cast<float *>(image + size_t(n) * nsb * wide_sb_bytes(format));
  if (format == SB_FMT_Q6K) wide_image_kernel<SB_FMT_Q6K><<<n, 128, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(weights), n, nsb, image, row_scale);
  else if (format == SB_FMT_Q80) wide_image_kernel<SB_FMT_Q80><<<n, 128, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(weights), n, nsb, image, row_scale);
  else wide_image_kernel<SB_FMT_NVFP4><<<n, 128, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(weights), n, nsb, image, row_scale);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" uint64_t sb_linear_wide_prepared_bytes(uint32_t rows, uint32_t k) {
  if (!rows || !k || k % 256) return 0;
  const uint64_t passes = (rows + kWideMaxRows - 1) / kWideMaxRows;
  return passes * (kWideHeader + uint64_t(kWideMaxRows) * k * 2);  // every pass sized for a full one
}

// One pass = up to 128 rows; pass i of the conversion starts at sb_linear_wide_prepared_bytes(128, k) * i.
static int wide_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride, const void *norm_weight, void *prepared_out,
                        uint32_t flags, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual, uint32_t residual_stride,
                        void *normed_out = nullptr);

extern "C" int sb_linear_wide_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride, const void *norm_weight,
                                      void *prepared_out, uint32_t flags) {
  return wide_prepare(stream, x, rows, k, x_stride, norm_weight, prepared_out, flags, nullptr, 0, 0, nullptr, 0);
}

extern "C" int sb_linear_wide_prepare_normed(void *stream, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual,
                                             uint32_t residual_stride, void *x_or_sum_out, uint32_t x_stride, uint32_t rows, uint32_t k,
                                             const void *norm_weight, void *prepared_out, void *normed_out, uint32_t flags) {
  if (!partials) return wide_prepare(stream, x_or_sum_out, rows, k, x_stride, norm_weight, prepared_out, flags, nullptr, 0, 0, nullptr, 0, normed_out);
  SB_REQUIRE(residual && x_or_sum_out && splits >= 1 && splits <= 64, "sb_linear_wide_prepare_normed: null residual or destination, or %u splits", splits);
  SB_REQUIRE(partial_stride >= k && partial_stride % 4 == 0 && residual_stride >= k && residual_stride % 8 == 0,
             "sb_linear_wide_prepare_normed: partial_stride %u or residual_stride %u", partial_stride, residual_stride);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(residual)) & 15) == 0, "sb_linear_wide_prepare_normed: pointers must be 16-byte aligned");
  return wide_prepare(stream, x_or_sum_out, rows, k, x_stride, norm_weight, prepared_out, flags, partials, splits, partial_stride, residual, residual_stride, normed_out);
}

extern "C" int sb_linear_wide_prepare_sum(void *stream, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual,
                                          uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                                          const void *norm_weight, void *prepared_out, uint32_t flags) {
  SB_REQUIRE(partials && residual && sum_out && splits >= 1 && splits <= 64, "sb_linear_wide_prepare_sum: null partials, residual or destination, or %u splits", splits);
  SB_REQUIRE(partial_stride >= k && partial_stride % 4 == 0 && residual_stride >= k && residual_stride % 8 == 0,
             "sb_linear_wide_prepare_sum: partial_stride %u or residual_stride %u", partial_stride, residual_stride);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(residual)) & 15) == 0, "sb_linear_wide_prepare_sum: pointers must be 16-byte aligned");
  return wide_prepare(stream, sum_out, rows, k, sum_stride, norm_weight, prepared_out, flags, partials, splits, partial_stride, residual, residual_stride);
}

static int wide_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride, const void *norm_weight, void *prepared_out,
                        uint32_t flags, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual, uint32_t residual_stride,
                        void *normed_out) {
  SB_NEED_DEVICE();
  SB_REQUIRE(!normed_out || (norm_weight && (reinterpret_cast<uintptr_t>(normed_out) & 15) == 0), "sb_linear_wide_prepare: normalised rows come with a norm weight, 16-byte aligned");
  SB_REQUIRE(x && prepared_out && rows >= 1, "sb_linear_wide_prepare: null x or destination, or no rows");
  SB_REQUIRE(k && k % 256 == 0 && x_stride >= k && x_stride % 8 == 0, "sb_linear_wide_prepare: k = %u is not a multiple of 256, or x_stride %u", k, x_stride);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(prepared_out) | reinterpret_cast<uintptr_t>(norm_weight)) & 15) == 0,
             "sb_linear_wide_prepare: pointers must be 16-byte aligned");
  const uint64_t pass_bytes = sb_linear_wide_prepared_bytes(kWideMaxRows, k);
  for (uint32_t r0 = 0, pass = 0; r0 < rows; r0 += kWideMaxRows, ++pass) {
    const uint32_t n = std::min(kWideMaxRows, rows - r0), padded = (n + 15) / 16 * 16;
    WidePrepParams pp{static_cast<const uint16_t *>(x) + size_t(r0) * x_stride, static_cast<const float *>(norm_weight),
                      static_cast<uint8_t *>(prepared_out) + pass * pass_bytes, n, padded, k, x_stride,
                      partials, residual ? static_cast<const uint16_t *>(residual) + size_t(r0) * residual_stride : nullptr,
                      splits, rows, r0, partial_stride, residual_stride};
    pp.normed_out = normed_out ? static_cast<uint16_t *>(normed_out) + size_t(r0) * k : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(padded), cfg.blockDim = dim3(kWidePrepThreads), cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = (flags & SB_LINEAR_PDL) ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&cfg, wide_prepare_kernel, pp));
  }
  return SB_OK;
}

extern "C" int sb_linear_wide(void *stream, const SbLinearArgs *a) {
  SB_NEED_DEVICE();
  const int valid = wide_check(a, "sb_linear_wide");
  if (valid != SB_OK) return valid;
  Context &c = ctx();
  const void *prepared = a->prepared;
  if (!prepared) {
    SB_REQUIRE(sb_linear_wide_prepared_bytes(a->rows, a->k) <= c.wide_prepared_bytes, "sb_linear_wide: %u rows of k = %u exceed the context's conversion scratch", a->rows, a->k);
    const int st = sb_linear_wide_prepare(stream, a->x, a->rows, a->k, a->x_stride, a->norm_weight, c.wide_prepared, a->flags);
    if (st != SB_OK) return st;
    prepared = c.wide_prepared;
  }
  const bool gate_up = a->epilogue == SB_EPILOGUE_GATE_UP, split_k = a->epilogue == SB_EPILOGUE_PARTIALS;
  WideMaps maps;
  const uint32_t sb_bytes = wide_sb_bytes(a->format), row_bytes = (a->k / 256) * sb_bytes;
  const bool image = a->format != SB_FMT_Q4K;
  const float *row_scale[2] = {image ? reinterpret_cast<const float *>(static_cast<const uint8_t *>(a->weights) + size_t(a->n) * row_bytes) : nullptr,
                               image && a->weights2 ? reinterpret_cast<const float *>(static_cast<const uint8_t *>(a->weights2) + size_t(a->n) * row_bytes) : nullptr};
  if (gate_up) {
    int st = encode_weight_map(&maps.m[0], reinterpret_cast<uintptr_t>(a->weights), row_bytes, a->n, sb_bytes, 128);
    if (st == SB_OK) st = encode_weight_map(&maps.m[1], reinterpret_cast<uintptr_t>(a->weights2), row_bytes, a->n, sb_bytes, 128);
    if (st != SB_OK) return st;
  } else {
    // The item's halves are rows [256 i, 256 i + 128) and [256 i + 128, 256 i + 256): two maps over every other block of 128
    // rows would need a 3-D map; instead the second half is the same map shifted by 128 rows (rows past n read as zero).
    int st = encode_weight_map(&maps.m[0], reinterpret_cast<uintptr_t>(a->weights), row_bytes, a->n, sb_bytes, 128);
    if (st != SB_OK) return st;
    maps.m[1] = maps.m[0];
  }
  {
    const int st = wide_set_attributes();
    if (st != SB_OK) return st;
  }
  const uint64_t pass_bytes = sb_linear_wide_prepared_bytes(kWideMaxRows, a->k);
  for (uint32_t r0 = 0, pass = 0; r0 < a->rows; r0 += kWideMaxRows, ++pass) {
    WideParams p{};
    p.prepared = static_cast<const uint8_t *>(prepared) + pass * pass_bytes;
    p.rows = std::min(kWideMaxRows, a->rows - r0), p.rows_padded = (p.rows + 15) / 16 * 16;
    const size_t esz = a->out_f32 ? 4 : 2;
    p.aux = a->aux ? static_cast<const uint16_t *>(a->aux) + size_t(r0) * a->aux_stride : nullptr;
    p.out = split_k ? static_cast<uint8_t *>(a->out) : static_cast<uint8_t *>(a->out) + size_t(r0) * a->out_stride * esz;
    p.status = c.status_dev;
    p.n = a->n, p.aux_stride = a->aux_stride, p.out_stride = a->out_stride, p.epilogue = a->epilogue, p.out_f32 = a->out_f32;
    p.nsb = a->k / 256, p.gate_up = gate_up;
    // Items of two halves read X once for 256 weight rows; where they would leave SMs idle, items of one half fill more.
    p.halves = gate_up || split_k || (a->n + 255) / 256 >= uint32_t(c.sm_count) ? 2 : 1;
    p.splits = split_k ? wide_splits(a->n, a->k, c.sm_count) : 1;
    p.rows_total = a->rows, p.row0 = r0;
    p.items = (gate_up ? (a->n + 127) / 128 : (a->n + 128 * p.halves - 1) / (128 * p.halves)) * p.splits;
    p.x_stage_bytes = p.rows_padded * 128;
    p.x_groups = std::min(kWideMaxXStages, kWideXBytes / (4 * p.x_stage_bytes));
    p.dbuf = p.rows_padded <= kWideDCols / 2 ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min<uint32_t>(p.items, uint32_t(c.sm_count)));
    cfg.blockDim = dim3(kWideThreads);
    cfg.dynamicSmemBytes = a->format == SB_FMT_Q4K ? wide_smem<SB_FMT_Q4K>() : a->format == SB_FMT_Q6K ? wide_smem<SB_FMT_Q6K>()
                         : a->format == SB_FMT_Q80 ? wide_smem<SB_FMT_Q80>() : wide_smem<SB_FMT_NVFP4>();
    p.row_scale[0] = row_scale[0], p.row_scale[1] = row_scale[1];
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = (a->flags & SB_LINEAR_PDL) ? 1 : 0;
    if (a->format == SB_FMT_Q4K) SB_CUDA(cudaLaunchKernelEx(&cfg, linear_wide_kernel<SB_FMT_Q4K>, p, maps));
    else if (a->format == SB_FMT_Q6K) SB_CUDA(cudaLaunchKernelEx(&cfg, linear_wide_kernel<SB_FMT_Q6K>, p, maps));
    else if (a->format == SB_FMT_Q80) SB_CUDA(cudaLaunchKernelEx(&cfg, linear_wide_kernel<SB_FMT_Q80>, p, maps));
    else SB_CUDA(cudaLaunchKernelEx(&cfg, linear_wide_kernel<SB_FMT_NVFP4>, p, maps));
  }
  return SB_OK;
}
