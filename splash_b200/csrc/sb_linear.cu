// Quantized linear for the verify step's small M (<= 16 rows): Y[M,N] = X[M,K] W[N,K]^T over
// GGUF native super-blocks streamed exactly once from HBM.
//
// Takes the place of the reference's decode projection kernels
// (runtime/metal/kernels/shared/gguf_linear.metal:113-130 staged tile,
// runtime/metal/kernels/decode/linear_gguf_sgmatrix.metal:1-27 register tile) and of the host
// encoding in runtime/ops/LinearGguf.cpp:281-362. The arithmetic follows the register tile's idea:
// integer codes are fed to the tensor cores as exactly represented operands and the floating
// scales are applied to fp32 sums, so for Q4_K the effective weight is the unrounded
// d*sc*q - dmin*mn.
//
// Layout of one launch
//   prepare   a small kernel converts the 16 x K activations once (optionally through a fused
//             RMSNorm) to fp16 with a per-row power-of-two scale, in MMA fragment order
//   grid      one persistent CTA per SM (a multiple of the k-slice count): 12 (Q4_K) or 8 (Q6_K, Q8_0) consumer
//             warps (2 row groups x 6 or 4 k-groups), 1 producer warp, 3 epilogue warps that take tiles in turn
//   k-slices  K's super-blocks are cut into S contiguous slices; a CTA owns one slice for the whole
//             launch and keeps its slice of the prepared activations resident in shared memory
//             (one bulk copy)
//   tiles     64 weight rows x slice; the producer warp streams each tile's rows into a ring of
//             stages (64 rows x 4 super-blocks) with tiled 2-D TMA copies (cp.async.bulk.tensor, no multicast)
//             completing on mbarriers; consumer warp (rg, kg) multiplies rows 32 rg..32 rg+31 of the stage's
//             super-blocks dealt to k-group kg: mma.sync m16n8k16 (A = 16 weight rows, B = 8 tokens) into fp32
//   Q4_K      operand = sc*q (exact integer <= 945 in fp16, built as (1024+q)*sc - 1024*sc with one
//             LOP3 and one HFMA2 per two weights); per super-block y += d*Aq - dmin*Am, where Am is
//             one more MMA of the 6-bit mins against the sub-block sums of x (split hi + lo fp16)
//   Q6_K      operand = fp16(sc*(q-32)) (one rounding when |.| > 2048); y += d*Aq per super-block
//   Q8_0      operand = fp16(d*q), the value the reference's staged tile rounds to
//   reduce    an epilogue warp adds the k-group warps' sums in order from shared memory while the
//             consumers start the next tile; with S > 1 the slices publish fp32 partials and the
//             last arriver adds them in slice order (or, SB_EPILOGUE_PARTIALS, leaves them to the next input conversion)
//             (runtime/metal/kernels/common/split_reduce.h:24-55), then applies the epilogue
//             (runtime/metal/kernels/common/gguf_tile.h:8-14, gguf_linear.metal:38)
#include <algorithm>

#include <cooperative_groups.h>
#include <cuda.h>

#include "sb_internal.h"
#include "sb_linear_internal.h"
#include "sb_tp_internal.cuh"
#include "sb_ptx.cuh"

#ifndef SB_Q4K_I2_UNROLL
#define SB_Q4K_I2_UNROLL 4
#endif
// Diagnostic switches (parts of the kernel turned off to time the rest) exist only in a build with -DSB_DIAG, where the
// flags word's bits 8.. carry them; the shipped library ignores nothing: it refuses unknown flag bits.
#ifdef SB_DIAG
#define SB_DBG(bit) ((p.debug & (bit)) != 0)
#else
#define SB_DBG(bit) false
#endif
#define SB_PRAGMA_(x) _Pragma(#x)
#define SB_PRAGMA(x) SB_PRAGMA_(x)
#define SB_UNROLL_Q4K_I2 SB_PRAGMA(unroll SB_Q4K_I2_UNROLL)

namespace sb {

constexpr int kTokens = 16;         // rows of X one launch multiplies
constexpr int kRG = 2, kMT = 2;          // row groups of consumer warps; m-tiles per warp
constexpr int kEpiWarps = 3;             // tiles of a CTA go to the epilogue warps in turn; a tile's finish takes longer than its sums
constexpr int kTileRows = kRG * kMT * 16; // 64
constexpr int kStageSb = 4;               // super-blocks per ring stage
constexpr int kMaxStages = 8;
constexpr int kMaxSliceSb = 10;           // super-blocks of activations a CTA keeps resident (80 KiB)
// A consumer warp's tile sums in shared memory: [token 16][row 32] floats with a token pitch of 36 (the writes of a
// warp's 8 x 4 lanes hit distinct banks, a lane's 32 rows read as 8 x 16 bytes) and 16 floats of padding per warp so
// the two row groups' readers do not share banks.
constexpr int kRedTokPitch = 36, kRedWarpFloats = 16 * kRedTokPitch + 16;
constexpr uint32_t kXsbBytes = kTokens * 256 * 2;  // fp16 activations of one super-block
constexpr uint32_t kSxSbBytes = 512;               // hi/lo sub-block sums of one super-block

struct LinearMaps {
  CUtensorMap m[2][8];  // [tensor: weights / weights2][row residue]
};

struct LinearParams {
  const uint8_t *w, *w2, *prepared;
  const uint16_t *aux;
  void *out;
  float *partials;
  uint32_t *counters, *status;
  uint32_t n, k, rows, aux_stride, out_stride, epilogue, out_f32;
  uint32_t nsb, slices, tiles, stages, row_bytes, pitch, stage_bytes;
  // Tiled-TMA geometry. A tensor's rows are served by `period` maps, map j holding rows = j (mod
  // period) so that every map's row stride is a multiple of 16 bytes; a stage is `pieces` column
  // pieces of `piece_sb` super-blocks, each piece one box per (tensor, map): box_rows x pitch bytes.
  uint32_t period, period_log2, pieces, piece_sb, box_rows, box_bytes, tensors;
  uint32_t lead[2][8];  // bytes between map j's 16-byte aligned base and its first row's first byte
  uint32_t x_off, red_off, ring_off;  // shared memory offsets
  uint32_t debug;
};

template <int FMT> struct WFmt;
// kSbBytes: bytes of 256 weights; kPieceSb: super-blocks per TMA column piece of a stage; kKG: k-group warps per
// row group (consumer warps = kRG * kKG: Q4_K gains from three per scheduler, Q6_K runs best with two).
template <> struct WFmt<SB_FMT_Q4K> { static constexpr uint32_t kSbBytes = 144, kPieceSb = 1; static constexpr bool kPairLayout = true; static constexpr int kKG = 6; };
template <> struct WFmt<SB_FMT_Q6K> { static constexpr uint32_t kSbBytes = 210, kPieceSb = 4; static constexpr bool kPairLayout = false; static constexpr int kKG = 4; };
template <> struct WFmt<SB_FMT_Q80> { static constexpr uint32_t kSbBytes = 272, kPieceSb = 2; static constexpr bool kPairLayout = false; static constexpr int kKG = 4; };

__device__ __forceinline__ void slice_range(uint32_t nsb, uint32_t slices, uint32_t s, uint32_t &b0, uint32_t &b1) {
  b0 = s * nsb / slices;
  b1 = (s + 1) * nsb / slices;
}

// ---- prepared activations ----
// The product reads its activations as fp16 MMA fragments, so they are converted once per
// projection input, not once per CTA: sb_linear_prepare writes, for all 16 row slots,
//   header   64 bytes: scale_back[16] floats, 2^e of each row's power-of-two scale
//   per super-block of 256 inputs, 8704 bytes:
//     8192 bytes of 16-byte units, one per (MMA step, token half, lane): 8 consecutive inputs of
//                one token in the order [0,2,1,3,4,6,5,7], scaled by 2^-e and rounded to fp16
//                (exact for bf16 inputs down to 2^-27 of the row's largest magnitude)
//      512 bytes of sub-block sums (32 inputs), each split into hi + lo halves, for the mins' MMA
// Unit order within a super-block, for lane L = 4 g + t holding token 8 h + g:
//   pair layout  (Q4_K: lane t multiplies sub-blocks 2t, 2t+1):   (((i2*2 + p)*2 + h)*32 + L), inputs
//                32 (2t + p) + 8 i2 .. + 7
//   range layout (Q6_K, Q8_0: lane t multiplies inputs 8t..8t+7 of every group j): ((j*2 + h)*32 + L)
// This mirrors the reference's prepared input (ops::LinearBuffers::prepared, PreparedInput of
// runtime/ops/Linear.hpp:265-347; kernel decode_linear_gguf_prepare of
// runtime/metal/kernels/decode/linear_gguf_sgmatrix.metal). An optional RMSNorm is fused in front:
// y = bf16((x * rsqrt(mean x^2 + 1e-6)) * w) (runtime/metal/kernels/shared/normalization.metal:60-94).
static_assert(kPrepSbBytes == kXsbBytes + kSxSbBytes, "prepared super-block size");
constexpr int kPrepThreads = 256;
constexpr int kPrepCluster = 8;    // CTAs per row: a thread-block cluster shares the row's sum of squares and maximum
constexpr int kPrepMaxChunks = 2;  // 8-element chunks a thread keeps in registers: k <= 8 * 2 * 256 * 8 = 32768

struct PrepareParams {
  const uint16_t *x;
  const float *norm_w;
  uint8_t *out;
  uint16_t *normed_out;  // optional bf16 [rows][k]: the (normalised) input as the product's fp32 side projections read it
  uint32_t rows, k, x_stride, pair_layout;  // layout: 0 range, 1 pair, 2 tensor-core tiles
  // Optional: x = bf16(residual + the slices' partial sums), also written to sum_out (see sb_linear_prepare_sum).
  const float *partials;
  uint16_t *sum_out;
  uint32_t partial_slices, partial_stride, sum_stride;
  uint32_t swiglu_n;  // non-zero: x = bf16(bf16(up) * silu(bf16(gate))) of the slices' sums at columns c (gate) and swiglu_n + c (up); no residual
  // Optional (tensor parallelism): the slices' sum is one rank's share; the ranks exchange their shares through each
  // other's memory and add them in rank order before the residual (sb_tp_internal.cuh).
  TpExchange tp;
};

// Sum of `s` and maximum of `m` over the block, both returned to every thread. Fixed order: butterfly within
// each warp, then the warps' values in index order.
__device__ __forceinline__ void block_reduce2(float &s, float &m, float *scratch) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  }
  if ((threadIdx.x & 31) == 0) {
    scratch[2 * (threadIdx.x >> 5)] = s;
    scratch[2 * (threadIdx.x >> 5) + 1] = m;
  }
  __syncthreads();
  s = scratch[0], m = scratch[1];
  for (int w = 1; w < kPrepThreads / 32; ++w) {
    s += scratch[2 * w];
    m = fmaxf(m, scratch[2 * w + 1]);
  }
}

// Where chunk c (8 values = 4 units) of a row starts in an inbox matrix: a warp's 32 chunks are 128 units in a row, and
// unit u of lane l sits at 32 u + l of them, so each of the warp's four stores (and loads) covers 512 consecutive bytes.
__device__ __forceinline__ size_t tp_unit(size_t matrix, uint32_t tok, uint32_t width, uint32_t c, uint32_t lane) {
  return ((matrix * kTokens + tok) * width + 8 * (c - lane)) / 2 + lane;
}

// Where chunk c's two units of finished sums (8 bf16) start in the second inbox, laid out like tp_unit.
__device__ __forceinline__ size_t tp_sum_unit(uint32_t slot, uint32_t tok, uint32_t width, uint32_t c, uint32_t lane) {
  return ((size_t(slot) * kTokens + tok) * width + 8 * (c - lane)) / 4 + lane;
}
// The rank that owns super-block sb of the row: contiguous ranges.
__device__ __forceinline__ uint32_t tp_owner(uint32_t sb, uint32_t nsb, uint32_t world) { return sb * world / nsb; }

// Polls `count` units 32 apart until all show `epoch`; gives up after the bounded wait (expired stays set).
template <int N>
__device__ __forceinline__ void tp_poll_units(const uint4 *from, uint4 (&got)[N], uint32_t epoch, uint64_t t0, bool &expired, uint32_t *status, uint64_t wait_ns) {
  for (uint32_t polls = 1;; ++polls) {
    bool all = true;
#pragma unroll
    for (int u = 0; u < N; ++u) {
      got[u] = tp_load_unit(from + 32 * u);
      all = all && got[u].y == epoch && got[u].w == epoch;
    }
    if (all || expired) return;
    if ((polls & 63u) == 0 && (global_timer_ns() - t0 > wait_ns || polls >= (1u << 30))) {
      atomicCAS(status, uint32_t(SB_DEV_OK), uint32_t(SB_DEV_WAIT_EXPIRED));
      expired = true;
    }
  }
}

// This rank's share of a sum (its k-slices added in order) on its way to the other ranks; the same grid and the same
// thread-to-element map as prepare_kernel (sb_tp_internal.cuh). One shot: into every peer's inbox. Two shots: to the
// columns' owner; the owner's threads add the shares in rank order, add the residual, round, and send the finished
// values to every rank.
__global__ void __launch_bounds__(kPrepThreads) tp_push_kernel(const PrepareParams p) {
  const uint32_t tok = blockIdx.x / kPrepCluster, rank = blockIdx.x % kPrepCluster, tid = threadIdx.x, lane = tid & 31;
  const uint32_t nsb = p.k / 256, c0 = rank * nsb / kPrepCluster * 32, chunks = (rank + 1) * nsb / kPrepCluster * 32;
  const TpExchange &x = p.tp;
  pdl_launch_dependents();
  pdl_wait();  // the projection that wrote the slices has completed
  const uint32_t epoch = tp_epoch(x);
  const bool healthy = tp_healthy(x);
  if (blockIdx.x == 0 && tid == 0) st_release_gpu(x.ready, epoch);
  if (tok >= p.rows) return;
  const size_t slot = size_t(epoch & 1u) * x.world;
  float own[kPrepMaxChunks][8];
  bool owned[kPrepMaxChunks];
#pragma unroll
  for (int i = 0; i < kPrepMaxChunks; ++i) {
    const uint32_t c = c0 + tid + kPrepThreads * i;
    owned[i] = false;
    if (c >= chunks) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t s0 = 0; s0 < p.partial_slices; s0 += 8) {  // the order and grouping of prepare_kernel's own sum
      float4 a4[8], b4[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sl = min(s0 + j, p.partial_slices - 1);
        const float4 *pp = reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * p.partial_stride + 8 * c);
        a4[j] = __ldcg(pp), b4[j] = __ldcg(pp + 1);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < p.partial_slices)
          acc[0] += a4[j].x, acc[1] += a4[j].y, acc[2] += a4[j].z, acc[3] += a4[j].w, acc[4] += b4[j].x, acc[5] += b4[j].y, acc[6] += b4[j].z,
              acc[7] += b4[j].w;
    }
    const size_t unit = tp_unit(slot + x.rank, tok, x.width, c, lane);
    const uint32_t owner = tp_owner(c >> 5, nsb, x.world);
    for (uint32_t peer = 0; peer < x.world; ++peer) {
      if (peer == x.rank || (x.two_shot && peer != owner)) continue;
      uint4 *dst = reinterpret_cast<uint4 *>(x.data[peer]) + unit;
#pragma unroll
      for (int u = 0; u < 4; ++u) tp_store_unit(dst + 32 * u, acc[2 * u], acc[2 * u + 1], epoch);
    }
    owned[i] = x.two_shot && owner == x.rank;
#pragma unroll
    for (int j = 0; j < 8; ++j) own[i][j] = acc[j];
  }
  if (!x.two_shot) return;
  const uint64_t t0 = global_timer_ns();
  bool expired = !healthy;
#pragma unroll
  for (int i = 0; i < kPrepMaxChunks; ++i) {
    const uint32_t c = c0 + tid + kPrepThreads * i;
    if (!owned[i]) continue;
    const uint4 raw = *reinterpret_cast<const uint4 *>(p.x + size_t(tok) * p.x_stride + 8 * c);  // the residual
    float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t src = 0; src < x.world; ++src) {
      if (src == x.rank) {
#pragma unroll
        for (int j = 0; j < 8; ++j) total[j] += own[i][j];
        continue;
      }
      uint4 got[4];
      tp_poll_units<4>(reinterpret_cast<const uint4 *>(x.data[x.rank]) + tp_unit(slot + src, tok, x.width, c, lane), got, epoch, t0, expired, x.status, x.wait_ns);
#pragma unroll
      for (int u = 0; u < 4; ++u) total[2 * u] += __uint_as_float(got[u].x), total[2 * u + 1] += __uint_as_float(got[u].z);
    }
    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t pk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = round_bf16(total[2 * j] + bf16_bits_to_float(r[j] & 0xffffu)), hi = round_bf16(total[2 * j + 1] + bf16_bits_to_float(r[j] >> 16));
      pk[j] = uint32_t(float_to_bf16_bits(lo)) | (uint32_t(float_to_bf16_bits(hi)) << 16);
    }
    const size_t sunit = tp_sum_unit(epoch & 1u, tok, x.width, c, lane);
    for (uint32_t peer = 0; peer < x.world; ++peer) {
      uint4 *dst = x.sums[peer] + sunit;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(pk[0]), "r"(epoch), "r"(pk[1]), "r"(epoch) : "memory");
      asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 32), "r"(pk[2]), "r"(epoch), "r"(pk[3]), "r"(epoch) : "memory");
    }
  }
}

template <bool TP> __global__ void __launch_bounds__(kPrepThreads) prepare_kernel(const PrepareParams p) {
  __shared__ float scratch[2 * (kPrepThreads / 32)];
  __shared__ float cluster_part[kPrepCluster][2];  // every CTA of the row stores its sum of squares and maximum here
  // A row is shared by the kPrepCluster CTAs of a cluster: CTA `rank` converts whole super-blocks
  // [rank nsb / C, (rank + 1) nsb / C) and the row's statistics meet through distributed shared memory.
  const uint32_t tok = blockIdx.x / kPrepCluster, rank = blockIdx.x % kPrepCluster, tid = threadIdx.x, lane = tid & 31;
  const bool live = tok < p.rows;
  const uint32_t nsb = p.k / 256, c0 = rank * nsb / kPrepCluster * 32, chunks = (rank + 1) * nsb / kPrepCluster * 32;
  pdl_launch_dependents();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // "this CTA runs": waited for before the statistics' exchange
  // The norm weights do not depend on the previous kernel: they are fetched before the dependency wait.
  float wn[kPrepMaxChunks][8];
  if (p.norm_w) {
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i) {
      const uint32_t c = c0 + tid + kPrepThreads * i;
      float4 w0 = make_float4(0, 0, 0, 0), w1 = w0;
      if (c < chunks) {
        w0 = *reinterpret_cast<const float4 *>(p.norm_w + 8 * c);
        w1 = *reinterpret_cast<const float4 *>(p.norm_w + 8 * c + 4);
      }
      wn[i][0] = w0.x, wn[i][1] = w0.y, wn[i][2] = w0.z, wn[i][3] = w0.w;
      wn[i][4] = w1.x, wn[i][5] = w1.y, wn[i][6] = w1.z, wn[i][7] = w1.w;
    }
  }
  // The conversion of an exchange does not wait for the kernel before it (the push kernel, whose completion includes
  // the flush of its stores to the peers) but for that kernel's word that the slices' sums are complete.
  uint32_t epoch = 0;
  bool healthy = true;
  if (TP) {
    epoch = tp_epoch(p.tp), healthy = tp_healthy(p.tp);
    if (healthy && !p.tp.two_shot) healthy = tp_wait_ready(p.tp, epoch);  // (two shots: everything arrives as finished sums)
  } else {
    pdl_wait();
  }
  float v[kPrepMaxChunks][8];
  float acc[kPrepMaxChunks][8];
  const uint16_t *row = p.x + size_t(tok) * p.x_stride;
#pragma unroll
  for (int i = 0; i < kPrepMaxChunks; ++i) {
    const uint32_t c = c0 + tid + kPrepThreads * i;
    uint4 raw = make_uint4(0, 0, 0, 0);
    const bool finished = TP && p.tp.two_shot;  // the values arrive whole (below): no residual, no slices to add here
    if (live && c < chunks && !p.swiglu_n && !finished) raw = *reinterpret_cast<const uint4 *>(row + 8 * c);
    const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[i][2 * j] = bf16_bits_to_float(u[j] & 0xffffu);
      v[i][2 * j + 1] = bf16_bits_to_float(u[j] >> 16);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    if (p.swiglu_n && live && c < chunks) {
      // x = bf16(bf16(up) * silu(bf16(gate))) of the slices' gate and up sums (added in slice order): the one-pass
      // SwiGLU epilogue of the projection pair, done here.
      float up[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (uint32_t s0 = 0; s0 < p.partial_slices; s0 += 2) {  // two slices' loads in flight
        float4 g4[2][2], u4[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint32_t sl = min(s0 + j, p.partial_slices - 1);
          const float4 *pg = reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * p.partial_stride + 8 * c);
          const float4 *pu = reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * p.partial_stride + p.swiglu_n + 8 * c);
          g4[j][0] = __ldcg(pg), g4[j][1] = __ldcg(pg + 1), u4[j][0] = __ldcg(pu), u4[j][1] = __ldcg(pu + 1);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (s0 + j < p.partial_slices) {
            acc[i][0] += g4[j][0].x, acc[i][1] += g4[j][0].y, acc[i][2] += g4[j][0].z, acc[i][3] += g4[j][0].w;
            acc[i][4] += g4[j][1].x, acc[i][5] += g4[j][1].y, acc[i][6] += g4[j][1].z, acc[i][7] += g4[j][1].w;
            up[0] += u4[j][0].x, up[1] += u4[j][0].y, up[2] += u4[j][0].z, up[3] += u4[j][0].w;
            up[4] += u4[j][1].x, up[5] += u4[j][1].y, up[6] += u4[j][1].z, up[7] += u4[j][1].w;
          }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = round_bf16(round_bf16(up[j]) * silu_f(round_bf16(acc[i][j])));
    } else if (p.partials && live && c < chunks && !finished) {
      // The sum of the slices in order: with the residual below, the projection's residual epilogue, done here.
      for (uint32_t s0 = 0; s0 < p.partial_slices; s0 += 8) {  // eight slices' loads in flight, added in slice order
        float4 a4[8], b4[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t sl = min(s0 + j, p.partial_slices - 1);
          const float4 *pp = reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * p.partial_stride + 8 * c);
          a4[j] = __ldcg(pp), b4[j] = __ldcg(pp + 1);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (s0 + j < p.partial_slices)
            acc[i][0] += a4[j].x, acc[i][1] += a4[j].y, acc[i][2] += a4[j].z, acc[i][3] += a4[j].w, acc[i][4] += b4[j].x,
                acc[i][5] += b4[j].y, acc[i][6] += b4[j].z, acc[i][7] += b4[j].w;
      }
    }
  }
  if (TP && live && p.tp.two_shot) {
    // The finished values of every column arrive from their owners (tp_push_kernel on their side, this rank's included).
    const TpExchange &x = p.tp;
    const uint64_t t0 = global_timer_ns();
    bool expired = !healthy;
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i) {
      const uint32_t c = c0 + tid + kPrepThreads * i;
      if (c >= chunks) continue;
      uint4 got[2];
      tp_poll_units<2>(x.sums[x.rank] + tp_sum_unit(epoch & 1u, tok, x.width, c, lane), got, epoch, t0, expired, x.status, x.wait_ns);
      const uint32_t u[4] = {got[0].x, got[0].z, got[1].x, got[1].z};
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][2 * j] = bf16_bits_to_float(u[j] & 0xffffu), acc[i][2 * j + 1] = bf16_bits_to_float(u[j] >> 16);
    }
  } else if (TP && live) {
    // The peers' shares arrive in this rank's inbox (tp_push_kernel on their side). The sum over the ranks runs in
    // rank order on every rank, so all ranks hold the same bits afterwards.
    const TpExchange &x = p.tp;
    const size_t slot = size_t(epoch & 1u) * x.world;
    const uint64_t t0 = global_timer_ns();
    bool expired = !healthy;
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i) {
      const uint32_t c = c0 + tid + kPrepThreads * i;
      if (c >= chunks) continue;
      float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (uint32_t src = 0; src < x.world; ++src) {
        if (src == x.rank) {
#pragma unroll
          for (int j = 0; j < 8; ++j) total[j] += acc[i][j];
          continue;
        }
        uint4 got[4];
        tp_poll_units<4>(reinterpret_cast<const uint4 *>(x.data[x.rank]) + tp_unit(slot + src, tok, x.width, c, lane), got, epoch, t0, expired, x.status, x.wait_ns);
#pragma unroll
        for (int u = 0; u < 4; ++u) total[2 * u] += __uint_as_float(got[u].x), total[2 * u + 1] += __uint_as_float(got[u].z);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = total[j];
    }
  }
  if (p.partials && live) {
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i) {
      const uint32_t c = c0 + tid + kPrepThreads * i;
      if (c >= chunks) continue;
      uint32_t pk[4];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = (p.swiglu_n || (TP && p.tp.two_shot)) ? acc[i][j] : round_bf16(acc[i][j] + v[i][j]);
#pragma unroll
      for (int j = 0; j < 4; ++j) pk[j] = uint32_t(float_to_bf16_bits(v[i][2 * j])) | (uint32_t(float_to_bf16_bits(v[i][2 * j + 1])) << 16);
      *reinterpret_cast<uint4 *>(p.sum_out + size_t(tok) * p.sum_stride + 8 * c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
  // One pass of block reductions gives both the sum of squares and the largest |x * w| (or |x| without a
  // norm): the largest normalised magnitude is then inv * that, up to the bf16 rounding allowed for below.
  float ss = 0.0f, mx = 0.0f;
#pragma unroll
  for (int i = 0; i < kPrepMaxChunks; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ss = fmaf(v[i][j], v[i][j], ss);
      mx = fmaxf(mx, fabsf(p.norm_w ? v[i][j] * wn[i][j] : v[i][j]));  // NaN does not win a max; it stays in the values
    }
  block_reduce2(ss, mx, scratch);
  {
    // The row's statistics: every CTA stores its own into all eight CTAs' shared memory, one cluster barrier, then
    // each adds its local copies in rank order. (The barrier that makes sure every CTA of the cluster runs before
    // anyone writes into it was arrived at when the kernel started, long before this point.)
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < kPrepCluster) {
      float *remote = cluster.map_shared_rank(&cluster_part[0][0], tid);
      remote[2 * rank] = ss, remote[2 * rank + 1] = mx;
    }
    cluster.sync();
    float ss_all = 0.0f, mx_all = 0.0f;
#pragma unroll
    for (int r = 0; r < kPrepCluster; ++r) {
      ss_all += cluster_part[r][0];
      mx_all = fmaxf(mx_all, cluster_part[r][1]);
    }
    ss = ss_all, mx = mx_all;
  }
  if (p.norm_w) {
    const float inv = rsqrtf(ss / float(p.k) + 1e-6f);
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = round_bf16((v[i][j] * inv) * wn[i][j]);
    mx = mx * inv * 1.0625f;  // (x inv) w against x w inv and the rounding to bf16: well inside 6 %
  }
  if (p.normed_out && live) {
#pragma unroll
    for (int i = 0; i < kPrepMaxChunks; ++i) {
      const uint32_t c = c0 + tid + kPrepThreads * i;
      if (c < chunks) {
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          pk[j] = uint32_t(float_to_bf16_bits(v[i][2 * j])) | (uint32_t(float_to_bf16_bits(v[i][2 * j + 1])) << 16);
        *reinterpret_cast<uint4 *>(p.normed_out + size_t(tok) * p.k + 8 * c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
  }
  int e = 0;
  if (mx > 0.0f && mx <= 3.0e38f) {
    (void)frexpf(mx, &e);  // mx = f * 2^e with f in [0.5, 1): scaled values stay below 2^10
    e -= 10;
  }
  const float down = ldexpf(1.0f, -e);
  if (tid == 0 && rank == 0) reinterpret_cast<float *>(p.out)[tok] = ldexpf(1.0f, e);
  const uint32_t h = tok >> 3, g = tok & 7;
#pragma unroll
  for (int i = 0; i < kPrepMaxChunks; ++i) {
    const uint32_t c = c0 + tid + kPrepThreads * i;  // chunk c = inputs 8c..8c+7; 32 consecutive chunks = one super-block
    if (c >= chunks) continue;                  // uniform per warp: chunks is a multiple of 32
    const uint32_t sb = c >> 5, j = lane >> 2, q = lane & 3;
    __half hv[8];
    float sum = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      hv[jj] = __float2half_rn(v[i][jj] * down);
      sum += __half2float(hv[jj]);
    }
    uint32_t unit = 0;
    if (p.pair_layout == 1) unit = (((q * 2 + (j & 1)) * 2 + h) * 8 + g) * 4 + (j >> 1);
    else if (p.pair_layout == 0) unit = ((j * 2 + h) * 8 + g) * 4 + q;
    const __half2 p0 = __halves2half2(hv[0], hv[2]), p1 = __halves2half2(hv[1], hv[3]);
    const __half2 p2 = __halves2half2(hv[4], hv[6]), p3 = __halves2half2(hv[5], hv[7]);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t *>(&p0);
    o.y = *reinterpret_cast<const uint32_t *>(&p1);
    o.z = *reinterpret_cast<const uint32_t *>(&p2);
    o.w = *reinterpret_cast<const uint32_t *>(&p3);
    uint8_t *sbp = p.out + kPrepHeader + size_t(sb) * kPrepSbBytes;
    if (p.pair_layout == 2) {
      // Tensor-core operand layout: 16 K-major tiles of 16 inputs x 16 tokens, each [token / 8][input / 8]
      // [token % 8][8 halves]. The inputs of a tile follow the order in which the Q4_K kernel unpacks a
      // row's nibbles: chunk (pair lane / 8, sub-block parity (lane / 4) % 2, quarter lane % 4) fills
      // inputs 4 parity .. + 3 of both halves of tile 4 pair + quarter.
      const uint32_t pair = lane >> 3, parity = (lane >> 2) & 1, quarter = lane & 3;
      uint8_t *tile = sbp + (4 * pair + quarter) * 512 + h * 256 + g * 16 + 8 * parity;
      *reinterpret_cast<uint2 *>(tile) = make_uint2(o.x, o.y);
      *reinterpret_cast<uint2 *>(tile + 128) = make_uint2(o.z, o.w);
    } else {
      *reinterpret_cast<uint4 *>(sbp + size_t(unit) * 16) = o;
    }
    // Sub-block sums: 32 inputs = 4 consecutive lanes.
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (q == 0) {
      const __half hi = __float2half_rn(sum);
      const __half lo = __float2half_rn(sum - __half2float(hi));
      __half *sx = reinterpret_cast<__half *>(sbp + kXsbBytes);
      if (p.pair_layout == 2) {
        // The 17th tile: input j = high part, input 8 + j = low part of sub-block j's sum.
        const uint32_t at = h * 128 + g * 8 + j;
        sx[at] = hi;
        sx[at + 64] = lo;
      } else {
        const uint32_t at = ((h * 8 + g) * 4 + (j >> 1)) * 4 + (j & 1) * 2;
        sx[at] = hi;
        sx[at + 1] = lo;
      }
    }
  }
}

// ---- per-format multiply of one super-block for kMT m-tiles of 16 rows ----
struct Q4Scales {
  uint32_t mlo, blo, mhi, bhi, mn0, mn1;
  float d, ndmin;
};
// The two sub-blocks (2t, 2t+1) a lane multiplies, from a super-block's 16-byte header
// {d, dmin, 12 packed 6-bit scale/min bytes}.
__device__ __forceinline__ Q4Scales q4_scales(const uint4 hdr, uint32_t t) {
  const uint32_t sh = (t & 1) * 16;
  const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, c = hdr.w >> sh;
  const uint32_t sc_lo = a & 0x3f3fu, mn_lo = b & 0x3f3fu;
  const uint32_t sc_hi = (c & 0x0f0fu) | ((a >> 2) & 0x3030u), mn_hi = ((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u);
  const uint32_t sc = t < 2 ? sc_lo : sc_hi, mn = t < 2 ? mn_lo : mn_hi;
  const uint32_t k1024 = 0x64006400u;
  // {0x6400 | byte, 0x6400 | byte} - 1024 = the byte as two exact halves.
  const uint32_t s0 = hsub2_u32(__byte_perm(sc, 0x64646464u, 0x4040), k1024);
  const uint32_t s1 = hsub2_u32(__byte_perm(sc, 0x64646464u, 0x4141), k1024);
  Q4Scales r;
  r.mn0 = hsub2_u32(__byte_perm(mn, 0x64646464u, 0x4040), k1024);
  r.mn1 = hsub2_u32(__byte_perm(mn, 0x64646464u, 0x4141), k1024);
  r.mlo = s0;
  r.blo = hmul2_u32(s0, 0xE400E400u);  // * -1024
  r.mhi = hmul2_u32(s1, 0x2C002C00u);  // * 1/16
  r.bhi = hmul2_u32(s1, 0xD400D400u);  // * -64
  const __half2 dd = *reinterpret_cast<const __half2 *>(&hdr.x);
  r.d = __low2float(dd);
  r.ndmin = -__high2float(dd);
  return r;
}

template <int NMT>
__device__ __forceinline__ void mul_q4k(const uint8_t *wbase, const uint32_t (*roff)[2], const uint8_t *xs_sb,
                                        const uint8_t *sx_sb, uint32_t lane, float (*y)[2][4]) {
  const uint32_t t = lane & 3;
  Q4Scales sc[NMT][2];
  const uint8_t *qrow[NMT][2];
#pragma unroll
  for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint8_t *row = wbase + roff[mt][r];
      sc[mt][r] = q4_scales(*reinterpret_cast<const uint4 *>(row), t);
      qrow[mt][r] = row + 16 + 32 * t;
    }
  float aq[NMT][2][4];
#pragma unroll
  for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 4; ++c) aq[mt][h][c] = 0.0f;
  const uint32_t kMagic = 0x64006400u;
  SB_UNROLL_Q4K_I2
  for (int i2 = 0; i2 < 4; ++i2) {
    uint4 bx[2][2];
#pragma unroll
    for (int p = 0; p < 2; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        bx[p][h] = *reinterpret_cast<const uint4 *>(xs_sb + ((((i2 * 2 + p) * 2 + h) * 32 + lane) << 4));
    uint2 qw[NMT][2];
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
      for (int r = 0; r < 2; ++r) qw[mt][r] = *reinterpret_cast<const uint2 *>(qrow[mt][r] + 8 * i2);
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
      for (int wi = 0; wi < 2; ++wi) {
        const uint32_t w0 = wi ? qw[mt][0].y : qw[mt][0].x, w1 = wi ? qw[mt][1].y : qw[mt][1].x;
        const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
        {
          const uint32_t a0 = hfma2_u32(and_or(w0, 0x000f000fu, kMagic), sc[mt][0].mlo, sc[mt][0].blo);
          const uint32_t a1 = hfma2_u32(and_or(w1, 0x000f000fu, kMagic), sc[mt][1].mlo, sc[mt][1].blo);
          const uint32_t a2 = hfma2_u32(and_or(w0s, 0x000f000fu, kMagic), sc[mt][0].mlo, sc[mt][0].blo);
          const uint32_t a3 = hfma2_u32(and_or(w1s, 0x000f000fu, kMagic), sc[mt][1].mlo, sc[mt][1].blo);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            mma_f16(aq[mt][h], a0, a1, a2, a3, wi ? bx[0][h].z : bx[0][h].x, wi ? bx[0][h].w : bx[0][h].y);
        }
        {
          const uint32_t a0 = hfma2_u32(and_or(w0, 0x00f000f0u, kMagic), sc[mt][0].mhi, sc[mt][0].bhi);
          const uint32_t a1 = hfma2_u32(and_or(w1, 0x00f000f0u, kMagic), sc[mt][1].mhi, sc[mt][1].bhi);
          const uint32_t a2 = hfma2_u32(and_or(w0s, 0x00f000f0u, kMagic), sc[mt][0].mhi, sc[mt][0].bhi);
          const uint32_t a3 = hfma2_u32(and_or(w1s, 0x00f000f0u, kMagic), sc[mt][1].mhi, sc[mt][1].bhi);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            mma_f16(aq[mt][h], a0, a1, a2, a3, wi ? bx[1][h].z : bx[1][h].x, wi ? bx[1][h].w : bx[1][h].y);
        }
      }
  }
  // Mins against the sub-block sums, then the super-block's two floating scales.
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint2 s = *reinterpret_cast<const uint2 *>(sx_sb + ((h * 32 + lane) << 3));
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      float am[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      mma_f16(am, sc[mt][0].mn0, sc[mt][1].mn0, sc[mt][0].mn1, sc[mt][1].mn1, s.x, s.y);
      y[mt][h][0] = fmaf(sc[mt][0].ndmin, am[0], fmaf(sc[mt][0].d, aq[mt][h][0], y[mt][h][0]));
      y[mt][h][1] = fmaf(sc[mt][0].ndmin, am[1], fmaf(sc[mt][0].d, aq[mt][h][1], y[mt][h][1]));
      y[mt][h][2] = fmaf(sc[mt][1].ndmin, am[2], fmaf(sc[mt][1].d, aq[mt][h][2], y[mt][h][2]));
      y[mt][h][3] = fmaf(sc[mt][1].ndmin, am[3], fmaf(sc[mt][1].d, aq[mt][h][3], y[mt][h][3]));
    }
  }
}

// Bytes [at, at + 8) of shared memory at any 2-byte alignment, as two words.
__device__ __forceinline__ uint2 lds8_unaligned(const uint8_t *base, uint32_t at) {
  const uint32_t *w = reinterpret_cast<const uint32_t *>(base + (at & ~3u));
  const uint32_t sh = (at & 3u) * 8;
  const uint32_t a = w[0], b = w[1], c = w[2];
  return make_uint2(__funnelshift_r(a, b, sh), __funnelshift_r(b, c, sh));
}
__device__ __forceinline__ uint32_t lds2_unaligned(const uint8_t *base, uint32_t at) {
  return *reinterpret_cast<const uint16_t *>(base + at);
}

template <int NMT>
__device__ __forceinline__ void mul_q6k(const uint8_t *wbase, const uint32_t (*roff)[2], const uint8_t *xs_sb,
                                        const uint8_t *, uint32_t lane, float (*y)[2][4]) {
  // Lane t of a row multiplies inputs 8t..8t+7 of each of the 8 groups of 32: for half n of the
  // block, ql[64n+8t..] (groups 4n, 4n+2 in its nibbles), ql[64n+32+8t..] (4n+1, 4n+3) and
  // qh[32n+8t..] (two bits per group). The 6-bit code lands in bits 4..9 of a half whose value is
  // 64 + code/... : 0x5400 | code << 4 = 64 + code, so (64 + code) * sc - 96 * sc = sc * (code - 32).
  const uint32_t t = lane & 3;
  const uint32_t kMagic = 0x54005400u, kLow = 0x00f000f0u, kHigh = 0x03000300u;
  float aq[NMT][2][4];
#pragma unroll
  for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 4; ++c) aq[mt][h][c] = 0.0f;
  float dscale[NMT][2];
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    uint2 qa[NMT][2], qb[NMT][2], qh[NMT][2];
    uint32_t ms[NMT][2][4], bs[NMT][2][4];
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t at = roff[mt][r];
        qa[mt][r] = lds8_unaligned(wbase, at + 64 * n + 8 * t);
        qb[mt][r] = lds8_unaligned(wbase, at + 64 * n + 32 + 8 * t);
        qh[mt][r] = lds8_unaligned(wbase, at + 128 + 32 * n + 8 * t);
        if (n == 0) {
          const __half dh = __ushort_as_half(uint16_t(lds2_unaligned(wbase, at + 208)));
          dscale[mt][r] = __half2float(dh);
        }
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          // int8 scale of group 4n+rr for inputs 8t..8t+7: index 8n + 2rr + (t >> 1).
          const uint32_t sat = at + 192 + 8 * n + 2 * rr + (t >> 1);
          const int sv = int(int8_t(wbase[sat]));
          const __half2 s2 = __half2half2(__int2half_rn(sv));
          ms[mt][r][rr] = *reinterpret_cast<const uint32_t *>(&s2);
          bs[mt][r][rr] = hmul2_u32(ms[mt][r][rr], 0xD600D600u);  // * -96
        }
      }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int j = 4 * n + rr;
      uint4 bx[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) bx[h] = *reinterpret_cast<const uint4 *>(xs_sb + (((j * 2 + h) * 32 + lane) << 4));
#pragma unroll
      for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
        for (int wi = 0; wi < 2; ++wi) {
          uint32_t a[2][2];  // [row][pair]: pair 0 = inputs (0,2), pair 1 = inputs (1,3) of the word
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t lw = (rr & 1) ? (wi ? qb[mt][r].y : qb[mt][r].x) : (wi ? qa[mt][r].y : qa[mt][r].x);
            const uint32_t hw = wi ? qh[mt][r].y : qh[mt][r].x;
            // nibbles: groups 4n, 4n+1 use the low nibble, 4n+2, 4n+3 the high one
            const uint32_t l02 = (rr & 2) ? (lw & kLow) : ((lw << 4) & kLow);
            const uint32_t l13 = (rr & 2) ? ((lw >> 8) & kLow) : ((lw >> 4) & kLow);
            // high bits of bytes 0,2 sit at bits 2rr..2rr+1 (+16); of bytes 1,3 at 8+2rr (+16)
            const uint32_t h02 = rr == 0 ? (hw << 8) : rr == 1 ? (hw << 6) : rr == 2 ? (hw << 4) : (hw << 2);
            const uint32_t h13 = rr == 0 ? hw : rr == 1 ? (hw >> 2) : rr == 2 ? (hw >> 4) : (hw >> 6);
            a[r][0] = hfma2_u32(and_or(h02, kHigh, l02 | kMagic), ms[mt][r][rr], bs[mt][r][rr]);
            a[r][1] = hfma2_u32(and_or(h13, kHigh, l13 | kMagic), ms[mt][r][rr], bs[mt][r][rr]);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h)
            mma_f16(aq[mt][h], a[0][0], a[1][0], a[0][1], a[1][1], wi ? bx[h].z : bx[h].x, wi ? bx[h].w : bx[h].y);
        }
    }
  }
#pragma unroll
  for (int mt = 0; mt < NMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      y[mt][h][0] = fmaf(dscale[mt][0], aq[mt][h][0], y[mt][h][0]);
      y[mt][h][1] = fmaf(dscale[mt][0], aq[mt][h][1], y[mt][h][1]);
      y[mt][h][2] = fmaf(dscale[mt][1], aq[mt][h][2], y[mt][h][2]);
      y[mt][h][3] = fmaf(dscale[mt][1], aq[mt][h][3], y[mt][h][3]);
    }
}

template <int NMT>
__device__ __forceinline__ void mul_q80(const uint8_t *wbase, const uint32_t (*roff)[2], const uint8_t *xs_sb,
                                        const uint8_t *, uint32_t lane, float (*y)[2][4]) {
  // A "super-block" is 8 consecutive Q8_0 blocks {half d, 32 int8}. Lane t multiplies bytes
  // 8t..8t+7 of each block; the operand is fp16(d * q), the product rounded once.
  const uint32_t t = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 bx[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) bx[h] = *reinterpret_cast<const uint4 *>(xs_sb + (((j * 2 + h) * 32 + lane) << 4));
#pragma unroll
    for (int mt = 0; mt < NMT; ++mt) {
      uint2 qw[2];
      uint32_t d2[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t at = roff[mt][r] + 34 * j;
        const uint32_t dh = lds2_unaligned(wbase, at);
        d2[r] = dh | (dh << 16);
        qw[r] = lds8_unaligned(wbase, at + 2 + 8 * t);
      }
#pragma unroll
      for (int wi = 0; wi < 2; ++wi) {
        uint32_t a[2][2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t w = (wi ? qw[r].y : qw[r].x) ^ 0x80808080u;  // q + 128 as unsigned bytes
          const uint32_t u02 = __byte_perm(w, 0x64646464u, 0x4240), u13 = __byte_perm(w, 0x64646464u, 0x4341);
          a[r][0] = hmul2_u32(hsub2_u32(u02, 0x64806480u), d2[r]);  // (1024 + q + 128) - 1152 = q
          a[r][1] = hmul2_u32(hsub2_u32(u13, 0x64806480u), d2[r]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
          mma_f16(y[mt][h], a[0][0], a[1][0], a[0][1], a[1][1], wi ? bx[h].z : bx[h].x, wi ? bx[h].w : bx[h].y);
      }
    }
  }
}

template <int FMT, int NMT>
__device__ __forceinline__ void multiply_super_block(const uint8_t *wbase, const uint32_t (*roff)[2], const uint8_t *xs_sb,
                                                     const uint8_t *sx_sb, uint32_t lane, float (*y)[2][4]) {
  if (FMT == SB_FMT_Q4K) mul_q4k<NMT>(wbase, roff, xs_sb, sx_sb, lane, y);
  else if (FMT == SB_FMT_Q6K) mul_q6k<NMT>(wbase, roff, xs_sb, sx_sb, lane, y);
  else mul_q80<NMT>(wbase, roff, xs_sb, sx_sb, lane, y);
}

// ---- the kernel ----
// Barriers in shared memory: full[s] / empty[s] per ring stage, xfull (activations landed),
// red_full / red_empty (the tile's partial sums handed to the epilogue warp).
template <int FMT>
__global__ void __launch_bounds__(32 * (kRG * WFmt<FMT>::kKG + 1 + kEpiWarps), 1) linear_kernel(const LinearParams p, const __grid_constant__ LinearMaps maps) {
  constexpr int kKG = WFmt<FMT>::kKG, kConsumerWarps = kRG * kKG;  // + producer warp + the epilogue warps
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + kMaxStages;
  uint64_t *xfull = empty + kMaxStages;
  uint64_t *red_full = xfull + 1;               // [kEpiWarps], one per epilogue warp
  uint64_t *red_empty = red_full + kEpiWarps;   // [kEpiWarps]
  float *scale_back = reinterpret_cast<float *>(smem + 256);  // 16 floats, copied from the prepared header
  constexpr uint32_t kSb = WFmt<FMT>::kSbBytes;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t slice = blockIdx.x % p.slices;
  uint32_t sb0, sb1;
  slice_range(p.nsb, p.slices, slice, sb0, sb1);
  const uint32_t slice_sb = sb1 - sb0, chunks = (slice_sb + kStageSb - 1) / kStageSb;
  const uint32_t items = p.tiles * p.slices;
  const bool gate_up = p.epilogue == SB_EPILOGUE_GATE_UP || p.epilogue == SB_EPILOGUE_GATE_UP_PARTIALS;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    mbar_init(xfull, 1);
    for (int e = 0; e < kEpiWarps; ++e) {
      mbar_init(&red_full[e], kConsumerWarps);
      mbar_init(&red_empty[e], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kConsumerWarps) {
    // ---- producer ----
    // Weights do not depend on the previous kernel: the ring fills before the dependency wait; the
    // prepared activations are fetched after it.
    const uint64_t policy = policy_evict_first();
    uint32_t fill = 0;  // stages issued so far
    bool ok = true, x_issued = false;
    auto issue_x = [&] {
      pdl_wait();
      if (lane == 0) {
        const uint32_t bytes = slice_sb * kPrepSbBytes;
        mbar_arrive_expect_tx(xfull, bytes + kPrepHeader);
        bulk_g2s(scale_back, p.prepared, kPrepHeader, xfull);
        bulk_g2s(smem + p.x_off, p.prepared + kPrepHeader + size_t(sb0) * kPrepSbBytes, bytes, xfull);
      }
      x_issued = true;
    };
    // (Asking the L2 for later stages ahead of the ring, with TMA prefetches of the same boxes, was measured and
    // dropped: the gate/up launch went from 36 to 44 us at every distance tried. The 3-stage ring alone streams 6.6
    // TB/s when its stages are released at once; what it lacks is early release, not bytes in flight.)
    uint32_t slot = 0, round = 0;
    for (uint32_t item = blockIdx.x; item < items && ok && !SB_DBG(16); item += gridDim.x) {
      const uint32_t tile = item / p.slices;
      for (uint32_t c = 0; c < chunks && ok; ++c, ++fill) {
        if (round > 0) {
          if (!x_issued) issue_x();
          ok = SB_DBG(4) ? mbar_wait(&empty[slot], (round - 1) & 1) : mbar_wait_backoff(&empty[slot], (round - 1) & 1);
        }
        if (!ok) break;
        const uint32_t csb0 = sb0 + c * kStageSb, nsb_c = min(uint32_t(kStageSb), sb1 - csb0);
        // One box per (piece, tensor, row residue): lane = box index.
        const uint32_t pieces_c = (nsb_c + p.piece_sb - 1) / p.piece_sb;
        const uint32_t per_piece = p.tensors * p.period, boxes = pieces_c * per_piece;
        if (lane == 0) mbar_arrive_expect_tx(&full[slot], boxes * p.box_bytes);
        __syncwarp();
        if (lane < boxes) {
          const uint32_t piece = lane / per_piece, tj = lane % per_piece, tn = tj >> p.period_log2, j = tj & (p.period - 1);
          const uint32_t row0 = gate_up ? tile * 32 : tile * kTileRows;
          const uint32_t byte0 = p.lead[tn][j] + (csb0 + piece * p.piece_sb) * kSb;
          uint8_t *dst = smem + p.ring_off + slot * p.stage_bytes + lane * p.box_bytes;
          tma_load_2d(dst, &maps.m[tn][j], int(byte0 >> 4) * 4, int(row0 >> p.period_log2), &full[slot], policy, SB_DBG(2) == 0);
        }
        if (++slot == p.stages) slot = 0, ++round;
      }
    }
    if (!x_issued) issue_x();
    if (!ok && lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
    // Do not leave while copies are in flight: wait (bounded) until the consumers have released the
    // last fill of every stage, which they do only after its bytes have landed.
    for (uint32_t f = fill > p.stages ? fill - p.stages : 0; f < fill; ++f)
      if (!mbar_wait_backoff(&empty[f % p.stages], (f / p.stages) & 1)) break;
    return;
  }

  float *red = reinterpret_cast<float *>(smem + p.red_off);

  if (warp > kConsumerWarps) {
    // ---- epilogue warps: tile i of this CTA belongs to epilogue warp i % kEpiWarps. Each adds the k-group
    // warps' sums in order, exchanges split-K partials and stores. Lane l owns token l / 2 and tile
    // rows 32 (l % 2) .. + 31, so every global access of a lane is 64 or 128 contiguous bytes. ----
    const uint32_t ew = warp - kConsumerWarps - 1;
    pdl_wait();  // aux / out / partials belong to the stream's earlier kernels until they finish
    const uint32_t pcols = gate_up ? 2 * p.n : p.n;
    const uint32_t tok = lane >> 1, half = lane & 1;
    if (!mbar_wait_backoff(xfull, 0)) { if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED); return; }
    const float sback = scale_back[tok];
    uint32_t done = 0;
    for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++done) {
      if (done % kEpiWarps != ew || SB_DBG(8)) continue;
      const uint32_t tile = item / p.slices;
      if (!mbar_wait_backoff(&red_full[ew], (done / kEpiWarps) & 1)) { if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED); return; }
      float v[32];
#pragma unroll
      for (int r = 0; r < 32; ++r) v[r] = 0.0f;
#pragma unroll
      for (int k = 0; k < kKG; ++k) {  // the k-group warps' sums in order
        // Plain tiles: rows 32 half .. + 31 of the tile (row group `half`). Gate/up tiles: columns 16 half .. + 15,
        // their gate sums (row group 0) in v[0..15] and their up sums (row group 1) in v[16..31].
        const float4 *s0 = reinterpret_cast<const float4 *>(red + ((gate_up ? 0 : half) * kKG + k) * kRedWarpFloats + tok * kRedTokPitch + (gate_up ? 16 * half : 0));
        const float4 *s1 = gate_up ? reinterpret_cast<const float4 *>(red + (kKG + k) * kRedWarpFloats + tok * kRedTokPitch + 16 * half) : s0 + 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 a4 = s0[q], b4 = s1[q];
          v[4 * q] += a4.x, v[4 * q + 1] += a4.y, v[4 * q + 2] += a4.z, v[4 * q + 3] += a4.w;
          v[16 + 4 * q] += b4.x, v[16 + 4 * q + 1] += b4.y, v[16 + 4 * q + 2] += b4.z, v[16 + 4 * q + 3] += b4.w;
        }
      }
#pragma unroll
      for (int r = 0; r < 32; ++r) v[r] *= sback;
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[ew]);
      // The lane's 32 values as two runs of 16 in the partials: columns c0 + 16 half (+ 16) of a plain tile, or
      // the gate run and, n columns on, the up run of columns c0 + 16 half of a gate/up tile.
      const uint32_t c0 = gate_up ? tile * 32 : tile * kTileRows + 32 * half;
      const uint32_t run0 = gate_up ? c0 + 16 * half : c0, run1 = gate_up ? run0 + p.n : c0 + 16;
      const bool col_ok = c0 < p.n;  // n is a multiple of 32: a 32-column run is inside or outside
      auto part = [&](uint32_t sl, uint32_t run) {
        return reinterpret_cast<float4 *>(p.partials + (size_t(sl) * kTokens + tok) * pcols + (run ? run1 : run0));
      };
      if (p.epilogue == SB_EPILOGUE_PARTIALS || p.epilogue == SB_EPILOGUE_GATE_UP_PARTIALS) {  // this slice's sums as they are; their consumer adds the slices
        if (col_ok) {
          float *dst = static_cast<float *>(p.out) + (size_t(slice) * kTokens + tok) * p.out_stride;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            reinterpret_cast<float4 *>(dst + (q < 4 ? run0 : run1))[q & 3] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        continue;
      }
      bool finish = true;
      if (p.slices > 1) {
        if (col_ok) {
#pragma unroll
          for (int q = 0; q < 8; ++q) part(slice, q >> 2)[q & 3] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atom_add_acq_rel_gpu(&p.counters[tile], 1u);  // releases the warp's partials, acquires the others'
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        __syncwarp();
        finish = arrived == p.slices - 1;
        if (finish) {
          if (col_ok && p.slices == 2) {
            // Two slices: a + b is b + a, so this warp keeps its own sums in registers (its stores may still be
            // on their way) and adds the other slice's from L2.
            float4 q[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = __ldcg(part(slice ^ 1, i >> 2) + (i & 3));
#pragma unroll
            for (int i = 0; i < 8; ++i) v[4 * i] += q[i].x, v[4 * i + 1] += q[i].y, v[4 * i + 2] += q[i].z, v[4 * i + 3] += q[i].w;
          } else if (col_ok) {
#pragma unroll
            for (int r = 0; r < 32; ++r) v[r] = 0.0f;
            // Two slices' loads in flight at a time, added in slice order.
            for (uint32_t sl = 0; sl < p.slices; sl += 2) {
              const bool two = sl + 1 < p.slices;
              float4 qa[8], qb[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) qa[i] = __ldcg(part(sl, i >> 2) + (i & 3));
#pragma unroll
              for (int i = 0; i < 8; ++i) qb[i] = __ldcg(part(two ? sl + 1 : sl, i >> 2) + (i & 3));
#pragma unroll
              for (int i = 0; i < 8; ++i) v[4 * i] += qa[i].x, v[4 * i + 1] += qa[i].y, v[4 * i + 2] += qa[i].z, v[4 * i + 3] += qa[i].w;
              if (two)
#pragma unroll
                for (int i = 0; i < 8; ++i) v[4 * i] += qb[i].x, v[4 * i + 1] += qb[i].y, v[4 * i + 2] += qb[i].z, v[4 * i + 3] += qb[i].w;
            }
          }
          if (lane == 0) p.counters[tile] = 0;
        }
      }
      if (!finish) continue;
      if (gate_up) {
        // v[0..15] are the gate sums and v[16..31] the up sums of columns c0 + 16 half .. + 15.
        const float *gsum = v, *usum = v + 16;
        if (col_ok && tok < p.rows) {
          uint32_t pk[8];
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const float o0 = round_bf16(usum[2 * r]) * silu_f(round_bf16(gsum[2 * r]));
            const float o1 = round_bf16(usum[2 * r + 1]) * silu_f(round_bf16(gsum[2 * r + 1]));
            pk[r] = uint32_t(float_to_bf16_bits(o0)) | (uint32_t(float_to_bf16_bits(o1)) << 16);
          }
          uint4 *op = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.out) + size_t(tok) * p.out_stride + c0 + 16 * half);
          op[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          op[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
        continue;
      }
      if (!col_ok || tok >= p.rows) continue;
      if (p.epilogue == SB_EPILOGUE_RESIDUAL || p.epilogue == SB_EPILOGUE_UP_WITH_GATE) {
        const uint4 *ap = reinterpret_cast<const uint4 *>(p.aux + size_t(tok) * p.aux_stride + c0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 a4 = ap[q];
          const uint32_t u[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float xa = bf16_bits_to_float(u[i] & 0xffffu), xb = bf16_bits_to_float(u[i] >> 16);
            float &a = v[8 * q + 2 * i], &b = v[8 * q + 2 * i + 1];
            if (p.epilogue == SB_EPILOGUE_RESIDUAL) {
              a += xa;
              b += xb;
            } else {
              a = round_bf16(a) * silu_f(xa);
              b = round_bf16(b) * silu_f(xb);
            }
          }
        }
      }
      if (p.out_f32) {
        float4 *op = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + size_t(tok) * p.out_stride + c0);
#pragma unroll
        for (int q = 0; q < 8; ++q) op[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
        uint4 *op = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.out) + size_t(tok) * p.out_stride + c0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t pk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            pk[i] = uint32_t(float_to_bf16_bits(v[8 * q + 2 * i])) | (uint32_t(float_to_bf16_bits(v[8 * q + 2 * i + 1])) << 16);
          op[q] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
    return;
  }

  // ---- consumers ----
  const uint32_t rg = warp / kKG, kg = warp % kKG;
  const uint32_t g = lane >> 2, t = lane & 3;
  if (!mbar_wait(xfull, 0)) {
    if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
    return;
  }
  // Super-blocks are dealt to the k-group warps round-robin over the CTA's whole stream (jmod = count so far
  // mod kKG), so a stage of 4 keeps 4 of the 6 warps of a row group busy and the next stage the other ones.
  uint32_t done = 0, jmod = 0;
  // The ring position is carried along (slot, phase) and each lane's row offsets inside a stage are formed once:
  // per stage a warp then spends a handful of instructions besides its multiply.
  uint32_t slot = 0, phase = 0;
  uint32_t row_at[kMT][2];  // where the lane's rows lie inside a piece: (tensor, row) -> bytes
  uint32_t row_lead[kMT][2];
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint32_t tr = rg * 32 + mt * 16 + r * 8 + g;          // tile row
      const uint32_t tn = gate_up ? tr >> 5 : 0, rl = gate_up ? tr & 31 : tr;
      if (FMT == SB_FMT_Q4K) {
        row_at[mt][r] = tn * p.box_bytes + rl * 144;
        row_lead[mt][r] = 0;
      } else {
        // A row sits in the box of its (piece, tensor, residue) at `lead` bytes past a 16-byte boundary.
        const uint32_t j = rl & (p.period - 1), i = rl >> p.period_log2;  // map and row within its box
        row_at[mt][r] = ((tn << p.period_log2) + j) * p.box_bytes + i * p.pitch;
        row_lead[mt][r] = p.lead[tn][j];
      }
    }
  const uint32_t piece_bytes = (p.tensors << p.period_log2) * p.box_bytes;
  const uint8_t *ring = smem + p.ring_off;
  for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++done) {
    float y[kMT][2][4];
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 4; ++c) y[mt][h][c] = 0.0f;
    uint32_t csb0 = sb0;
    for (uint32_t c = 0; c < chunks; ++c, csb0 += kStageSb) {
      // Every warp follows every stage's barrier, with or without work in it: the parity wait tells only
      // consecutive phases apart.
      if (!SB_DBG(16) && !mbar_wait(&full[slot], phase)) {
        if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
        return;  // the launch has failed; the status word says so
      }
      const uint32_t nsb_c = min(uint32_t(kStageSb), sb1 - csb0);
      const uint32_t sbi = kg >= jmod ? kg - jmod : kg + kKG - jmod;  // the stage's super-block dealt to this k-group
      jmod += nsb_c;
      if (jmod >= kKG) jmod -= kKG;
      if (sbi < nsb_c && !SB_DBG(1)) {
        const uint8_t *stage = ring + slot * p.stage_bytes;
        constexpr uint32_t kPieceSb = WFmt<FMT>::kPieceSb;
        const uint32_t lsb = csb0 + sbi - sb0;
        const uint32_t piece = sbi / kPieceSb, within = sbi % kPieceSb;
        uint32_t roff[kMT][2];
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            if (FMT == SB_FMT_Q4K) {
              roff[mt][r] = piece * piece_bytes + row_at[mt][r];
            } else {
              const uint32_t lead = (row_lead[mt][r] + (csb0 + piece * kPieceSb) * kSb) & 15u;
              roff[mt][r] = piece * piece_bytes + row_at[mt][r] + lead + within * kSb;
            }
          }
        const uint8_t *xs_sb = smem + p.x_off + lsb * kPrepSbBytes;
        multiply_super_block<FMT, kMT>(stage, roff, xs_sb, xs_sb + kXsbBytes, lane, y);
      }
      __syncwarp();
      if (lane == 0 && !SB_DBG(16)) mbar_arrive(&empty[slot]);
      if (++slot == p.stages) slot = 0, phase ^= 1;
    }
    if (SB_DBG(8)) continue;
    // Hand the tile's sums to the epilogue warp once it has read the previous tile's.
    if (done > 0 && !mbar_wait(&red_empty[(done - 1) % kEpiWarps], ((done - 1) / kEpiWarps) & 1)) {
      if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
      return;
    }
    float *mine = red + warp * kRedWarpFloats;
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mine[(h * 8 + 2 * t) * kRedTokPitch + mt * 16 + g] = y[mt][h][0];
        mine[(h * 8 + 2 * t + 1) * kRedTokPitch + mt * 16 + g] = y[mt][h][1];
        mine[(h * 8 + 2 * t) * kRedTokPitch + mt * 16 + g + 8] = y[mt][h][2];
        mine[(h * 8 + 2 * t + 1) * kRedTokPitch + mt * 16 + g + 8] = y[mt][h][3];
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(&red_full[done % kEpiWarps]);
  }
}

// ---- host side ----
static uint32_t pick_slices(uint32_t nsb, uint32_t sb_bytes) {
  // Activations of a slice stay resident: at most kMaxSliceSb super-blocks, fewer where a format's
  // wider stages need the room.
  uint32_t cap = sb_bytes > 250 ? 6 : sb_bytes > 160 ? 8 : kMaxSliceSb;
#ifdef SB_DIAG
  if (const char *e = getenv("SB_SLICE_CAP")) cap = std::min<uint32_t>(cap, std::max(1, atoi(e)));  // (diagnostic builds: shorter slices, more items)
#endif
  const uint32_t s = (nsb + cap - 1) / cap;
  return s < 1 ? 1 : s;
}

static int make_plan(uint32_t format, uint32_t n, uint32_t k, uint32_t epilogue, LinearParams &p, SbLinearPlan &plan) {
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80,
             "sb_linear: format %u is not a quantized block format of this kernel", format);
  SB_REQUIRE(k && k % 256 == 0, "sb_linear: k = %u is not a multiple of 256", k);
  SB_REQUIRE(n && n % 32 == 0, "sb_linear: n = %u is not a multiple of 32", n);
  const bool gate_up = epilogue == SB_EPILOGUE_GATE_UP || epilogue == SB_EPILOGUE_GATE_UP_PARTIALS;
  const uint32_t sb_bytes = format == SB_FMT_Q4K ? 144 : format == SB_FMT_Q6K ? 210 : 272;
  p.nsb = k / 256;
  p.slices = pick_slices(p.nsb, sb_bytes);
  p.tiles = gate_up ? (n + 31) / 32 : (n + kTileRows - 1) / kTileRows;
  p.row_bytes = uint32_t(sb_row_bytes(format, k));
  // Stage geometry. Q4_K rows are 16-byte multiples: one map, one box of 64 x 144 bytes per
  // super-block (pitch 144 = 16 mod 32: the 16-byte reads of 8 rows x 4 lanes hit distinct banks).
  // Q6_K / Q8_0 rows are only 2-byte aligned: `period` maps of every period-th row, boxes wide
  // enough for piece_sb super-blocks at any 2-byte lead.
  p.tensors = gate_up ? 2 : 1;
  const uint32_t tile_rows_per_tensor = gate_up ? 32 : kTileRows;
  if (format == SB_FMT_Q4K) {
    p.period = 1, p.pieces = kStageSb, p.piece_sb = 1, p.pitch = 144;
  } else {
    uint32_t gcd = 16;
    while (p.row_bytes % gcd) gcd >>= 1;
    p.period = 16 / gcd;
    p.piece_sb = format == SB_FMT_Q6K ? kStageSb : 2;
    p.pieces = kStageSb / p.piece_sb;
    p.pitch = (p.piece_sb * sb_bytes + 14 + 15) & ~15u;
  }
  p.period_log2 = p.period == 1 ? 0 : p.period == 2 ? 1 : p.period == 4 ? 2 : 3;
  p.box_rows = tile_rows_per_tensor / p.period;
  p.box_bytes = p.box_rows * p.pitch;
  SB_REQUIRE(p.box_bytes % 128 == 0 && p.pitch <= 1024, "sb_linear: unsupported stage geometry (k = %u)", k);
  p.stage_bytes = p.pieces * p.tensors * p.period * p.box_bytes;
  const uint32_t slice_max = (p.nsb + p.slices - 1) / p.slices;
  p.x_off = 384;  // barriers 0..231, scale_back 256..319
  p.red_off = p.x_off + slice_max * kPrepSbBytes;
  const uint32_t consumer_warps = kRG * (format == SB_FMT_Q4K ? WFmt<SB_FMT_Q4K>::kKG : format == SB_FMT_Q6K ? WFmt<SB_FMT_Q6K>::kKG : WFmt<SB_FMT_Q80>::kKG);
  p.ring_off = (p.red_off + consumer_warps * kRedWarpFloats * 4 + 127) & ~127u;
  const uint32_t budget = 227 * 1024;
  SB_REQUIRE(p.ring_off + 2 * p.stage_bytes <= budget, "sb_linear: shared memory plan does not fit (k = %u)", k);
  p.stages = std::min(uint32_t(kMaxStages), (budget - p.ring_off) / p.stage_bytes);
  const uint32_t sms = uint32_t(ctx().sm_count ? ctx().sm_count : 148);
  uint32_t ctas = sms / p.slices * p.slices;
  const uint32_t items = p.tiles * p.slices;
  if (ctas > items) ctas = items;
  plan = {p.slices, ctas, uint32_t(kTileRows), p.stages, p.ring_off + p.stages * p.stage_bytes, uint32_t(kStageSb),
          slice_max, p.tiles};
  return SB_OK;
}

// A 2-D map over `rows` rows of `stride` bytes starting at the 16-byte aligned `base`: u32 elements,
// box = box_rows x box_bytes. Rows past the end and bytes past a row read as zero.
int encode_weight_map(CUtensorMap *map, uintptr_t base, uint32_t stride, uint32_t rows, uint32_t box_bytes, uint32_t box_rows) {
  using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = nullptr;
  if (!encode) {
    cudaDriverEntryPointQueryResult qr;
    void *fn = nullptr;
    SB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
    if (!fn || qr != cudaDriverEntryPointSuccess) return fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable");
    encode = reinterpret_cast<Encode>(fn);
  }
  SB_REQUIRE(stride % 16 == 0 && box_bytes % 16 == 0 && box_bytes / 4 <= 256 && box_rows <= 256 && box_rows >= 1,
             "sb_linear: tensor map geometry (stride %u, box %u x %u)", stride, box_rows, box_bytes);
  const cuuint64_t dims[2] = {stride / 4, rows};
  const cuuint64_t strides[1] = {stride};
  const cuuint32_t box[2] = {box_bytes / 4, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, reinterpret_cast<void *>(base), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", int(r));
  return SB_OK;
}

static int launch_prepare(cudaStream_t stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride,
                          const void *norm_w, uint32_t layout, void *out, void *normed_out, bool pdl, const float *partials = nullptr,
                          uint32_t slices = 0, uint32_t partial_stride = 0, void *sum_out = nullptr, uint32_t sum_stride = 0,
                          const TpExchange *tp = nullptr, uint32_t swiglu_n = 0) {
  PrepareParams pp{static_cast<const uint16_t *>(x), static_cast<const float *>(norm_w), static_cast<uint8_t *>(out),
                   static_cast<uint16_t *>(normed_out), rows, k, x_stride, layout, partials, static_cast<uint16_t *>(sum_out), slices,
                   partial_stride, sum_stride, swiglu_n, tp ? *tp : TpExchange{}};
  if (tp) {  // the share's way to the peers, ahead of the conversion and not waited for by it
    cudaLaunchConfig_t push = {};
    push.gridDim = dim3(kTokens * kPrepCluster), push.blockDim = dim3(kPrepThreads), push.stream = stream;
    cudaLaunchAttribute pattr[1];
    pattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pattr[0].val.programmaticStreamSerializationAllowed = 1;
    push.attrs = pattr, push.numAttrs = pdl ? 1 : 0;
    SB_CUDA(cudaLaunchKernelEx(&push, tp_push_kernel, pp));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kTokens * kPrepCluster);
  cfg.blockDim = dim3(kPrepThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPrepCluster, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  SB_CUDA(tp ? cudaLaunchKernelEx(&cfg, prepare_kernel<true>, pp) : cudaLaunchKernelEx(&cfg, prepare_kernel<false>, pp));
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" int sb_linear_plan(uint32_t format, uint32_t n, uint32_t k, uint32_t rows, uint32_t epilogue,
                              SbLinearPlan *out_plan) {
  SB_REQUIRE(out_plan, "sb_linear_plan: null plan");
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_linear_plan: rows = %u outside 1..%d", rows, kTokens);
  LinearParams p{};
  return make_plan(format, n, k, epilogue, p, *out_plan);
}

extern "C" int sb_linear_plan_flags(uint32_t format, uint32_t n, uint32_t k, uint32_t rows, uint32_t epilogue, uint32_t flags,
                                    SbLinearPlan *out_plan) {
  SB_REQUIRE(out_plan, "sb_linear_plan: null plan");
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_linear_plan: rows = %u outside 1..%d", rows, kTokens);
  if (format == SB_FMT_Q4K && (flags & SB_LINEAR_TCGEN05)) return tc_plan(n, k, epilogue, *out_plan);
  return sb_linear_plan(format, n, k, rows, epilogue, out_plan);
}

extern "C" uint64_t sb_linear_prepared_bytes(uint32_t k) { return k % 256 ? 0 : kPrepHeader + uint64_t(k / 256) * kPrepSbBytes; }

extern "C" int sb_linear_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride,
                                 const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out,
                                 uint32_t flags) {
  SB_NEED_DEVICE();
  SB_REQUIRE(x && prepared_out, "sb_linear_prepare: null x or destination");
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_linear_prepare: rows = %u outside 1..%d", rows, kTokens);
  SB_REQUIRE(k && k % 256 == 0 && k <= 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster, "sb_linear_prepare: k = %u is not a multiple of 256 up to %d",
             k, 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster);
  SB_REQUIRE(x_stride >= k && x_stride % 8 == 0, "sb_linear_prepare: x_stride %u < k or not a multiple of 8", x_stride);
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80, "sb_linear_prepare: format %u", format);
  SB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(prepared_out) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(norm_weight) & 15) == 0,
             "sb_linear_prepare: x, norm_weight and the destination must be 16-byte aligned");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(normed_out) & 15) == 0, "sb_linear_prepare: normed_out must be 16-byte aligned");
  const uint32_t layout = format != SB_FMT_Q4K ? 0u : (flags & SB_LINEAR_TCGEN05) ? 2u : 1u;
  return launch_prepare(as_stream(stream), x, rows, k, x_stride, norm_weight, layout, prepared_out, normed_out,
                        (flags & SB_LINEAR_PDL) != 0);
}

extern "C" int sb_linear_prepare_sum(void *stream, const float *partials, uint32_t slices, uint32_t partial_stride, const void *residual,
                                     uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                                     const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out, uint32_t flags) {
  SB_NEED_DEVICE();
  SB_REQUIRE(partials && residual && sum_out && prepared_out, "sb_linear_prepare_sum: null pointer");
  SB_REQUIRE(slices >= 1 && slices <= 64, "sb_linear_prepare_sum: %u slices outside 1..64", slices);
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_linear_prepare_sum: rows = %u outside 1..%d", rows, kTokens);
  SB_REQUIRE(k && k % 256 == 0 && k <= 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster, "sb_linear_prepare_sum: k = %u is not a multiple of 256 up to %d",
             k, 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster);
  SB_REQUIRE(partial_stride >= k && partial_stride % 4 == 0 && residual_stride >= k && residual_stride % 8 == 0 && sum_stride >= k && sum_stride % 8 == 0,
             "sb_linear_prepare_sum: a stride is below k or misaligned");
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80, "sb_linear_prepare_sum: format %u", format);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(sum_out) |
               reinterpret_cast<uintptr_t>(prepared_out) | reinterpret_cast<uintptr_t>(norm_weight) | reinterpret_cast<uintptr_t>(normed_out)) & 15) == 0,
             "sb_linear_prepare_sum: pointers must be 16-byte aligned");
  const uint32_t layout = format != SB_FMT_Q4K ? 0u : (flags & SB_LINEAR_TCGEN05) ? 2u : 1u;
  return launch_prepare(as_stream(stream), residual, rows, k, residual_stride, norm_weight, layout, prepared_out, normed_out,
                        (flags & SB_LINEAR_PDL) != 0, partials, slices, partial_stride, sum_out, sum_stride);
}

extern "C" int sb_linear_prepare_gate_up(void *stream, const float *partials, uint32_t slices, uint32_t partial_stride, uint32_t n, void *act_out,
                                         uint32_t act_stride, uint32_t rows, uint32_t format, void *prepared_out, uint32_t flags) {
  SB_NEED_DEVICE();
  SB_REQUIRE(partials && act_out && prepared_out, "sb_linear_prepare_gate_up: null pointer");
  SB_REQUIRE(slices >= 1 && slices <= 64, "sb_linear_prepare_gate_up: %u slices outside 1..64", slices);
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_linear_prepare_gate_up: rows = %u outside 1..%d", rows, kTokens);
  SB_REQUIRE(n && n % 256 == 0 && n <= 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster, "sb_linear_prepare_gate_up: n = %u is not a multiple of 256 up to %d", n,
             8 * kPrepThreads * kPrepMaxChunks * kPrepCluster);
  SB_REQUIRE(partial_stride >= 2 * n && partial_stride % 4 == 0 && act_stride >= n && act_stride % 8 == 0,
             "sb_linear_prepare_gate_up: the partial rows hold 2 n columns, the output rows n; strides in fours and eights");
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80, "sb_linear_prepare_gate_up: format %u", format);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(act_out) | reinterpret_cast<uintptr_t>(prepared_out)) & 15) == 0,
             "sb_linear_prepare_gate_up: pointers must be 16-byte aligned");
  const uint32_t layout = format != SB_FMT_Q4K ? 0u : (flags & SB_LINEAR_TCGEN05) ? 2u : 1u;
  return launch_prepare(as_stream(stream), nullptr, rows, n, 0, nullptr, layout, prepared_out, nullptr, (flags & SB_LINEAR_PDL) != 0, partials, slices,
                        partial_stride, act_out, act_stride, nullptr, n);
}

extern "C" int sb_tp_prepare_sum(void *stream, void *group, uint32_t index, const float *partials, uint32_t slices, uint32_t partial_stride,
                                 const void *residual, uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                                 const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out, uint32_t flags) {
  SB_NEED_DEVICE();
  TpExchange x;
  const int st = tp_exchange(group, index, false, x);
  if (st != SB_OK) return st;
  SB_REQUIRE(partials && residual && sum_out && prepared_out, "sb_tp_prepare_sum: null pointer");
  SB_REQUIRE(slices >= 1 && slices <= 64, "sb_tp_prepare_sum: %u slices outside 1..64", slices);
  SB_REQUIRE(rows >= 1 && rows <= kTokens, "sb_tp_prepare_sum: rows = %u outside 1..%d", rows, kTokens);
  SB_REQUIRE(k == x.width, "sb_tp_prepare_sum: k = %u, the group exchanges rows of %u", k, x.width);
  SB_REQUIRE(k && k % 256 == 0 && k <= 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster, "sb_tp_prepare_sum: k = %u is not a multiple of 256 up to %d",
             k, 8 * kPrepThreads * kPrepMaxChunks * kPrepCluster);
  SB_REQUIRE(partial_stride >= k && partial_stride % 4 == 0 && residual_stride >= k && residual_stride % 8 == 0 && sum_stride >= k && sum_stride % 8 == 0,
             "sb_tp_prepare_sum: a stride is below k or misaligned");
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80, "sb_tp_prepare_sum: format %u", format);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(sum_out) |
               reinterpret_cast<uintptr_t>(prepared_out) | reinterpret_cast<uintptr_t>(norm_weight) | reinterpret_cast<uintptr_t>(normed_out)) & 15) == 0,
             "sb_tp_prepare_sum: pointers must be 16-byte aligned");
  const uint32_t layout = format != SB_FMT_Q4K ? 0u : (flags & SB_LINEAR_TCGEN05) ? 2u : 1u;
  return launch_prepare(as_stream(stream), residual, rows, k, residual_stride, norm_weight, layout, prepared_out, normed_out,
                        (flags & SB_LINEAR_PDL) != 0, partials, slices, partial_stride, sum_out, sum_stride, &x);
}

extern "C" int sb_linear(void *stream, const SbLinearArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a, "sb_linear: null arguments");
  // The many-row kernel (tensor memory, fp16 weights): more than 16 rows, and every NVFP4 projection (given as its image).
  if (a->rows > uint32_t(kTokens) || (a->flags & SB_LINEAR_WIDE_IMAGE) || a->format == SB_FMT_NVFP4) return sb_linear_wide(stream, a);
  SB_REQUIRE(a->weights && a->out && (a->x || a->prepared), "sb_linear: null weights, out, or neither x nor prepared");
  SB_REQUIRE(a->rows >= 1 && a->rows <= kTokens, "sb_linear: rows = %u outside 1..%d", a->rows, kTokens);
  SB_REQUIRE(a->epilogue <= SB_EPILOGUE_GATE_UP_PARTIALS, "sb_linear: unknown epilogue %u", a->epilogue);
  const bool unreduced = a->epilogue == SB_EPILOGUE_PARTIALS || a->epilogue == SB_EPILOGUE_GATE_UP_PARTIALS;
  const bool pair = a->epilogue == SB_EPILOGUE_GATE_UP || a->epilogue == SB_EPILOGUE_GATE_UP_PARTIALS;
  SB_REQUIRE(pair == (a->weights2 != nullptr), "sb_linear: weights2 is given exactly with the gate/up epilogues");
  SB_REQUIRE(a->epilogue != SB_EPILOGUE_GATE_UP_PARTIALS || (a->out_f32 && a->out_stride >= 2 * a->n),
             "sb_linear: SB_EPILOGUE_GATE_UP_PARTIALS writes fp32 rows of at least 2 n columns");
  SB_REQUIRE((a->epilogue == SB_EPILOGUE_RESIDUAL || a->epilogue == SB_EPILOGUE_UP_WITH_GATE) == (a->aux != nullptr),
             "sb_linear: aux is given exactly with the residual and up-with-gate epilogues");
  SB_REQUIRE(a->out_stride >= a->n && a->out_stride % 8 == 0, "sb_linear: out_stride %u < n or not a multiple of 8", a->out_stride);
  SB_REQUIRE(!a->aux || (a->aux_stride >= a->n && a->aux_stride % 8 == 0), "sb_linear: aux_stride %u < n or not a multiple of 8", a->aux_stride);
  SB_REQUIRE(!(a->out_f32 && a->epilogue != SB_EPILOGUE_NONE && !unreduced), "sb_linear: an fp32 destination takes no epilogue");
  SB_REQUIRE(!unreduced || !(a->flags & SB_LINEAR_TCGEN05), "sb_linear: unreduced k-slice sums are not offered by the tcgen05 kernel");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->aux) & 15) == 0,
             "sb_linear: out and aux must be 16-byte aligned");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(a->weights) & 1) == 0 && (reinterpret_cast<uintptr_t>(a->weights2) & 1) == 0,
             "sb_linear: weights must be 2-byte aligned");
  const bool tensor_core = a->format == SB_FMT_Q4K && (a->flags & SB_LINEAR_TCGEN05);
  LinearParams p{};
  SbLinearPlan plan;
  int st = tensor_core ? tc_plan(a->n, a->k, a->epilogue, plan) : make_plan(a->format, a->n, a->k, a->epilogue, p, plan);
  if (st != SB_OK) return st;
  if (a->format == SB_FMT_Q4K)
    SB_REQUIRE((reinterpret_cast<uintptr_t>(a->weights) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a->weights2) & 15) == 0,
               "sb_linear: Q4_K weights must be 16-byte aligned");
  Context &c = ctx();
  if (tensor_core) {
    const void *prep = a->prepared;
    if (!prep) {
      SB_REQUIRE(sb_linear_prepared_bytes(a->k) <= c.prepared_bytes, "sb_linear: k = %u exceeds the context's prepared-input scratch", a->k);
      st = sb_linear_prepare(stream, a->x, a->rows, a->k, a->x_stride, a->norm_weight, a->format, c.prepared, nullptr, a->flags);
      if (st != SB_OK) return st;
      prep = c.prepared;
    } else {
      SB_REQUIRE((reinterpret_cast<uintptr_t>(prep) & 15) == 0, "sb_linear: prepared must be 16-byte aligned");
    }
    return launch_linear_tc(as_stream(stream), a, prep, (a->flags & SB_LINEAR_PDL) != 0);
  }
  const uint32_t pcols = pair ? 2 * a->n : a->n;
  SB_REQUIRE(p.slices == 1 || unreduced || size_t(p.slices) * kTokens * pcols * 4 <= c.linear_partials_bytes,
             "sb_linear: split-K scratch too small for n = %u with %u slices", a->n, p.slices);
  SB_REQUIRE(p.tiles <= c.linear_counter_count, "sb_linear: too many tiles (%u)", p.tiles);
  const bool pdl = (a->flags & SB_LINEAR_PDL) != 0;
  const void *prepared = a->prepared;
  if (!prepared) {
    SB_REQUIRE(sb_linear_prepared_bytes(a->k) <= c.prepared_bytes, "sb_linear: k = %u exceeds the context's prepared-input scratch", a->k);
    st = sb_linear_prepare(stream, a->x, a->rows, a->k, a->x_stride, a->norm_weight, a->format, c.prepared, nullptr, a->flags);
    if (st != SB_OK) return st;
    prepared = c.prepared;
  } else {
    SB_REQUIRE((reinterpret_cast<uintptr_t>(prepared) & 15) == 0, "sb_linear: prepared must be 16-byte aligned");
  }
  p.w = static_cast<const uint8_t *>(a->weights);
  p.w2 = static_cast<const uint8_t *>(a->weights2);
  p.prepared = static_cast<const uint8_t *>(prepared);
  p.aux = static_cast<const uint16_t *>(a->aux);
  p.out = a->out;
  p.partials = c.linear_partials;
  p.counters = c.linear_counters;
  p.status = c.status_dev;
  p.n = a->n, p.k = a->k, p.rows = a->rows;
  p.aux_stride = a->aux_stride, p.out_stride = a->out_stride;
  p.epilogue = a->epilogue, p.out_f32 = a->out_f32;
#ifdef SB_DIAG
  p.debug = a->flags >> 8;
#else
  SB_REQUIRE((a->flags & ~uint32_t(SB_LINEAR_PDL | SB_LINEAR_TCGEN05)) == 0, "sb_linear: unknown flags 0x%x", a->flags);
#endif

  void (*kernel)(const LinearParams, const LinearMaps) = a->format == SB_FMT_Q4K   ? linear_kernel<SB_FMT_Q4K>
                                       : a->format == SB_FMT_Q6K ? linear_kernel<SB_FMT_Q6K>
                                                                 : linear_kernel<SB_FMT_Q80>;
  // The shared-memory cap is a per-device attribute of the function: remembered per (device, format).
  static bool attr_set[64][3] = {};
  const int ki = a->format == SB_FMT_Q4K ? 0 : a->format == SB_FMT_Q6K ? 1 : 2;
  const int dev = c.device >= 0 && c.device < 64 ? c.device : 0;
  if (!attr_set[dev][ki]) {
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev][ki] = true;
  }
  LinearMaps maps;
  for (uint32_t tn = 0; tn < p.tensors; ++tn)
    for (uint32_t j = 0; j < p.period; ++j) {
      const uintptr_t first = reinterpret_cast<uintptr_t>(tn ? a->weights2 : a->weights) + size_t(j) * p.row_bytes;
      p.lead[tn][j] = uint32_t(first & 15u);
      st = encode_weight_map(&maps.m[tn][j], first & ~uintptr_t(15), p.row_bytes * p.period,
                             (a->n - j + p.period - 1) / p.period, p.pitch, p.box_rows);
      if (st != SB_OK) return st;
    }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.ctas);
  cfg.blockDim = dim3(32 * (kRG * (a->format == SB_FMT_Q4K ? WFmt<SB_FMT_Q4K>::kKG : a->format == SB_FMT_Q6K ? WFmt<SB_FMT_Q6K>::kKG : WFmt<SB_FMT_Q80>::kKG) + 1 + kEpiWarps));
  cfg.dynamicSmemBytes = plan.smem_bytes;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, maps));
  return SB_OK;
}
