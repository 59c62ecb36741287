// Q4_K linear for the verify step's 16 rows on the tcgen05 tensor cores: Y[16,N] = X[16,K] W[N,K]^T
// with the weights streamed once from HBM as native GGUF super-blocks.
//
// Same contract and arithmetic as the warp-MMA kernel (exact integer operand sc*q <= 945 in fp16,
// fp32 sums, y += d*Aq - dmin*Am per super-block; reference: runtime/ops/LinearGguf.cpp:281-362,
// runtime/metal/kernels/decode/linear_gguf_sgmatrix.metal:1-27), re-cut for Blackwell:
//
//   tile      128 weight rows = the 128 lanes of tensor memory; one thread owns one weight row
//   producer  one thread streams 128 x 144-byte boxes (one super-block column of the tile) into a ring
//             with tiled TMA loads completing on mbarriers
//   dequant   16 warps: warp (quadrant q, pair p) turns sub-blocks 2p, 2p+1 of rows 32q..32q+31 into
//             64 exact fp16 integers per row (one LOP3 + one HFMA2 per two weights) and writes them
//             with tcgen05.st straight into the A operand in tensor memory: no shared-memory round
//             trip for the expanded weights, no fragment shuffling
//   mma       one thread issues, per super-block, 16 tcgen05.mma (M 128, N 16, K 16; A from tensor
//             memory, B = the prepared activations in shared memory) into a fresh accumulator and one
//             more for the 6-bit mins against the sub-block sums of x; tcgen05.commit releases the
//             A buffer and publishes the accumulator
//   epilogue  two groups of 4 warps alternate tiles: per super-block a thread reads its row's 16 + 16
//             sums from tensor memory and folds them with its row's d, dmin; at the end of a tile it
//             exchanges split-K partials (slice order, runtime/metal/kernels/common/split_reduce.h:24-55)
//             and applies the epilogue while the other group already accumulates the next tile
//
// Measured on B200 (cycle counters in the roles): one tcgen05.mma of this shape holds the issuing thread for
// about 75 cycles whatever N is, so the 17 MMAs of a super-block cost about 1300 cycles per 18 KB of weights,
// a ceiling near 4 TB/s per GPU at 16 tokens. The same 17 MMAs serve up to 256 tokens, which is where this
// kernel belongs; at 16 rows the warp-MMA kernel in sb_linear.cu is the default and this one is selected
// with SB_LINEAR_TCGEN05.
//
// Tensor-memory columns: 3 A buffers x 136 (128 packed weight columns + 8 of mins), then 2
// accumulator sets x 48 (16 tokens of Aq from even K-steps, 16 from odd K-steps, 16 of Am).
#include <algorithm>

#include <cuda.h>

#include "sb_internal.h"
#include "sb_linear_internal.h"
#include "sb_ptx.cuh"
#include "sb_tcgen05.cuh"

namespace sb {

constexpr int kTcDequantWarps = 12, kTcEpilogueWarps = 8;  // dequant: 3 groups (one per A buffer) x 4 quadrants
constexpr int kTcProducerWarp = kTcDequantWarps + kTcEpilogueWarps, kTcMmaWarp = kTcProducerWarp + 1;
constexpr int kTcMmaWarps = 2;                     // each issues the K-steps of one parity
constexpr int kTcThreads = 32 * (kTcMmaWarp + kTcMmaWarps);  // 736
constexpr uint32_t kTcTileRows = 128;
constexpr uint32_t kTcStageBytes = kTcTileRows * 144;  // one super-block column of a tile
constexpr uint32_t kTcBoxes = 1, kTcBoxRows = kTcTileRows / kTcBoxes;  // TMA boxes per stage
constexpr uint32_t kTcMaxStages = 8, kTcABufs = 3, kTcDBufs = 2, kTcDmSlots = 8;
constexpr uint32_t kTcACols = 136, kTcDCol0 = kTcABufs * kTcACols, kTcDCols = 48, kTcTmemCols = 512;
constexpr uint32_t kTcXOff = 4480;  // barriers 0..239, tmem slot 248, scale_back 256..319, d/dmin ring 320..4415

struct TcParams {
  const uint8_t *prepared;
  const uint16_t *aux;
  void *out;
  float *partials;
  uint32_t *counters, *status;
  uint32_t n, rows, aux_stride, out_stride, epilogue, out_f32;
  uint32_t nsb, slices, tiles, stages, ring_off;
  uint32_t debug;  // diagnostics: 1 no MMA issue, 2 no tensor-memory stores, 4 no accumulator loads, 8 arrivals for commits (with 1), 16 ring only, 64 no tile finish
};
struct TcMaps {
  CUtensorMap m[2];  // weights, weights2 (gate/up)
};

// The 6-bit scales and mins of a super-block's 8 sub-blocks as bytes: sc[0], mn[0] hold sub-blocks 0..3,
// sc[1], mn[1] sub-blocks 4..7, from the 16-byte header {d, dmin, 12 packed bytes}.
struct TcScaleBytes {
  uint32_t sc[2], mn[2];
};
__device__ __forceinline__ TcScaleBytes tc_scale_bytes(const uint4 hdr) {
  TcScaleBytes r;
  r.sc[0] = hdr.y & 0x3f3f3f3fu;
  r.mn[0] = hdr.z & 0x3f3f3f3fu;
  r.sc[1] = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
  r.mn[1] = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
  return r;
}
// Bytes (2i, 2i+1) of `bytes` (i = 0, 1) as two exact halves: {0x6400 | byte} - 1024.
__device__ __forceinline__ uint32_t byte_pair_as_halves(uint32_t bytes, uint32_t i) {
  return hsub2_u32(__byte_perm(bytes, 0x64646464u, i ? 0x4342 : 0x4140), 0x64006400u);
}
__device__ __forceinline__ uint32_t byte_as_half2(uint32_t bytes, uint32_t i) {
  const uint32_t sel = i == 0 ? 0x4040 : i == 1 ? 0x4141 : i == 2 ? 0x4242 : 0x4343;
  return hsub2_u32(__byte_perm(bytes, 0x64646464u, sel), 0x64006400u);
}

// A bounded wait whose outcome is the same in every lane, so the .aligned tensor-memory instructions
// that follow always run with the whole warp.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity);  // one lane polls; the barrier word is not hammered 32-fold
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Records which wait gave up: low byte SB_DEV_WAIT_EXPIRED, bits 8..15 the wait site (1 producer ring, 2
// activations, 3 A full, 4 accumulator empty, 5 ring full, 6 A empty, 7 hand-over, 8 accumulator full),
// bits 16..31 the super-block count of the role at that moment. The first report of a launch stays.
__device__ __forceinline__ void report_expired(uint32_t *status, uint32_t site, uint32_t unit) {
  atomicCAS(status, 0u, uint32_t(SB_DEV_WAIT_EXPIRED) | (site << 8) | (unit << 16));
}

__device__ __forceinline__ bool warp_wait_backoff(uint64_t *bar, uint32_t parity) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_backoff(bar, parity);
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <bool GATE_UP>
__global__ void __launch_bounds__(kTcThreads, 1) linear_tc_kernel(const TcParams p, const __grid_constant__ TcMaps maps) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *raw_full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *raw_empty = raw_full + kTcMaxStages;
  uint64_t *a_full = raw_empty + kTcMaxStages;
  uint64_t *a_empty = a_full + kTcABufs;
  uint64_t *d_full = a_empty + kTcABufs;
  uint64_t *d_empty = d_full + kTcDBufs;
  uint64_t *xfull = d_empty + kTcDBufs;
  uint64_t *turn = xfull + 1;  // hand-over between the epilogue groups: phase j completes when tile j's sums are all read
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 248);
  float *scale_back = reinterpret_cast<float *>(smem + 256);
  uint32_t *dm_s = reinterpret_cast<uint32_t *>(smem + 320);  // [kTcDmSlots][128] {d, dmin} of a row's super-block
  uint8_t *x_s = smem + kTcXOff;
  uint8_t *ring = smem + p.ring_off;
  constexpr uint32_t kTensors = GATE_UP ? 2 : 1;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t slice = blockIdx.x % p.slices;
  const uint32_t sb0 = slice * p.nsb / p.slices, sb1 = (slice + 1) * p.nsb / p.slices;
  const uint32_t slice_sb = sb1 - sb0, units = kTensors * slice_sb;
  const uint32_t items = p.tiles * p.slices;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 4);
    }
    for (uint32_t i = 0; i < kTcABufs; ++i) {
      mbar_init(&a_full[i], 4);
      mbar_init(&a_empty[i], kTcMmaWarps);
    }
    for (uint32_t i = 0; i < kTcDBufs; ++i) {
      mbar_init(&d_full[i], kTcMmaWarps);
      mbar_init(&d_empty[i], 4);
    }
    mbar_init(xfull, 1);
    mbar_init(turn, 4);
    fence_mbar_init();
  }
  if (warp == kTcMmaWarp) tmem_alloc(tmem_slot, kTcTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();

  if (warp == kTcProducerWarp) {
    // ---- producer: weights do not depend on the previous kernel, so the ring fills at once. A stage is
    // fetched as kTcBoxes boxes issued by as many lanes: the copy engine works on them side by side. ----
    const uint64_t policy = policy_evict_first();
    uint32_t u = 0, st = 0, phase = 0;
    bool ok = true;
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const uint32_t tile = item / p.slices;
      for (uint32_t tn = 0; tn < kTensors && ok; ++tn)
        for (uint32_t c = 0; c < slice_sb; ++c, ++u) {
          if (u >= p.stages && !warp_wait_backoff(&raw_empty[st], phase ^ 1)) {
            if (lane == 0) report_expired(p.status, 1, u);
            ok = false;
            break;
          }
          if (lane == 0) mbar_arrive_expect_tx(&raw_full[st], kTcStageBytes);
          __syncwarp();
          if (lane < kTcBoxes)
            tma_load_2d(ring + st * kTcStageBytes + lane * (kTcBoxRows * 144), &maps.m[tn], int((sb0 + c) * 36),
                        int(tile * kTcTileRows + lane * kTcBoxRows), &raw_full[st], policy, true);
          if (++st == p.stages) st = 0, phase ^= 1;
        }
    }
    // Do not leave while copies are in flight: the dequant warps release a stage only after its bytes landed.
    for (uint32_t f = u > p.stages ? u - p.stages : 0; f < u; ++f)
      if (!warp_wait_backoff(&raw_empty[f % p.stages], (f / p.stages) & 1)) break;
  } else if (warp >= kTcMmaWarp) {
    // ---- MMA issuers: one thread per K-step parity ----
    if (lane == 0) {
      const uint32_t half = warp - kTcMmaWarp;
      if (half == 0) {
        pdl_wait();  // the prepared activations come from the previous kernel
        mbar_arrive_expect_tx(xfull, slice_sb * kPrepSbBytes + kPrepHeader);
        bulk_g2s(scale_back, p.prepared, kPrepHeader, xfull);
        bulk_g2s(x_s, p.prepared + kPrepHeader + size_t(sb0) * kPrepSbBytes, slice_sb * kPrepSbBytes, xfull);
      }
      bool ok = mbar_wait(xfull, 0);
      if (!ok) report_expired(p.status, 2, 0);
      constexpr uint32_t idesc = umma_idesc_f16(128, 16);
      uint32_t u = 0;
      for (uint32_t item = blockIdx.x; item < items && ok && !(p.debug & 16); item += gridDim.x)
        for (uint32_t tn = 0; tn < kTensors && ok; ++tn)
          for (uint32_t c = 0; c < slice_sb; ++c, ++u) {
            const uint32_t ab = u % kTcABufs, db = u % kTcDBufs;
            ok = mbar_wait(&a_full[ab], (u / kTcABufs) & 1);
            if (!ok) report_expired(p.status, 3, u);
            if (ok && u >= kTcDBufs) {
              ok = mbar_wait(&d_empty[db], (u / kTcDBufs - 1) & 1);
              if (!ok) report_expired(p.status, 4, u);
            }
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a0 = tmem + ab * kTcACols, d0 = tmem + kTcDCol0 + db * kTcDCols;
            const uint64_t b0 = umma_smem_desc(smem_u32(x_s + c * kPrepSbBytes), 128, 256);
            if (!(p.debug & 1)) umma_q4k_super_block_half(d0, a0, b0, idesc, half);
            if (p.debug & 8) {  // only with 1: plain arrivals in place of the commits
              mbar_arrive(&a_empty[ab]);
              mbar_arrive(&d_full[db]);
            } else {
              umma_commit(&a_empty[ab]);
              umma_commit(&d_full[db]);
            }
          }
    }
  } else if (warp < kTcDequantWarps) {
    // ---- dequant: group grp owns A buffer grp and every third super-block of this CTA's stream; a thread
    // expands its weight row's whole super-block, pair by pair (sub-blocks 2p, 2p+1 = 32 bytes of nibbles) ----
    const uint32_t q = warp & 3, grp = warp >> 2, row = 32 * q + lane;
    const uint32_t ta = tmem_addr(tmem, 32 * q, grp * kTcACols);
    const uint32_t my_items = (items - blockIdx.x + gridDim.x - 1) / gridDim.x, total = my_items * units;
    uint32_t st = grp % p.stages, raw_phase = 0, use = 0;
    for (uint32_t u = grp; u < total; u += kTcABufs, ++use) {
      if (!warp_wait(&raw_full[st], raw_phase)) {
        if (lane == 0) report_expired(p.status, 5, u);
        break;
      }
      const uint8_t *src = ring + st * kTcStageBytes + row * 144;
      const uint4 hdr = *reinterpret_cast<const uint4 *>(src);
      const TcScaleBytes sb = tc_scale_bytes(hdr);
      if (use > 0 && !(p.debug & 16) && !warp_wait(&a_empty[grp], (use - 1) & 1)) {
        if (lane == 0) report_expired(p.status, 6, u);
        break;
      }
      tc_fence_after_sync();
      dm_s[(u % kTcDmSlots) * 128 + row] = hdr.x;
      const uint32_t k1024 = 0x64006400u;
#pragma unroll
      for (uint32_t pr = 0; pr < 4; ++pr) {
        const uint4 qa = *reinterpret_cast<const uint4 *>(src + 16 + 32 * pr);
        const uint4 qb = *reinterpret_cast<const uint4 *>(src + 32 + 32 * pr);
        const uint32_t s0 = byte_as_half2(sb.sc[pr >> 1], 2 * (pr & 1)), s1 = byte_as_half2(sb.sc[pr >> 1], 2 * (pr & 1) + 1);
        const uint32_t mlo = s0, blo = hmul2_u32(s0, 0xE400E400u);                         // sc, -1024 sc
        const uint32_t mhi = hmul2_u32(s1, 0x2C002C00u), bhi = hmul2_u32(s1, 0xD400D400u);  // sc / 16, -64 sc
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t hi8 = w[c] >> 8;
          r[4 * c + 0] = hfma2_u32(and_or(w[c], 0x000f000fu, k1024), mlo, blo);
          r[4 * c + 1] = hfma2_u32(and_or(hi8, 0x000f000fu, k1024), mlo, blo);
          r[4 * c + 2] = hfma2_u32(and_or(w[c], 0x00f000f0u, k1024), mhi, bhi);
          r[4 * c + 3] = hfma2_u32(and_or(hi8, 0x00f000f0u, k1024), mhi, bhi);
        }
        if (!(p.debug & 2)) {
          tmem_st16(ta + 32 * pr, r);
          tmem_st16(ta + 32 * pr + 16, r + 16);
        }
      }
      if (!(p.debug & 2)) {
        // Mins of sub-blocks 0..7 as 4 packed columns, twice: against the high and the low parts of the sums.
        const uint32_t m[4] = {byte_pair_as_halves(sb.mn[0], 0), byte_pair_as_halves(sb.mn[0], 1),
                               byte_pair_as_halves(sb.mn[1], 0), byte_pair_as_halves(sb.mn[1], 1)};
        tmem_st8(ta + 128, m[0], m[1], m[2], m[3], m[0], m[1], m[2], m[3]);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&raw_empty[st]);
        if (!(p.debug & 16)) mbar_arrive(&a_full[grp]);
      }
      st += kTcABufs;
      if (st >= p.stages) st -= p.stages, raw_phase ^= 1;
    }
  } else {
    // ---- epilogue: group (warp - 16) / 4 takes this CTA's tiles alternately; thread = weight row ----
    const uint32_t grp = (warp - kTcDequantWarps) >> 2, q = warp & 3, row = 32 * q + lane;
    const uint32_t tq = tmem_addr(tmem, 32 * q, kTcDCol0);
    pdl_wait();  // aux / out / partials belong to the stream's earlier kernels until they finish
    bool ok = warp_wait(xfull, 0);
    if (!ok && lane == 0) report_expired(p.status, 2, 1);
    const uint32_t pcols = kTensors * p.n;
    uint32_t u = 0, done = 0;
    for (uint32_t item = blockIdx.x; item < items && ok && !(p.debug & 16); item += gridDim.x, ++done) {
      if ((done & 1) != grp) {
        u += units;
        continue;
      }
      // The accumulator barriers tell consecutive phases apart by parity only, so a group starts polling
      // them once the other group has seen the last accumulators of the tile before.
      if (done > 0 && !warp_wait(turn, (done - 1) & 1)) {
        if (lane == 0) report_expired(p.status, 7, u);
        ok = false;
        break;
      }
      const uint32_t tile = item / p.slices;
      float y[kTensors][16];
#pragma unroll
      for (uint32_t tn = 0; tn < kTensors; ++tn)
#pragma unroll
        for (int t = 0; t < 16; ++t) y[tn][t] = 0.0f;
#pragma unroll
      for (uint32_t tn = 0; tn < kTensors; ++tn) {
        for (uint32_t c = 0; c < slice_sb && ok; ++c, ++u) {
          const uint32_t db = u % kTcDBufs;
          if (!warp_wait(&d_full[db], (u / kTcDBufs) & 1)) {
            if (lane == 0) report_expired(p.status, 8, u);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          float acc[48];  // 16 tokens of Aq from the even K-steps, 16 from the odd ones, then 16 of Am
          if (!(p.debug & 4)) tmem_ld48_wait(tq + db * kTcDCols, acc);
          else
#pragma unroll
            for (int t = 0; t < 48; ++t) acc[t] = 0.0f;
          tc_fence_before_sync();
          const uint32_t dm = dm_s[(u % kTcDmSlots) * 128 + row];
          __syncwarp();
          if (lane == 0) mbar_arrive(&d_empty[db]);
          const __half2 dd = *reinterpret_cast<const __half2 *>(&dm);
          const float d = __low2float(dd), ndmin = -__high2float(dd);
#pragma unroll
          for (int t = 0; t < 16; ++t) y[tn][t] = fmaf(d, acc[t] + acc[16 + t], fmaf(ndmin, acc[32 + t], y[tn][t]));
        }
      }
      if (!ok) break;
      if (lane == 0) mbar_arrive(turn);

      // ---- tile finish: undo the rows' power-of-two scales, split-K exchange, epilogue, store ----
      const uint32_t col = tile * kTcTileRows + row;
      const bool col_ok = tile * kTcTileRows + 32 * q < p.n;  // n is a multiple of 32: uniform per warp
      if (!col_ok || (p.debug & 64)) continue;
#pragma unroll
      for (uint32_t tn = 0; tn < kTensors; ++tn)
#pragma unroll
        for (int t = 0; t < 16; ++t) y[tn][t] *= scale_back[t];
      if (p.slices > 1) {
#pragma unroll
        for (uint32_t tn = 0; tn < kTensors; ++tn)
#pragma unroll
          for (int t = 0; t < 16; ++t) p.partials[(size_t(slice) * 16 + t) * pcols + tn * p.n + col] = y[tn][t];
        __threadfence();
        __syncwarp();
        uint32_t arrived = 0;
        if (lane == 0) arrived = atomicAdd(&p.counters[tile * 4 + q], 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != p.slices - 1) continue;
        __threadfence();
#pragma unroll
        for (uint32_t tn = 0; tn < kTensors; ++tn)
#pragma unroll
          for (int t = 0; t < 16; ++t) y[tn][t] = 0.0f;
        for (uint32_t sl = 0; sl < p.slices; ++sl) {
#pragma unroll
          for (uint32_t tn = 0; tn < kTensors; ++tn) {
            float v[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) v[t] = __ldcg(p.partials + (size_t(sl) * 16 + t) * pcols + tn * p.n + col);
#pragma unroll
            for (int t = 0; t < 16; ++t) y[tn][t] += v[t];
          }
        }
        if (lane == 0) p.counters[tile * 4 + q] = 0;
      }
      if (GATE_UP) {
        uint16_t *out = static_cast<uint16_t *>(p.out) + col;
#pragma unroll
        for (int t = 0; t < 16; ++t)
          if (uint32_t(t) < p.rows) {
            const float o = round_bf16(y[kTensors - 1][t]) * silu_f(round_bf16(y[0][t]));
            out[size_t(t) * p.out_stride] = float_to_bf16_bits(o);
          }
        continue;
      }
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        if (uint32_t(t) >= p.rows) break;
        float v = y[0][t];
        if (p.epilogue == SB_EPILOGUE_RESIDUAL) v += bf16_bits_to_float(p.aux[size_t(t) * p.aux_stride + col]);
        else if (p.epilogue == SB_EPILOGUE_UP_WITH_GATE) v = round_bf16(v) * silu_f(bf16_bits_to_float(p.aux[size_t(t) * p.aux_stride + col]));
        if (p.out_f32) static_cast<float *>(p.out)[size_t(t) * p.out_stride + col] = v;
        else static_cast<uint16_t *>(p.out)[size_t(t) * p.out_stride + col] = float_to_bf16_bits(v);
      }
    }
  }

  // Everyone meets here, also after a wait that gave up, so tensor memory is always returned.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kTcMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTcTmemCols);
  }
}

// ---- host side ----
struct TcGeometry {
  uint32_t nsb, slices, tiles, stages, ring_off, smem_bytes, ctas, slice_max;
};

// k-slices: a CTA keeps its slice of the prepared activations resident, the grid is the largest
// multiple of the slice count that fits the SMs, and every CTA walks tiles with a fixed stride. Among
// the slice counts that fit shared memory take the one that keeps the SMs busiest (whole rounds of
// tiles), preferring long slices (fewer split-K partials) on ties.
static int tc_geometry(uint32_t n, uint32_t k, TcGeometry &g) {
  SB_REQUIRE(k && k % 256 == 0, "sb_linear: k = %u is not a multiple of 256", k);
  SB_REQUIRE(n && n % 32 == 0, "sb_linear: n = %u is not a multiple of 32", n);
  g.nsb = k / 256;
  g.tiles = (n + kTcTileRows - 1) / kTcTileRows;
  const uint32_t sms = uint32_t(ctx().sm_count ? ctx().sm_count : 148), budget = 227 * 1024;
  double best = -1.0;
  for (uint32_t s = 1; s <= 16 && s <= g.nsb; ++s) {
    const uint32_t slice_max = (g.nsb + s - 1) / s;
    const uint32_t ring_off = (kTcXOff + slice_max * kPrepSbBytes + 127) & ~127u;
    if (ring_off + 6 * kTcStageBytes > budget) continue;
    const uint32_t groups = sms / s;
    if (!groups) continue;
    const uint32_t rounds = (g.tiles + groups - 1) / groups;
    const double busy = double(g.tiles) * g.nsb / (double(rounds) * slice_max * sms);  // the longest slice sets the pace
    const double score = busy * slice_max / (slice_max + 0.5);
    if (score > best + 1e-9) {
      best = score;
      g.slices = s, g.slice_max = slice_max, g.ring_off = ring_off;
    }
  }
  SB_REQUIRE(best > 0.0, "sb_linear: shared memory plan does not fit (k = %u)", k);
  // A multiple of the dequant group count: every ring stage then always belongs to the same group, which has
  // itself seen the stage's previous fill complete (mbarrier waits tell consecutive phases apart by parity only).
  g.stages = std::min(kTcMaxStages, (budget - g.ring_off) / kTcStageBytes) / kTcABufs * kTcABufs;
  g.smem_bytes = g.ring_off + g.stages * kTcStageBytes;
  g.ctas = std::min(sms / g.slices * g.slices, g.tiles * g.slices);
  return SB_OK;
}

int tc_plan(uint32_t n, uint32_t k, uint32_t, SbLinearPlan &plan) {
  TcGeometry g{};
  const int st = tc_geometry(n, k, g);
  if (st != SB_OK) return st;
  plan = {g.slices, g.ctas, kTcTileRows, g.stages, g.smem_bytes, 1u, g.slice_max, g.tiles};
  return SB_OK;
}

int launch_linear_tc(cudaStream_t stream, const SbLinearArgs *a, const void *prepared, bool pdl) {
  TcGeometry g{};
  int st = tc_geometry(a->n, a->k, g);
  if (st != SB_OK) return st;
  const bool gate_up = a->epilogue == SB_EPILOGUE_GATE_UP;
  Context &c = ctx();
  const uint32_t pcols = gate_up ? 2 * a->n : a->n;
  SB_REQUIRE(g.slices == 1 || size_t(g.slices) * 16 * pcols * 4 <= c.linear_partials_bytes,
             "sb_linear: split-K scratch too small for n = %u with %u slices", a->n, g.slices);
  SB_REQUIRE(g.tiles * 4 <= c.linear_counter_count, "sb_linear: too many tiles (%u)", g.tiles);
  TcParams p{};
  p.prepared = static_cast<const uint8_t *>(prepared);
  p.aux = static_cast<const uint16_t *>(a->aux);
  p.out = a->out;
  p.partials = c.linear_partials;
  p.counters = c.linear_counters;
  p.status = c.status_dev;
  p.n = a->n, p.rows = a->rows, p.aux_stride = a->aux_stride, p.out_stride = a->out_stride;
  p.epilogue = a->epilogue, p.out_f32 = a->out_f32;
  p.debug = (a->flags >> 8) & 127 & ~32u;
  p.nsb = g.nsb, p.slices = g.slices, p.tiles = g.tiles, p.stages = g.stages, p.ring_off = g.ring_off;
  TcMaps maps;
  const uint32_t row_bytes = g.nsb * 144;
  for (uint32_t tn = 0; tn < (gate_up ? 2u : 1u); ++tn) {
    st = encode_weight_map(&maps.m[tn], reinterpret_cast<uintptr_t>(tn ? a->weights2 : a->weights), row_bytes, a->n, 144, kTcBoxRows);
    if (st != SB_OK) return st;
  }
  if (!gate_up) maps.m[1] = maps.m[0];
  void (*kernel)(const TcParams, const TcMaps) = gate_up ? linear_tc_kernel<true> : linear_tc_kernel<false>;
  static bool attr_set[64][2] = {};  // a function attribute is per device
  const int dev = ctx().device >= 0 && ctx().device < 64 ? ctx().device : 0;
  if (!attr_set[dev][gate_up]) {
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev][gate_up] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.ctas);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = g.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, maps));
  return SB_OK;
}

}  // namespace sb
