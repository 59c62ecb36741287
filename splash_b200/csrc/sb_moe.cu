// MoE expert passes for the few rows of one lane's verify block (M <= 16 rows, up to 32 routes a row): every route
// (row, expert) is a matrix-vector product against the expert's native Q4_K rows. Replaces, for that regime, the
// expert passes of MoE::addRouted (runtime/ops/MoE.cpp:122-187,260-270; kernels moe_gguf_expert_tile of
// runtime/metal/kernels/common/moe_gguf_expert_tile.h:33-84, the gate/up pass runtime/metal/kernels/shared/moe_gguf.metal:
// 94-160 and moe_combine, runtime/metal/kernels/shared/moe.metal:367-392):
//   intermediate = bf16(bf16(up . x) * silu(bf16(gate . x)))     per route
//   y            = bf16(down . intermediate)                     per route
//   out          = bf16(residual + sum over the row's routes, in slot order, of weight * float(y))
// The reference groups routes by expert into tiles so that an expert's weights stream once for many rows; with at
// most 16 rows nearly every route has its expert to itself, so a route streams its expert's rows directly: a warp per
// output column, a lane per 8 consecutive weights of every super-block, effective weights d sc q - dmin m unrounded
// (as in linear_kernel), fp32 sums. The grouped tile kernel for the M >= 64 regime is not built.
#include <algorithm>

#include "sb_internal.h"
#include "sb_linear_internal.h"
#include "sb_ptx.cuh"

namespace sb {

constexpr int kMoeThreads = 256, kMoeWarps = kMoeThreads / 32;
constexpr int kMoeColsPair = 8, kMoeColsDown = 8;  // output columns a warp computes against the staged row (gate/up pass, down pass)

// scale and min of sub-block j of a Q4_K super-block from its 12 packed bytes (three words), in registers: bytes 0-3
// hold the low 6 bits of scales 0-3 (and in their top 2 bits the high bits of scales 4-7), bytes 4-7 the same for the mins,
// bytes 8-11 the low nibbles of scales 4-7 (low half) and mins 4-7 (high half).
__device__ __forceinline__ void q4k_scale_min(const uint32_t (&w)[3], uint32_t j, float &sc, float &mn) {
  const uint32_t s8 = 8 * (j & 3);
  uint32_t isc, imn;
  if (j < 4) {
    isc = (w[0] >> s8) & 63u, imn = (w[1] >> s8) & 63u;
  } else {
    isc = ((w[2] >> s8) & 0xFu) | (((w[0] >> (s8 + 6)) & 3u) << 4);
    imn = ((w[2] >> (s8 + 4)) & 0xFu) | (((w[1] >> (s8 + 6)) & 3u) << 4);
  }
  sc = float(isc), mn = float(imn);
}

// acc[m][c] += lane's share of dot(row c of matrix m, x) for NC consecutive Q4_K rows of each of NM matrices; x staged in
// shared memory as floats; lane l takes weights 32 (l / 4) + 8 (l % 4) .. + 7 of every super-block, so the lane's x values
// and their sum are fetched once per super-block for all the rows.
template <int NM, int NC>
__device__ __forceinline__ void q4k_rows_dot(const uint8_t *const (&rows)[NM], size_t row_bytes, const float *x, uint32_t k, uint32_t lane,
                                             float (&acc)[NM][NC]) {
  const uint32_t sub = lane >> 2, t0 = 8 * (lane & 3), shift = (sub & 1) * 4;
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[m][c] = 0.0f;
#pragma unroll 2
  for (uint32_t sb = 0; sb < k / 256; ++sb) {
    const float4 x0 = *reinterpret_cast<const float4 *>(x + 256 * sb + 32 * sub + t0), x1 = *reinterpret_cast<const float4 *>(x + 256 * sb + 32 * sub + t0 + 4);
    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const float xsum = ((xs[0] + xs[1]) + (xs[2] + xs[3])) + ((xs[4] + xs[5]) + (xs[6] + xs[7]));
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const uint8_t *blk = rows[m] + size_t(c) * row_bytes + size_t(sb) * 144;
        const uint32_t dm = *reinterpret_cast<const uint32_t *>(blk);
        const float d = __half2float(__ushort_as_half(uint16_t(dm & 0xffffu))), dmin = __half2float(__ushort_as_half(uint16_t(dm >> 16)));
        const uint32_t sw[3] = {*reinterpret_cast<const uint32_t *>(blk + 4), *reinterpret_cast<const uint32_t *>(blk + 8),
                                *reinterpret_cast<const uint32_t *>(blk + 12)};
        float sc, mn;
        q4k_scale_min(sw, sub, sc, mn);
        const uint2 qs = *reinterpret_cast<const uint2 *>(blk + 16 + 32 * (sub >> 1) + t0);
        float qx = 0.0f;
        const uint32_t n0 = (qs.x >> shift) & 0x0F0F0F0Fu, n1 = (qs.y >> shift) & 0x0F0F0F0Fu;  // the lane's eight codes, a byte each
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // the code as a float without a conversion instruction (quarter rate): 2^23 + q in the mantissa, minus 2^23
          const float q = __uint_as_float(0x4B000000u | __byte_perm(j < 4 ? n0 : n1, 0, 0x4440 + (j & 3))) - 8388608.0f;
          qx = fmaf(q, xs[j], qx);
        }
        acc[m][c] = fmaf(d * sc, qx, acc[m][c]);
        acc[m][c] = fmaf(-dmin * mn, xsum, acc[m][c]);
      }
  }
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
      for (int o = 16; o; o >>= 1) acc[m][c] += __shfl_xor_sync(0xffffffffu, acc[m][c], o);
}

struct MoeParams {
  SbMoeExpertArgs a;
  uint16_t *intermediate;  // bf16 [rows * routes, inter]
  uint16_t *y;             // bf16 [rows * routes, hidden]
};

// PAIR: gate and up of the route's expert over the row's input -> intermediate. Otherwise: down over the route's
// intermediate -> y. grid (rows * routes, column blocks).
template <bool PAIR> __global__ void __launch_bounds__(kMoeThreads) moe_expert_kernel(const MoeParams p) {
  constexpr int kMoeColsPerWarp = PAIR ? kMoeColsPair : kMoeColsDown;
  extern __shared__ float xrow[];
  pdl_launch_dependents();
  pdl_wait();
  const SbMoeExpertArgs &a = p.a;
  const uint32_t route = blockIdx.x, row = route / a.routes, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t k = PAIR ? a.hidden : a.inter, n = PAIR ? a.inter : a.hidden;
  const uint32_t expert = min(a.selected[route], a.experts_total - 1);
  const uint16_t *src = PAIR ? static_cast<const uint16_t *>(a.input) + size_t(row) * a.hidden : p.intermediate + size_t(route) * a.inter;
  for (uint32_t i = tid; i < k; i += kMoeThreads) xrow[i] = bf16_bits_to_float(src[i]);
  __syncthreads();
  const size_t row_bytes = size_t(k / 256) * 144;
  const uint8_t *w0 = static_cast<const uint8_t *>(PAIR ? a.gate : a.down) + size_t(expert) * n * row_bytes;
  const uint8_t *w1 = PAIR ? static_cast<const uint8_t *>(a.up) + size_t(expert) * n * row_bytes : nullptr;
  const uint32_t c0 = (blockIdx.y * kMoeWarps + warp) * kMoeColsPerWarp;
  if (c0 >= n) return;  // n is a multiple of 256, so a warp's columns are inside or outside together
  if (PAIR) {
    const uint8_t *const rows[2] = {w0 + size_t(c0) * row_bytes, w1 + size_t(c0) * row_bytes};
    float acc[2][kMoeColsPerWarp];
    q4k_rows_dot<2, kMoeColsPerWarp>(rows, row_bytes, xrow, k, lane, acc);
    if (lane < kMoeColsPerWarp) {
      float g = 0.0f, u = 0.0f;
#pragma unroll
      for (int c = 0; c < kMoeColsPerWarp; ++c)
        if (lane == uint32_t(c)) g = acc[0][c], u = acc[1][c];
      p.intermediate[size_t(route) * a.inter + c0 + lane] = float_to_bf16_bits(round_bf16(u) * silu_f(round_bf16(g)));
    }
  } else {
    const uint8_t *const rows[1] = {w0 + size_t(c0) * row_bytes};
    float acc[1][kMoeColsPerWarp];
    q4k_rows_dot<1, kMoeColsPerWarp>(rows, row_bytes, xrow, k, lane, acc);
    if (lane < kMoeColsPerWarp) {
      float v = 0.0f;
#pragma unroll
      for (int c = 0; c < kMoeColsPerWarp; ++c)
        if (lane == uint32_t(c)) v = acc[0][c];
      p.y[size_t(route) * a.hidden + c0 + lane] = float_to_bf16_bits(v);
    }
  }
}

// out = bf16(residual + sum over the row's routes in slot order of weight * float(y)).
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const SbMoeExpertArgs &a = p.a;
  const uint32_t row = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.hidden) return;
  float acc = 0.0f;
  for (uint32_t s = 0; s < a.routes; ++s)
    acc += a.weights[size_t(row) * a.routes + s] * bf16_bits_to_float(p.y[(size_t(row) * a.routes + s) * a.hidden + c]);
  const float res = a.residual ? bf16_bits_to_float(static_cast<const uint16_t *>(a.residual)[size_t(row) * a.hidden + c]) : 0.0f;
  static_cast<uint16_t *>(a.out)[size_t(row) * a.hidden + c] = float_to_bf16_bits(res + acc);
}

// ---- many rows (the rows of several lanes): routes grouped by expert, the experts' passes on the many-row kernel ----
// (MoE::addRouted's grouping: runtime/metal/kernels/shared/moe.metal:187-287, the row gather :347-365, the expert tiles
// runtime/metal/kernels/common/moe_gguf_expert_tile.h:33-84, the combine moe.metal:367-392.)
constexpr uint32_t kMoeMaxExperts = 512, kMoeMaxRoutes = 16384, kMoeGroupRows = 64, kMoeGroupThreads = 512;
struct MoeGrouping {
  uint32_t *counts;         // [0] groups, [1] row slots
  uint4 *groups;            // {expert, first slot, rows, rows padded to 16}
  uint32_t *slot_of_route;  // [rows * routes]
  uint32_t *slot_src;       // [slots] the input row a slot holds, ~0 for padding
  uint32_t *slot_self;      // [slots] the slot itself, ~0 for padding
  uint32_t *slot_group;     // [slots] group << 8 | row inside the group
};
struct MoeGroupLayout {
  uint64_t counts, groups, slot_of_route, slot_src, slot_self, slot_group, scales1, scales2, prepared1, prepared2, act, y, bytes;
  uint32_t max_groups, max_slots;
};
static MoeGroupLayout moe_group_layout(uint32_t rows, uint32_t routes, uint32_t hidden, uint32_t inter) {
  MoeGroupLayout l{};
  const uint64_t n = uint64_t(rows) * routes;
  l.max_groups = uint32_t(kMoeMaxExperts + n / kMoeGroupRows + 1);
  l.max_slots = uint32_t((n + 15ull * l.max_groups + 15) / 16 * 16);  // every group ends with fewer than 16 padding slots
  uint64_t at = 0;
  auto take = [&](uint64_t bytes) { const uint64_t here = at; at += (bytes + 255) / 256 * 256; return here; };
  l.counts = take(16), l.groups = take(uint64_t(l.max_groups) * 16), l.slot_of_route = take(n * 4);
  l.slot_src = take(uint64_t(l.max_slots) * 4), l.slot_self = take(uint64_t(l.max_slots) * 4), l.slot_group = take(uint64_t(l.max_slots) * 4);
  l.scales1 = take(uint64_t(l.max_slots) * 4), l.scales2 = take(uint64_t(l.max_slots) * 4);
  l.prepared1 = take(uint64_t(l.max_slots) * hidden * 2), l.prepared2 = take(uint64_t(l.max_slots) * inter * 2);
  l.act = take(uint64_t(l.max_slots) * inter * 2), l.y = take(uint64_t(l.max_slots) * hidden * 2);
  l.bytes = at;
  return l;
}

// One CTA of 16 warps: a stable counting sort of the routes by expert. Warp w owns a run of consecutive routes; it counts
// them by expert (a step of 32 routes at a time, equal experts found with a warp match), a thread per expert then adds the
// warps' counts in warp order, one warp lays the experts' groups out one after the other (an expert's routes in groups of
// 64, the last padded to 16 row slots), and the warps walk their runs again to number the routes: a route's place among
// its expert's routes is the earlier warps' count, plus this warp's count so far, plus its rank inside the step.
constexpr uint32_t kMoeGroupWarps = kMoeGroupThreads / 32;
// Which routes a launch takes, and the expert's place in its tensors: all of them (experts0 = 0, local = experts), or a
// rank's share under expert parallelism: experts [expert0, expert0 + local) at 0 .., the shared expert (shared_id) for rows
// [own_row0, own_row0 + own_rows) at `local`.
struct MoeShare {
  uint32_t expert0, local, shared_id, own_row0, own_rows;
};
__global__ void __launch_bounds__(kMoeGroupThreads) moe_group_kernel(const uint32_t *selected, uint32_t n, uint32_t routes, uint32_t experts, MoeGrouping g,
                                                                     uint32_t *status, MoeShare share) {
  __shared__ uint16_t warp_count[kMoeGroupWarps][kMoeMaxExperts];  // then: the place of the warp's next route of the expert
  __shared__ uint32_t count_s[kMoeMaxExperts], slot0_s[kMoeMaxExperts], group0_s[kMoeMaxExperts];
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (uint32_t i = tid; i < kMoeGroupWarps * kMoeMaxExperts; i += kMoeGroupThreads) (&warp_count[0][0])[i] = 0;
  __syncthreads();
  const uint32_t run = ((n + kMoeGroupWarps - 1) / kMoeGroupWarps + 31) / 32 * 32, first = warp * run, last = min(n, first + run);
  const uint32_t lt = (1u << lane) - 1u;
  auto expert_at = [&](uint32_t i) -> uint32_t {
    if (i >= last) return 0xffffffffu;
    const uint32_t e = selected[i];
    if (e == share.shared_id) {
      const uint32_t row = i / routes;
      return row >= share.own_row0 && row - share.own_row0 < share.own_rows ? share.local : 0xffffffffu;
    }
    if (e - share.expert0 < share.local) return e - share.expert0;
    if (share.expert0 == 0 && share.shared_id == 0xffffffffu && share.local == experts) {  // a whole block: an id outside it breaks the contract
      atomicCAS(status, 0u, uint32_t(SB_DEV_CONTRACT));
    }
    return 0xffffffffu;  // another rank's expert (or a dropped route)
  };
  for (uint32_t i0 = first; i0 < last; i0 += 32) {
    const uint32_t e = expert_at(i0 + lane);
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (e != 0xffffffffu && !(same & lt)) warp_count[warp][e] += uint16_t(__popc(same));
    __syncwarp();
  }
  __syncthreads();
  for (uint32_t e = tid; e < experts; e += kMoeGroupThreads) {
    uint32_t total = 0;
    for (uint32_t w = 0; w < kMoeGroupWarps; ++w) {
      const uint32_t c = warp_count[w][e];
      warp_count[w][e] = uint16_t(total);
      total += c;
    }
    count_s[e] = total;
  }
  __syncthreads();
  if (warp == 0) {
    // 32 experts a round: their group counts and padded slots scanned over the lanes
    uint32_t slot = 0, group = 0;
    for (uint32_t e0 = 0; e0 < experts; e0 += 32) {
      const uint32_t e = e0 + lane, c = e < experts ? count_s[e] : 0;
      const uint32_t groups = (c + kMoeGroupRows - 1) / kMoeGroupRows, slots = (c + 15) / 16 * 16;
      uint32_t gs = groups, ss = slots;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, gs, o), b = __shfl_up_sync(0xffffffffu, ss, o);
        if (lane >= uint32_t(o)) gs += a, ss += b;
      }
      const uint32_t my_group = group + gs - groups, my_slot = slot + ss - slots;
      if (e < experts) {
        slot0_s[e] = my_slot, group0_s[e] = my_group;
        for (uint32_t k = 0; k < groups; ++k) {
          const uint32_t rows = min(c - k * kMoeGroupRows, kMoeGroupRows);
          g.groups[my_group + k] = make_uint4(e, my_slot + k * kMoeGroupRows, rows, (rows + 15) / 16 * 16);
        }
        // the padding slots behind the expert's last route
        const uint32_t lastg = my_group + (groups ? groups - 1 : 0);
        for (uint32_t r = c; r < slots; ++r) {
          g.slot_src[my_slot + r] = 0xffffffffu, g.slot_self[my_slot + r] = 0xffffffffu;
          g.slot_group[my_slot + r] = (lastg << 8) | (r - (lastg - my_group) * kMoeGroupRows);
        }
      }
      group += __shfl_sync(0xffffffffu, gs, 31), slot += __shfl_sync(0xffffffffu, ss, 31);
    }
    if (lane == 0) g.counts[0] = group, g.counts[1] = slot;
  }
  __syncthreads();
  for (uint32_t i0 = first; i0 < last; i0 += 32) {
    const uint32_t i = i0 + lane, e = expert_at(i);
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (e != 0xffffffffu) {
      const uint32_t j = warp_count[warp][e] + __popc(same & lt), slot = slot0_s[e] + j;  // (full groups carry no padding)
      g.slot_of_route[i] = slot;
      g.slot_src[slot] = i / routes, g.slot_self[slot] = slot;
      g.slot_group[slot] = ((group0_s[e] + j / kMoeGroupRows) << 8) | (j % kMoeGroupRows);
    } else if (i < last) {
      g.slot_of_route[i] = 0xffffffffu;
    }
    __syncwarp();
    if (e != 0xffffffffu && !(same & lt)) warp_count[warp][e] += uint16_t(__popc(same));
    __syncwarp();
  }
}

// out = bf16(residual + sum over the row's routes in slot order of weight * float(y)), y at the routes' row slots.
// partial != 0: the routes the launch took only (slot_of_route says which: the others hold ~0), fp32 sums without the residual.
__global__ void __launch_bounds__(256) moe_combine_grouped_kernel(const SbMoeExpertArgs a, const uint32_t *slot_of_route, const uint16_t *y, uint32_t partial) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t row = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= a.hidden) return;
  float acc0 = 0.0f, acc1 = 0.0f;
  for (uint32_t s = 0; s < a.routes; ++s) {
    const uint32_t route = row * a.routes + s, slot = slot_of_route[route];
    if (slot == 0xffffffffu) continue;  // (not taken by the grouping)
    const float w = a.weights[route];
    const uint32_t pair = *reinterpret_cast<const uint32_t *>(y + size_t(slot) * a.hidden + c);
    acc0 += w * bf16_bits_to_float(pair & 0xffffu), acc1 += w * bf16_bits_to_float(pair >> 16);
  }
  if (partial) {
    *reinterpret_cast<float2 *>(static_cast<float *>(a.out) + size_t(row) * a.hidden + c) = make_float2(acc0, acc1);
    return;
  }
  float r0 = 0.0f, r1 = 0.0f;
  if (a.residual) {
    const uint32_t pair = *reinterpret_cast<const uint32_t *>(static_cast<const uint16_t *>(a.residual) + size_t(row) * a.hidden + c);
    r0 = bf16_bits_to_float(pair & 0xffffu), r1 = bf16_bits_to_float(pair >> 16);
  }
  *reinterpret_cast<uint32_t *>(static_cast<uint16_t *>(a.out) + size_t(row) * a.hidden + c) =
      uint32_t(float_to_bf16_bits(r0 + acc0)) | (uint32_t(float_to_bf16_bits(r1 + acc1)) << 16);
}

template <class K> static int launch_moe(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const MoeParams &p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = ctx().pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" uint64_t sb_moe_scratch_bytes(uint32_t rows, uint32_t routes, uint32_t hidden, uint32_t inter) {
  if (rows > 16) return moe_group_layout(rows, routes, hidden, inter).bytes;
  return uint64_t(rows) * routes * (uint64_t(hidden) + inter) * 2 + 256;
}

// More than 16 rows: group the routes by expert, gather and convert each group's rows, the experts' one-pass gate/up and
// down on the many-row kernel over the groups, and the combine.
static int moe_experts_grouped(cudaStream_t s, const SbMoeExpertArgs *a, const MoeShare *part = nullptr) {
  const uint64_t n = uint64_t(a->rows) * a->routes;
  SB_REQUIRE(n <= kMoeMaxRoutes && a->experts_total <= kMoeMaxExperts, "sb_moe_experts: %u rows x %u routes over %u experts (up to %u routes, %u experts)",
             a->rows, a->routes, a->experts_total, kMoeMaxRoutes, kMoeMaxExperts);
  SB_REQUIRE(a->inter % 128 == 0 && a->hidden % 256 == 0, "sb_moe_experts: many rows need an intermediate width in 128s and a hidden width in 256s");
  const MoeGroupLayout l = moe_group_layout(a->rows, a->routes, a->hidden, a->inter);
  uint8_t *base = static_cast<uint8_t *>(a->scratch);
  auto at = [&](uint64_t off) { return base + off; };
  MoeGrouping g{reinterpret_cast<uint32_t *>(at(l.counts)), reinterpret_cast<uint4 *>(at(l.groups)), reinterpret_cast<uint32_t *>(at(l.slot_of_route)),
                reinterpret_cast<uint32_t *>(at(l.slot_src)), reinterpret_cast<uint32_t *>(at(l.slot_self)), reinterpret_cast<uint32_t *>(at(l.slot_group))};
  const bool pdl = ctx().pdl;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1), cfg.blockDim = dim3(kMoeGroupThreads), cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
    const MoeShare share = part ? *part : MoeShare{0, a->experts_total, 0xffffffffu, 0, 0};
    SB_CUDA(cudaLaunchKernelEx(&cfg, moe_group_kernel, a->selected, uint32_t(n), a->routes, a->experts_total, g, ctx().status_dev, share));
  }
  WidePrepareGroupedArgs c1{a->input, a->hidden, a->hidden, g.slot_src, g.slot_group, g.counts + 1, l.max_slots, g.groups, at(l.prepared1),
                            reinterpret_cast<float *>(at(l.scales1)), pdl};
  int st = launch_wide_prepare_grouped(s, c1);
  if (st != SB_OK) return st;
  WideGroupedArgs pair{a->gate, a->up, a->experts_total, a->inter, a->hidden, at(l.prepared1), reinterpret_cast<const float *>(at(l.scales1)), g.groups,
                       g.counts, l.max_groups, kMoeGroupRows, at(l.act), a->inter, pdl};
  st = launch_linear_wide_grouped(s, pair);
  if (st != SB_OK) return st;
  WidePrepareGroupedArgs c2{at(l.act), a->inter, a->inter, g.slot_self, g.slot_group, g.counts + 1, l.max_slots, g.groups, at(l.prepared2),
                            reinterpret_cast<float *>(at(l.scales2)), pdl};
  st = launch_wide_prepare_grouped(s, c2);
  if (st != SB_OK) return st;
  WideGroupedArgs down{a->down, nullptr, a->experts_total, a->hidden, a->inter, at(l.prepared2), reinterpret_cast<const float *>(at(l.scales2)), g.groups,
                       g.counts, l.max_groups, kMoeGroupRows, at(l.y), a->hidden, pdl};
  st = launch_linear_wide_grouped(s, down);
  if (st != SB_OK) return st;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a->hidden / 2 + 255) / 256, a->rows), cfg.blockDim = dim3(256), cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, moe_combine_grouped_kernel, *a, static_cast<const uint32_t *>(g.slot_of_route), reinterpret_cast<const uint16_t *>(at(l.y)),
                             part ? 1u : 0u));
  return SB_OK;
}

static int moe_check(const SbMoeExpertArgs *a, const char *who);

extern "C" int sb_moe_experts_partial(void *stream, const SbMoeExpertArgs *a, uint32_t expert0, uint32_t experts_local, uint32_t shared_id,
                                      uint32_t own_row0, uint32_t own_rows) {
  SB_NEED_DEVICE();
  const int st = moe_check(a, "sb_moe_experts_partial");
  if (st != SB_OK) return st;
  const bool shared = shared_id != 0xffffffffu;
  SB_REQUIRE(experts_local >= 1 && a->experts_total == experts_local + (shared ? 1u : 0u), "sb_moe_experts_partial: %u experts here (+ the shared one) against %u in the tensors",
             experts_local, a->experts_total);
  SB_REQUIRE(!shared || (shared_id >= expert0 + experts_local || shared_id < expert0), "sb_moe_experts_partial: the shared expert's id lies inside the rank's range");
  SB_REQUIRE(own_row0 + own_rows <= a->rows, "sb_moe_experts_partial: own rows [%u, %u) of %u", own_row0, own_row0 + own_rows, a->rows);
  const MoeShare share{expert0, experts_local, shared_id, own_row0, own_rows};
  return moe_experts_grouped(as_stream(stream), a, &share);
}

extern "C" int sb_moe_experts(void *stream, const SbMoeExpertArgs *a) {
  SB_NEED_DEVICE();
  const int valid = moe_check(a, "sb_moe_experts");
  if (valid != SB_OK) return valid;
  if (a->rows > 16) return moe_experts_grouped(as_stream(stream), a);
  MoeParams p{*a, static_cast<uint16_t *>(a->scratch), static_cast<uint16_t *>(a->scratch) + size_t(a->rows) * a->routes * a->inter};
  const uint32_t routes = a->rows * a->routes, pair_block = kMoeWarps * kMoeColsPair, down_block = kMoeWarps * kMoeColsDown;
  cudaStream_t s = as_stream(stream);
  int st = launch_moe(moe_expert_kernel<true>, dim3(routes, (a->inter + pair_block - 1) / pair_block), dim3(kMoeThreads), size_t(a->hidden) * 4, s, p);
  if (st != SB_OK) return st;
  st = launch_moe(moe_expert_kernel<false>, dim3(routes, (a->hidden + down_block - 1) / down_block), dim3(kMoeThreads), size_t(a->inter) * 4, s, p);
  if (st != SB_OK) return st;
  return launch_moe(moe_combine_kernel, dim3((a->hidden + 255) / 256, a->rows), dim3(256), 0, s, p);
}

static int moe_check(const SbMoeExpertArgs *a, const char *who) {
  SB_REQUIRE(a && a->input && a->selected && a->weights && a->gate && a->up && a->down && a->scratch && a->out, "%s: null pointer", who);
  SB_REQUIRE(a->format == SB_FMT_Q4K, "%s: experts in format %u (Q4_K only)", who, a->format);
  SB_REQUIRE(a->rows >= 1 && a->routes >= 1 && a->routes <= 32, "%s: %u rows x %u routes (1..32)", who, a->rows, a->routes);
  SB_REQUIRE(a->hidden && a->hidden % 256 == 0 && a->inter && a->inter % 256 == 0 && a->hidden <= 8192 && a->inter <= 8192,
             "%s: hidden %u and intermediate %u are multiples of 256 up to 8192", who, a->hidden, a->inter);
  SB_REQUIRE(a->experts_total >= 1, "%s: no experts", who);
  SB_REQUIRE(((reinterpret_cast<uintptr_t>(a->gate) | reinterpret_cast<uintptr_t>(a->up) | reinterpret_cast<uintptr_t>(a->down) |
               reinterpret_cast<uintptr_t>(a->scratch)) & 15) == 0,
             "%s: expert tensors and scratch must be 16-byte aligned", who);
  return SB_OK;
}
