// Gated-DeltaNet verify step of one lane and one layer with fp32 state and warp-shuffle reductions.
//
// Takes the place of the reference's verify_gdn_fused* kernels (runtime/metal/kernels/decode/gdn.metal:
// prologue :139-264, fold :270-298, chain scan :312-415, gate :489-526; primitives
// runtime/metal/kernels/common/gdn_primitives.h:63-106) and of ops::GDN::addDecode / addFold
// (runtime/ops/GDN.cpp:225-328).
//
//   grid     (4, value_heads): the reference runs one threadgroup per value head (48 on the 27B shape,
//            too few for 148 SMs); a head's 128 state rows (value dimensions) are independent given
//            k, v and the gates, so each CTA takes 32 of them
//   CTA      256 threads; warp w owns state rows 4w..4w+3 of the CTA's 32, each lane four fp32 key
//            columns of each row (16 registers of state); dot products are butterfly shuffles
//   steps    (1) conv history = last three input rows before the block (carried rows ++ pending rows);
//            (2) conv + SiLU, q/k RMS norm and scales (2^-7, 128^-1/2), beta and decay per row;
//            (3) fold the pending rows into the state -> committed state stored; (4) chain scan from the
//            committed state, outputs only; (5) the head's last CTA normalises (RMS over the 128 value
//            dimensions), gates by silu(z) and writes the hidden rows; (6) this step's tape
//   rollback the state after the block is never stored: the caller passes how many tape rows were accepted
//            (pending_rows, or a device word written by sb_accept) to the next step, which folds them
#include <algorithm>
#include <atomic>
#include <cooperative_groups.h>

#include "sb_internal.h"
#include "sb_ptx.cuh"
#include "sb_dot.cuh"

namespace sb {

constexpr int kGdnThreads = 256;
constexpr int kGdnRows = 16;      // rows of a verify block
constexpr int kGdnSplit = 4;      // CTAs per value head
constexpr int kGdnVd = 128 / kGdnSplit;  // value dimensions per CTA
constexpr int kD = 128, kTaps = 4;

struct GdnParams {
  SbGdnArgs a;
  uint16_t *scratch;    // bf16 [value_heads][16][128] recurrent outputs before the gate
  uint32_t *counters;   // [value_heads]
};

// Lane blockIdx.z's view of a launch over several lanes: its 16 row slots of the row-indexed buffers, its cell, tapes and
// pending words, its share of the scratch and the counters.
__device__ __forceinline__ GdnParams gdn_lane_view(GdnParams p) {
  const uint32_t z = blockIdx.z;
  if (z == 0 && gridDim.z == 1) return p;
  SbGdnArgs &a = p.a;
  const size_t KW = size_t(a.key_heads) * 128, VW = size_t(a.value_heads) * 128, C = 2 * KW + VW, R = 16 * size_t(z);
  auto rows16 = [&](const void *q, size_t stride) { return q ? static_cast<const void *>(static_cast<const uint16_t *>(q) + R * stride) : q; };
  a.qkvz = rows16(a.qkvz, a.qkvz_stride), a.b = rows16(a.b, a.ab_stride), a.a = rows16(a.a, a.ab_stride);
  a.gate_input = rows16(a.gate_input, a.gate_input_stride);
  a.hidden = const_cast<void *>(rows16(a.hidden, a.hidden_stride));
  if (a.tree) a.tree = static_cast<const uint2 *>(a.tree) + R;
  a.conv_state_in = static_cast<const uint16_t *>(a.conv_state_in) + size_t(z) * 3 * C;
  a.conv_state_out = static_cast<uint16_t *>(a.conv_state_out) + size_t(z) * 3 * C;
  a.state_in += size_t(z) * a.value_heads * 128 * 128, a.state_out += size_t(z) * a.value_heads * 128 * 128;
  auto tape = [&](SbGdnTape &t) {
    if (t.inputs) t.inputs = static_cast<uint16_t *>(t.inputs) + R * C;
    if (t.k) t.k = static_cast<uint16_t *>(t.k) + R * KW;
    if (t.v) t.v = static_cast<uint16_t *>(t.v) + R * VW;
    if (t.beta) t.beta = static_cast<uint16_t *>(t.beta) + R * a.value_heads;
    if (t.decay) t.decay += R * a.value_heads;
  };
  tape(a.pending), tape(a.step);
  if (a.pending_rows_dev) a.pending_rows_dev += z;
  if (a.pending_path_dev) a.pending_path_dev += z;
  p.scratch += size_t(z) * a.value_heads * 16 * 128;
  p.counters += size_t(z) * a.value_heads;
  return p;
}

// Row of the n-th token (from the anchor) of a path mask.
__device__ __forceinline__ uint32_t path_row(uint32_t path, uint32_t n) {
  for (uint32_t i = 0; i < n; ++i) path &= path - 1;
  return path ? uint32_t(__ffs(int(path))) - 1u : 0u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The kGdnSplit CTAs of a value head form a cluster: the fused gate projection is divided among them by rows and
// meets in every CTA's shared memory.
// kTree: the rows may form a tree and the pending path may be any row mask (tap tables, transformed queries); without
// it the rows are a chain and the pending rows the tape's first, which is the verify step's usual case and keeps the
// indirections out of its kernel.
// kResident: CTAs per SM the registers are held to. A launch of one lane (192 CTAs on the 27B shape) runs fastest with the 96
// registers that two per SM allow; a launch of several lanes has CTAs to spare, and four per SM at 64 registers hide more
// of the chain's latency (measured on 8 lanes: the 27B step 25.95 ms at two per SM, 24.69 at three, 24.51 at four).
template <bool kTree, int kResident = 2>
__global__ void __cluster_dims__(kGdnSplit, 1, 1) __launch_bounds__(kGdnThreads, kResident) gdn_kernel(const GdnParams p_in) {
  const GdnParams p = gdn_lane_view(p_in);  // (one lane: p_in itself)
  const SbGdnArgs &a = p.a;
  __shared__ float q_s[kGdnRows][kD], k_s[kGdnRows][kD], pk_s[kGdnRows][kD];
  __shared__ float v_s[kGdnRows][kGdnVd], pv_s[kGdnRows][kGdnVd], o_s[kGdnRows][kGdnVd];
  __shared__ float beta_s[kGdnRows], decay_s[kGdnRows], pbeta_s[kGdnRows], pdecay_s[kGdnRows];
  __shared__ float gate_s[kDotGroups][kGdnRows][2];  // group partial sums of the head's b and a per row (fused gate projection)
  __shared__ __align__(16) uint16_t in_s[kGdnRows + 3][2 * kD + kGdnVd];
  __shared__ uint2 w_s[2 * kD + kGdnVd];
  __shared__ uint32_t s_last;
  __shared__ uint8_t tap_s[kGdnRows][kTaps];   // where in in_s a row's four convolution taps lie (its path's last tokens)
  __shared__ uint32_t path_s[kGdnRows];         // the row's path from the anchor, itself included
  __shared__ float coef_s[kGdnRows][kGdnRows];  // tree rows: the coefficient of each row of the path
  pdl_launch_dependents();
  const bool fused_gates = a.gate_weight && a.rows > 0;
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // "this CTA runs", waited for before the first store into a peer CTA
  bool peers_run = false;
  auto wait_peers_run = [&] {
    if (!peers_run) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    peers_run = true;
  };
  const uint32_t vs = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t KH = a.key_heads, VH = a.value_heads, KW = KH * kD, VW = VH * kD, C = 2 * KW + VW;
  const uint32_t per_key = VH / KH, kh = h / per_key, vd0 = vs * kGdnVd;
  const uint32_t rows = a.rows;
  const uint16_t *qkvz = static_cast<const uint16_t *>(a.qkvz);
  const uint16_t *conv_w = static_cast<const uint16_t *>(a.conv_w);
  const uint16_t *cs_in = static_cast<const uint16_t *>(a.conv_state_in);
  const uint16_t *pin = static_cast<const uint16_t *>(a.pending.inputs);
  const bool qk_writer = h % per_key == 0 && vs == 0;

  // The state of this warp's 4 value dimensions, requested first so the latency hides behind the prologue and, where
  // the caller allows it (below), before the wait for the kernel ahead: in the model's step the cell was written a
  // whole step ago, and this CTA may be resident while the projection before it drains.
  // lane l holds row 4 warp + l / 8, key columns 32 c + 4 (l % 8) .. + 3 for c = 0..3 (the 8 lanes of a row read 128
  // contiguous bytes at a time, from global and from shared memory), so a dot product over the 128 key columns
  // is 16 multiply-adds in the lane and three butterfly rounds over its 8-lane group.
  float S[16];
  const uint32_t srow = 4 * warp + (lane >> 3), scol = 4 * (lane & 7);
  const size_t sbase = (size_t(h) * kD + vd0 + srow) * kD + scol;
  auto load_state = [&] {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float4 s4 = *reinterpret_cast<const float4 *>(a.state_in + sbase + 32 * c);
      S[4 * c] = s4.x, S[4 * c + 1] = s4.y, S[4 * c + 2] = s4.z, S[4 * c + 3] = s4.w;
    }
  };
  // Only a caller that vouches for the cell (SB_GDN_STATE_SETTLED: nothing still running on the stream writes
  // state_in) gets the early load; otherwise the launch ahead may be the one that produced the cell (a fold
  // followed at once by a step on the swapped cells), and the load waits for it like every other read.
  const bool settled = (a.flags & SB_GDN_STATE_SETTLED) != 0;
  if (settled) load_state();
  pdl_wait();
  if (!settled) load_state();
  // The previous step's accepted path in its tape: a row mask, or the tape's first rows.
  uint32_t pending_path = a.pending_path_dev ? *a.pending_path_dev : a.pending_path;
  if (!a.pending_path_dev && !a.pending_path) {
    const uint32_t n = a.pending_rows_dev ? min(*a.pending_rows_dev, uint32_t(kGdnRows)) : a.pending_rows;
    pending_path = (1u << n) - 1u;
  }
  pending_path &= (1u << kGdnRows) - 1u;
  const uint32_t pending = uint32_t(__popc(pending_path));
  auto pending_row = [&](uint32_t n) { return kTree ? path_row(pending_path, n) : n; };
  if (kTree && tid < rows) {
    const uint32_t path = (a.tree ? static_cast<const uint2 *>(a.tree)[tid].x & ((2u << tid) - 1u) : (2u << tid) - 1u) | (1u << tid);
    const int depth = __popc(path) - 1;
    for (int tap = 0; tap < kTaps; ++tap) {
      const int at = depth - 3 + tap;  // the tap's token, counted from the anchor; before it: the carried history
      tap_s[tid][tap] = uint8_t(at < 0 ? 3 + at : 3 + int(path_row(path, uint32_t(at))));
    }
    path_s[tid] = path;
  }
  // Fused gate projection: this CTA takes rows 4 vs .. 4 vs + 3; warp w computes group w's partial sums of those rows x
  // {b, a} over the layer's normalised input and stores them into all four CTAs of the head; the rows' threads add the
  // 8 groups in order below (the order of sb_linear_f32, so the bits agree with the unfused way).
  if (fused_gates) {
    static_assert(kGdnThreads / 32 == kDotGroups, "one warp per group of the dot product");
    static_assert(kGdnRows == 4 * kGdnSplit, "four rows of the gate projection per CTA of the head");
    const float *const wrow[2] = {a.gate_weight + size_t(h) * a.gate_k, a.gate_weight + size_t(VH + h) * a.gate_k};
    const uint16_t *gx = static_cast<const uint16_t *>(a.gate_input);
    const uint16_t *xrow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) xrow[r] = gx + size_t(min(4 * vs + uint32_t(r), rows - 1)) * a.gate_input_stride;
    float d[4][2];
    warp_dot_group_f32_bf16<2, 4>(wrow, xrow, a.gate_k, lane, warp, d);
    wait_peers_run();
    if (lane < kGdnSplit) {
      cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
      float *remote = cluster.map_shared_rank(&gate_s[0][0][0], lane);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        remote[(warp * kGdnRows + 4 * vs + r) * 2] = d[r][0];
        remote[(warp * kGdnRows + 4 * vs + r) * 2 + 1] = d[r][1];
      }
    }
  }
  // Conv inputs of this CTA's channels (q and k of the key head, 32 value dimensions) for history rows
  // -3..-1 and the block's rows, staged with 16-byte loads: in_s[3 + row][local channel]. History row i
  // (0..2, oldest first) is row pending - 3 + i of (carried rows ++ pending rows).
  constexpr int kLocal = 2 * kD + kGdnVd;  // 288 local channels
  const uint32_t chan0[3] = {kh * kD, KW + kh * kD, 2 * KW + h * kD + vd0};
  auto global_channel = [&](uint32_t lc) { return lc < kD ? chan0[0] + lc : lc < 2 * kD ? chan0[1] + lc - kD : chan0[2] + lc - 2 * kD; };
  for (uint32_t i = tid; i < (3 + rows) * (kLocal / 8); i += kGdnThreads) {
    const uint32_t r = i / (kLocal / 8), lc = (i % (kLocal / 8)) * 8, ch = global_channel(lc);
    const uint16_t *src;
    if (r >= 3) {
      src = qkvz + size_t(r - 3) * a.qkvz_stride + ch;
    } else {
      const int hsrc = int(pending) - 3 + int(r);
      src = hsrc >= 0 ? pin + size_t(pending_row(uint32_t(hsrc))) * C + ch : cs_in + size_t(3 + hsrc) * C + ch;
    }
    *reinterpret_cast<uint4 *>(&in_s[r][lc]) = *reinterpret_cast<const uint4 *>(src);
  }
  for (uint32_t lc = tid; lc < kLocal; lc += kGdnThreads)
    w_s[lc] = *reinterpret_cast<const uint2 *>(conv_w + size_t(global_channel(lc)) * kTaps);
  if (fused_gates) cooperative_groups::this_cluster().sync();  // the gates of all rows are here (and the CTA's staging is complete)
  else __syncthreads();
  auto conv = [&](uint32_t row, uint32_t lc) -> float {
    const uint2 wv = w_s[lc];
    const float w[4] = {bf16_bits_to_float(wv.x & 0xffffu), bf16_bits_to_float(wv.x >> 16), bf16_bits_to_float(wv.y & 0xffffu),
                        bf16_bits_to_float(wv.y >> 16)};
    float value = 0.0f;
#pragma unroll
    for (int tap = 0; tap < kTaps; ++tap) value = __fadd_rn(value, __fmul_rn(bf16_bits_to_float(in_s[kTree ? uint32_t(tap_s[row][tap]) : row + tap][lc]), w[tap]));
    value = round_bf16(value);
    return round_bf16(silu_f(value));
  };

  // (2) conv outputs: this CTA's 32 value dimensions, and q, k of the key head (128 each) for rows 4 vs .. 4 vs + 3 only:
  // the head's four CTAs divide the rows, normalise their own and store the result into all four (below).
  const uint32_t qk_row0 = min(4 * vs, rows), qk_rows = min(4 * vs + 4, rows) - qk_row0;
#pragma unroll 2
  for (uint32_t i = tid; i < qk_rows * kD; i += kGdnThreads) {
    const uint32_t r = qk_row0 + i / kD, d = i % kD;
    q_s[r][d] = conv(r, d);
    k_s[r][d] = conv(r, kD + d);
  }
#pragma unroll 2
  for (uint32_t i = tid; i < rows * kGdnVd; i += kGdnThreads) {
    const uint32_t r = i / kGdnVd, d = i % kGdnVd;
    v_s[r][d] = conv(r, 2 * kD + d);
  }
  // pending rows' keys, values and gates from their tape
  for (uint32_t i = tid; i < pending * kD; i += kGdnThreads)
    pk_s[i / kD][i % kD] =
        bf16_bits_to_float(static_cast<const uint16_t *>(a.pending.k)[size_t(pending_row(i / kD)) * KW + kh * kD + i % kD]);
  for (uint32_t i = tid; i < pending * kGdnVd; i += kGdnThreads)
    pv_s[i / kGdnVd][i % kGdnVd] = bf16_bits_to_float(
        static_cast<const uint16_t *>(a.pending.v)[size_t(pending_row(i / kGdnVd)) * VW + h * kD + vd0 + i % kGdnVd]);
  if (tid < pending) {
    const uint32_t trow = pending_row(tid);
    pbeta_s[tid] = bf16_bits_to_float(static_cast<const uint16_t *>(a.pending.beta)[size_t(trow) * VH + h]);
    pdecay_s[tid] = a.pending.decay[size_t(trow) * VH + h];
  }
  if (tid < rows) {
    float bb, aa;
    if (a.gate_weight) {
      bb = gate_s[0][tid][0], aa = gate_s[0][tid][1];
#pragma unroll
      for (int g = 1; g < kDotGroups; ++g) bb += gate_s[g][tid][0], aa += gate_s[g][tid][1];
      bb = round_bf16(bb), aa = round_bf16(aa);
    } else {
      bb = bf16_bits_to_float(static_cast<const uint16_t *>(a.b)[size_t(tid) * a.ab_stride + h]);
      aa = bf16_bits_to_float(static_cast<const uint16_t *>(a.a)[size_t(tid) * a.ab_stride + h]);
    }
    const float be = round_bf16(sigmoid_f(bb));
    const float x = round_bf16(__fadd_rn(aa, bf16_bits_to_float(static_cast<const uint16_t *>(a.dt_bias)[h])));
    const float sp = round_bf16(fmaxf(x, 0.0f) + log2f(1.0f + exp2f(-1.44269504089f * fabsf(x))) * 0.69314718056f);
    const float de = expf(a.a_scale[h] * sp);
    beta_s[tid] = be;
    decay_s[tid] = de;
    if (vs == 0) {
      static_cast<uint16_t *>(a.step.beta)[size_t(tid) * VH + h] = float_to_bf16_bits(be);
      a.step.decay[size_t(tid) * VH + h] = de;
    }
  }
  __syncthreads();
  // q/k RMS norm over the head's 128 dimensions: a warp per (row, q or k); 4 dims per lane in order,
  // then the butterfly.
  wait_peers_run();
  cooperative_groups::cluster_group head_ctas = cooperative_groups::this_cluster();
  for (uint32_t task = warp; task < 2 * qk_rows; task += kGdnThreads / 32) {
    const uint32_t r = qk_row0 + (task >> 1);
    float *vec = (task & 1) ? k_s[r] : q_s[r];
    float ss = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float x = vec[32 * g + lane];
      ss += warp_sum(x * x);
    }
    const float inv = rsqrtf(ss / float(kD) + 1e-6f);
    const float post = (task & 1) ? 0.08838834765f : 0.0078125f;
    float out[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) out[g] = round_bf16(round_bf16(vec[32 * g + lane] * inv) * post);
#pragma unroll
    for (int peer = 0; peer < kGdnSplit; ++peer) {
      float *remote = head_ctas.map_shared_rank(vec, peer);
#pragma unroll
      for (int g = 0; g < 4; ++g) remote[32 * g + lane] = out[g];
    }
  }
  head_ctas.sync();  // every row's q and k are in every CTA of the head
  // (6) tape and carried conv rows, from the staged inputs.
  {
    uint16_t *tin = static_cast<uint16_t *>(a.step.inputs), *cs_out = static_cast<uint16_t *>(a.conv_state_out);
    for (uint32_t i = tid; i < (3 + rows) * kLocal; i += kGdnThreads) {
      const uint32_t r = i / kLocal, lc = i % kLocal;
      if (lc < 2 * kD && !qk_writer) continue;
      const uint32_t ch = global_channel(lc);
      if (r < 3) cs_out[size_t(r) * C + ch] = in_s[r][lc];
      else tin[size_t(r - 3) * C + ch] = in_s[r][lc];
    }
    for (uint32_t i = tid; i < rows * kGdnVd; i += kGdnThreads)
      static_cast<uint16_t *>(a.step.v)[size_t(i / kGdnVd) * VW + h * kD + vd0 + i % kGdnVd] = float_to_bf16_bits(v_s[i / kGdnVd][i % kGdnVd]);
    if (qk_writer)
      for (uint32_t i = tid; i < rows * kD; i += kGdnThreads)
        static_cast<uint16_t *>(a.step.k)[size_t(i / kD) * KW + kh * kD + i % kD] = float_to_bf16_bits(k_s[i / kD][i % kD]);
  }

  // (3) + (4): one delta-rule step on the lane's 16 state values (runtime/metal/kernels/common/gdn_primitives.h:63-97):
  // S *= decay; mem = S k; delta = (v - mem) beta; S += delta k^T; out = S q.
  auto group_sum = [&](float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
  };
  auto advance = [&](const float *key, const float *val, float d, float b, const float *query, float *out) {
    float kk[16];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float4 k4 = *reinterpret_cast<const float4 *>(key + scol + 32 * c);
      kk[4 * c] = k4.x, kk[4 * c + 1] = k4.y, kk[4 * c + 2] = k4.z, kk[4 * c + 3] = k4.w;
    }
    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      S[i] *= d;
      part[i & 3] = fmaf(S[i], kk[i], part[i & 3]);
    }
    const float mem = group_sum((part[0] + part[1]) + (part[2] + part[3]));
    const float delta = (val[srow] - mem) * b;
    if (query) {
      float qq[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 q4 = *reinterpret_cast<const float4 *>(query + scol + 32 * c);
        qq[4 * c] = q4.x, qq[4 * c + 1] = q4.y, qq[4 * c + 2] = q4.z, qq[4 * c + 3] = q4.w;
      }
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        S[i] = fmaf(kk[i], delta, S[i]);
        acc[i & 3] = fmaf(S[i], qq[i], acc[i & 3]);
      }
      const float res = group_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
      if ((lane & 7) == 0) out[srow] = res;
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) S[i] = fmaf(kk[i], delta, S[i]);
    }
  };
  for (uint32_t t = 0; t < pending; ++t) advance(pk_s[t], pv_s[t], pdecay_s[t], pbeta_s[t], nullptr, nullptr);
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<float4 *>(a.state_out + sbase + 32 * c) = make_float4(S[4 * c], S[4 * c + 1], S[4 * c + 2], S[4 * c + 3]);
  bool chain = true;
  if (kTree)
    for (uint32_t r = 0; r < rows; ++r) chain = chain && path_s[r] == (2u << r) - 1u;
  if (!kTree || chain) {
    for (uint32_t t = 0; t < rows; ++t) advance(k_s[t], v_s[t], decay_s[t], beta_s[t], q_s[t], o_s[t]);
  } else {
    // Tree rows (runtime/metal/kernels/decode/gdn.metal:418-478): a row's output is the state after its own path,
    // S_committed z + sum_j c_j v_j, with the query taken up the path: c_j = beta_j (k_j . z_j), z_j-1 = d_j (z_j - c_j k_j).
    // A warp transforms rows warp and warp + 8 (four dimensions a lane); the transformed queries take the queries' place.
    float z[2][4], cf[2] = {0.0f, 0.0f};
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const uint32_t r = warp + 8 * pass;
      if (r >= rows) continue;
      const float4 q4 = *reinterpret_cast<const float4 *>(&q_s[r][4 * lane]);
      z[pass][0] = q4.x, z[pass][1] = q4.y, z[pass][2] = q4.z, z[pass][3] = q4.w;
      for (uint32_t up = path_s[r]; up;) {
        const uint32_t row = 31u - uint32_t(__clz(int(up)));
        up &= ~(1u << row);
        const float4 k4 = *reinterpret_cast<const float4 *>(&k_s[row][4 * lane]);
        const float c = beta_s[row] * warp_sum(k4.x * z[pass][0] + k4.y * z[pass][1] + k4.z * z[pass][2] + k4.w * z[pass][3]);
        const float d = decay_s[row];
        z[pass][0] = d * (z[pass][0] - c * k4.x), z[pass][1] = d * (z[pass][1] - c * k4.y);
        z[pass][2] = d * (z[pass][2] - c * k4.z), z[pass][3] = d * (z[pass][3] - c * k4.w);
        if (lane == row) cf[pass] = c;
      }
    }
    __syncthreads();  // every warp has read the queries it needs
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const uint32_t r = warp + 8 * pass;
      if (r >= rows) continue;
      *reinterpret_cast<float4 *>(&q_s[r][4 * lane]) = make_float4(z[pass][0], z[pass][1], z[pass][2], z[pass][3]);
      if (lane < kGdnRows) coef_s[r][lane] = cf[pass];
    }
    __syncthreads();
    for (uint32_t t = 0; t < rows; ++t) {
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float4 q4 = *reinterpret_cast<const float4 *>(&q_s[t][scol + 32 * c]);
        acc[0] = fmaf(S[4 * c], q4.x, acc[0]), acc[1] = fmaf(S[4 * c + 1], q4.y, acc[1]);
        acc[2] = fmaf(S[4 * c + 2], q4.z, acc[2]), acc[3] = fmaf(S[4 * c + 3], q4.w, acc[3]);
      }
      float res = group_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
      if ((lane & 7) == 0) {
        for (uint32_t up = path_s[t]; up; up &= up - 1) {
          const uint32_t j = uint32_t(__ffs(int(up))) - 1u;
          res = fmaf(coef_s[t][j], v_s[j][srow], res);
        }
        o_s[t][srow] = res;
      }
    }
  }
  __syncthreads();
  // recurrent outputs (bf16) of this CTA's value dimensions -> scratch
  for (uint32_t i = tid; i < rows * kGdnVd; i += kGdnThreads)
    p.scratch[(size_t(h) * kGdnRows + i / kGdnVd) * kD + vd0 + i % kGdnVd] = float_to_bf16_bits(o_s[i / kGdnVd][i % kGdnVd]);
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&p.counters[h], 1u) == kGdnSplit - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // (5) gated RMSNorm: a warp per row, dimensions 32 g + lane, the four partial sums added in order.
  const uint32_t out_head = a.tiled ? (h % per_key) * KH + h / per_key : h;
  for (uint32_t r = warp; r < rows; r += kGdnThreads / 32) {
    float val[4], total = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      val[g] = bf16_bits_to_float(__ldcg(p.scratch + (size_t(h) * kGdnRows + r) * kD + 32 * g + lane));
      total += warp_sum(val[g] * val[g]);
    }
    const float inv = rsqrtf(total / float(kD) + 1e-6f);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t d = 32 * g + lane;
      const float normalized = round_bf16((val[g] * inv) * a.norm_w[d]);
      const float z = bf16_bits_to_float(qkvz[size_t(r) * a.qkvz_stride + C + h * kD + d]);
      static_cast<uint16_t *>(a.hidden)[size_t(r) * a.hidden_stride + out_head * kD + d] =
          float_to_bf16_bits((normalized * z) / (1.0f + exp2f(-1.44269504089f * z)));
    }
  }
  if (tid == 0) p.counters[h] = 0;
}


// Whether the call needs the tree kernel: tree rows, or a pending path that is not known here to be the tape's first rows.
static bool needs_tree_kernel(const SbGdnArgs &a) {
  return a.tree || a.pending_path_dev || (a.pending_path & (a.pending_path + 1u)) != 0;
}

// ---- the same step with no allocation anywhere ----
// Some hosts of this library may not allocate device memory at all once they are running: a runtime that
// reserved the whole GPU for its own arena up front, a plugin loaded into such a process, or code that runs
// where cudaMalloc would fail or stall (inside a memory-pool callback, under a fixed memory budget). The
// regular entry point uses two pieces of scratch that sb_init allocated: the recurrent rows awaiting their
// gate and one arrival counter per value head. This variant keeps both in a fixed array that is part of the
// library image, so every GPU that loads the library holds kStaticScratchBytes of it until the process exits.
constexpr uint32_t kStaticMaxValueHeads = 64;  // the 27B shape has 48
constexpr size_t kStaticRowsBytes = size_t(kStaticMaxValueHeads) * kGdnRows * kD * sizeof(uint16_t);  // 256 KiB
constexpr size_t kStaticScratchBytes = kStaticRowsBytes + kStaticMaxValueHeads * sizeof(uint32_t);
static __device__ __align__(256) uint8_t g_gdn_static_scratch[kStaticScratchBytes];

// In host code the array's name only stands for the symbol; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch_address(uint8_t **out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<uint8_t *> address[kMaxDevices];  // (two threads racing here store the same value)
  int device = -1;
  SB_CUDA(cudaGetDevice(&device));
  SB_REQUIRE(device >= 0 && device < kMaxDevices, "sb_gdn_verify_static: device index %d outside 0..%d", device, kMaxDevices - 1);
  if (!address[device].load(std::memory_order_acquire)) {
    void *p = nullptr;
    SB_CUDA(cudaGetSymbolAddress(&p, g_gdn_static_scratch));
    SB_REQUIRE(p != nullptr, "sb_gdn_verify_static: the scratch symbol has no address on device %d", device);
    address[device].store(static_cast<uint8_t *>(p), std::memory_order_release);
  }
  *out = address[device].load(std::memory_order_acquire);
  return SB_OK;
}

}  // namespace sb

using namespace sb;

namespace sb {
// The argument checks both entry points share; `who` names the caller in the message.
static int gdn_validate(const SbGdnArgs *a, const char *who) {
  SB_REQUIRE(a, "%s: null arguments", who);
  SB_REQUIRE(a->qkvz && ((a->b && a->a) || a->gate_weight) && a->conv_w && a->a_scale && a->dt_bias && a->norm_w && a->conv_state_in &&
                 a->conv_state_out && a->state_in && a->state_out && a->hidden,
             "%s: null pointer", who);
  SB_REQUIRE(a->rows <= kGdnRows && a->pending_rows <= kGdnRows, "%s: rows %u or pending rows %u above %d", who, a->rows, a->pending_rows, kGdnRows);
  SB_REQUIRE(a->key_heads >= 1 && a->value_heads >= 1 && a->value_heads % a->key_heads == 0 && a->value_heads <= 256,
             "%s: %u value heads over %u key heads", who, a->value_heads, a->key_heads);
  const uint32_t C = (2 * a->key_heads + a->value_heads) * kD;
  SB_REQUIRE(a->qkvz_stride >= C + a->value_heads * kD && (a->gate_weight || a->ab_stride >= a->value_heads) && a->hidden_stride >= a->value_heads * kD,
             "%s: a stride is below its row", who);
  SB_REQUIRE(a->rows == 0 || (a->step.inputs && a->step.k && a->step.v && a->step.beta && a->step.decay), "%s: null tape of this step", who);
  SB_REQUIRE((a->pending_rows == 0 && !a->pending_rows_dev && !a->pending_path && !a->pending_path_dev) ||
                 (a->pending.inputs && a->pending.k && a->pending.v && a->pending.beta && a->pending.decay),
             "%s: null pending tape", who);
  SB_REQUIRE(a->pending_path < (1u << kGdnRows), "%s: pending path 0x%x names rows above %d", who, a->pending_path, kGdnRows);
  SB_REQUIRE(a->state_in != a->state_out && a->conv_state_in != a->conv_state_out, "%s: the committed cell is a second cell", who);
  SB_REQUIRE(!a->gate_weight || (a->gate_input && a->gate_k && a->gate_k % 8 == 0 && a->gate_input_stride >= a->gate_k && a->gate_input_stride % 8 == 0 &&
                                 (reinterpret_cast<uintptr_t>(a->gate_weight) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->gate_input) & 15) == 0),
             "%s: fused gate projection needs a 16-byte aligned input and weight, k a multiple of 8 and stride >= k", who);
  SB_REQUIRE((a->flags & ~uint32_t(SB_GDN_STATE_SETTLED)) == 0, "%s: unknown flags 0x%x", who, a->flags);
  SB_REQUIRE(a->lanes <= 64 && size_t(std::max(1u, a->lanes)) * a->value_heads <= kGdnScratchHeads, "%s: %u lanes of %u value heads exceed the scratch", who,
             a->lanes, a->value_heads);
  return SB_OK;
}
}  // namespace sb

extern "C" int sb_gdn_verify(void *stream, const SbGdnArgs *a) {
  SB_NEED_DEVICE();
  const int valid = gdn_validate(a, "sb_gdn_verify");
  if (valid != SB_OK) return valid;
  Context &c = ctx();
  GdnParams p{*a, c.gdn_scratch, c.gdn_counters};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kGdnSplit, a->value_heads, std::max(1u, a->lanes));
  cfg.blockDim = dim3(kGdnThreads);
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = c.pdl ? 1 : 0;
  if (a->lanes > 1)
    SB_CUDA(needs_tree_kernel(*a) ? cudaLaunchKernelEx(&cfg, gdn_kernel<true, 4>, p) : cudaLaunchKernelEx(&cfg, gdn_kernel<false, 4>, p));
  else
    SB_CUDA(needs_tree_kernel(*a) ? cudaLaunchKernelEx(&cfg, gdn_kernel<true>, p) : cudaLaunchKernelEx(&cfg, gdn_kernel<false>, p));
  return SB_OK;
}

extern "C" int sb_gdn_verify_static(void *stream, const SbGdnArgs *a) {
  SB_REQUIRE(a, "sb_gdn_verify_static: null arguments");
  SB_REQUIRE(a->value_heads <= kStaticMaxValueHeads,
             "sb_gdn_verify_static: %u value heads exceed the %u the built-in scratch holds; use sb_gdn_verify", a->value_heads,
             kStaticMaxValueHeads);
  SB_REQUIRE(a->lanes <= 1, "sb_gdn_verify_static: one lane a call (the built-in scratch holds one lane's rows)");
  const int valid = gdn_validate(a, "sb_gdn_verify_static");
  if (valid != SB_OK) return valid;
  uint8_t *scratch = nullptr;
  const int st = static_scratch_address(&scratch);
  if (st != SB_OK) return st;
  // The array keeps whatever the last call left. The arrival counters must start at zero; the rows are
  // written in full before they are read.
  uint32_t *counters = reinterpret_cast<uint32_t *>(scratch + kStaticRowsBytes);
  SB_CUDA(cudaMemsetAsync(counters, 0, kStaticMaxValueHeads * sizeof(uint32_t), as_stream(stream)));
  GdnParams p{*a, reinterpret_cast<uint16_t *>(scratch), counters};
  if (needs_tree_kernel(*a)) gdn_kernel<true><<<dim3(kGdnSplit, a->value_heads), dim3(kGdnThreads), 0, as_stream(stream)>>>(p);
  else gdn_kernel<false><<<dim3(kGdnSplit, a->value_heads), dim3(kGdnThreads), 0, as_stream(stream)>>>(p);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
