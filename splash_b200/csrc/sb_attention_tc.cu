// INT8 paged-KV attention over the verify block on the tcgen05 tensor cores. Same contract, partials and
// merge as sb_attention.cu (reference: runtime/metal/kernels/common/paged_attention_tile.h:178-285,339-471,
// merge :498-535, gate runtime/metal/kernels/common/attention_gate.h:19-45); the page loop is re-cut for
// Blackwell:
//
//   rows      the step's rows x the KV head's query heads are the <= 128 fused rows = the 128 lanes of tensor
//             memory; a softmax thread owns one fused row, so row maxima and sums need no shuffles
//   Q         fp16 in tensor memory (D / 2 packed columns), written once; the A operand of S = Q K^T
//   chunk     64 tokens. One thread keeps a ring of raw chunks (int8 K, V and their scales) full with bulk
//             async copies; 4 converter warps turn a chunk into fp16 (exact) in the two shared-memory
//             layouts the MMAs read: K as K-major 8 x 16-byte core matrices per 16 dimensions, V with the
//             dimensions contiguous (MN-major) per 8 tokens
//   mma       one thread: S[128 x 64] = Q K^T (D / 16 tcgen05.mma, A from tensor memory) for chunk c + 1
//             while the softmax warps work on chunk c, then O[128 x D] += P V (4 MMAs, P from tensor memory,
//             where the softmax threads wrote it over their own S columns)
//   softmax   score = S * k_scale[token] / sqrt(D) in log2 units, masks as in the warp kernel, p = exp2(s - m),
//             P = fp16(p * v_scale[token]). The reference maximum m only moves when a chunk's maximum exceeds it
//             by more than 8 (p <= 256 stays far inside fp16); then the thread rescales its row of O in tensor
//             memory once the previous chunk's P V has completed. The merge weighs splits by their own m.
//
// Tensor-memory columns: Q [0, D/2), S / P double buffer 2 x 64, O D columns: 512 at D = 256.
#include <algorithm>

#include "sb_attention_internal.cuh"
#include "sb_tcgen05.cuh"

namespace sb {

constexpr int kAtChunk = 64;                 // tokens per chunk
constexpr int kAtRaw = 3;                    // raw chunks in flight
constexpr int kAtConvWarps = 4;               // converter warps
constexpr int kAtConvThreads = 32 * kAtConvWarps;
constexpr int kAtMmaWarp = 4 + kAtConvWarps;
constexpr int kAtThreads = 32 * (kAtMmaWarp + 1);  // 4 softmax warps, the converter warps, 1 MMA warp
constexpr float kAtLazy = 8.0f;              // the reference maximum moves when exceeded by more than 2^8

template <int D>
struct AtLayout {
  static constexpr uint32_t kConvBytes = kAtChunk * D * 2;                       // one tensor of one chunk in fp16
  static constexpr uint32_t kRawBytes = 2 * kAtChunk * D + 2 * kAtChunk * 4;     // K, V codes and room for fp32 scales
  static constexpr uint32_t kK = 0, kV = 2 * kConvBytes, kRaw = 4 * kConvBytes;  // offsets: K[2], V[2], raw ring
  static constexpr uint32_t kScales = kRaw + kAtRaw * kRawBytes;                 // [2][ks 64, vs 64] floats
  static constexpr uint32_t kBars = kScales + 2 * 2 * kAtChunk * 4;
  static constexpr uint32_t kBytes = kBars + 128;
  static constexpr uint32_t kQCols = D / 2, kSCol0 = D / 2, kOCol0 = D / 2 + 2 * kAtChunk;
};

__device__ __forceinline__ float ex2_approx(float x) {  // 2^x, one MUFU; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool at_wait(uint64_t *bar, uint32_t parity) {  // same outcome in every lane of the warp
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity);
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1) attention_tc_kernel(const AttnParams p_in) {
  const AttnParams p = attn_lane_view(p_in);  // (one lane: p_in itself)
  using L = AtLayout<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *raw_full = reinterpret_cast<uint64_t *>(smem + L::kBars);  // [kAtRaw]
  uint64_t *kv_full = raw_full + kAtRaw;                               // [2] converters -> MMA
  uint64_t *kv_empty = kv_full + 2;                                    // [2] MMA (commit) -> converters
  uint64_t *s_full = kv_empty + 2;                                     // [2] MMA (commit) -> softmax
  uint64_t *p_full = s_full + 2;                                       // [2] softmax -> MMA
  uint64_t *o_done = p_full + 2;                                       // phase c: P V of chunk c has completed
  uint64_t *q_ready = o_done + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(q_ready + 1);
  uint32_t *s_last = tmem_slot + 1;
  float *scales = reinterpret_cast<float *>(smem + L::kScales);

  const uint32_t split = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t F = p.fused, G = p.group;
  if (tid == 0) {
    for (int i = 0; i < kAtRaw; ++i) mbar_init(&raw_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    mbar_init(o_done, 1);
    mbar_init(q_ready, 4);
    fence_mbar_init();
  }
  if (warp == kAtMmaWarp) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  const uint32_t committed = p.committed_dev ? min(*p.committed_dev, p.committed) : p.committed;
  const uint32_t visible = committed + p.rows;
  const uint32_t chunks = (visible + kAtChunk - 1) / kAtChunk;
  const uint32_t c_begin = split * p.chunks_per_split, c_end = min(chunks, c_begin + p.chunks_per_split);
  const uint32_t n = c_end > c_begin ? c_end - c_begin : 0;
  const float score_scale = (D == 256 ? 0.0625f : 0.08838834764831845f) * 1.44269504089f;  // 1/sqrt(D) * log2(e)
  const uint32_t sbytes = p.cache.scale_f16 ? 2u : 4u;

  if (warp < 4) {
    // ---- softmax warps: thread = fused row f = TMEM lane ----
    const uint32_t f = tid, tl = tmem_addr(tmem, 32 * warp, 0);
    {  // Q row -> fp16 -> tensor memory (zeros past the fused rows)
      const uint32_t row = f / G, hg = f % G;
      const uint4 *src = reinterpret_cast<const uint4 *>(p.queries + (size_t(min(row, p.rows - 1)) * p.q_heads + kvh * G + hg) * D);
#pragma unroll
      for (int b = 0; b < D / 32; ++b) {  // 32 dimensions = 16 packed columns per store
        uint32_t r[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 raw = make_uint4(0, 0, 0, 0);
          if (f < F) raw = src[4 * b + q];
          const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 hv = __floats2half2_rn(bf16_bits_to_float(u[j] & 0xffffu), bf16_bits_to_float(u[j] >> 16));
            r[4 * q + j] = *reinterpret_cast<const uint32_t *>(&hv);
          }
        }
        tmem_st16(tl + 16 * b, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }
    const uint32_t row = min(f / G, p.rows - 1);
    uint32_t limit = committed + row + 1, anc = 0xffffffffu;  // chain: tokens below `limit` are visible
    if (p.tree) limit = visible, anc = p.tree[row].x;
    float m_ref = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (uint32_t i = 0; i < n && ok; ++i) {
      const uint32_t b = i & 1, tok0 = (c_begin + i) * kAtChunk;
      if (!at_wait(&s_full[b], (i >> 1) & 1)) {
        if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float s[kAtChunk];
      tmem_ld32_wait(tl + L::kSCol0 + b * kAtChunk, s);
      tmem_ld32_wait(tl + L::kSCol0 + b * kAtChunk + 32, s + 32);
      const float4 *ks4 = reinterpret_cast<const float4 *>(scales + b * 2 * kAtChunk), *vs4 = ks4 + kAtChunk / 4;
      // Scores in log2 units; four running maxima keep the chain short. A chunk of pure history (the common
      // case) needs no mask; otherwise the row's visibility is a 64-bit mask built once: tokens below `limit`,
      // and inside the block only the row's ancestors.
      const bool plain = tok0 + kAtChunk <= committed;
      unsigned long long vis = ~0ull;
      if (!plain) {
        const long long rel = (long long)limit - (long long)tok0;
        vis = rel >= 64 ? ~0ull : rel <= 0 ? 0ull : ((1ull << rel) - 1ull);
        if (p.tree) {
          const long long j0 = (long long)committed - (long long)tok0;  // the block's first token, relative to the chunk
          const unsigned long long a64 = anc;
          vis &= j0 >= 64 ? ~0ull : j0 >= 0 ? ((a64 << j0) | ((1ull << j0) - 1ull)) : (a64 >> (-j0));
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kAtChunk; j += 4) {
        const float4 k4 = ks4[j / 4];
        s[j] *= k4.x, s[j + 1] *= k4.y, s[j + 2] *= k4.z, s[j + 3] *= k4.w;
        if (!plain) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (!((vis >> (j + q)) & 1ull)) s[j + q] = -INFINITY;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], s[j + q]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Move the reference maximum only when it is exceeded by more than kAtLazy; rescale O then.
      float factor = 1.0f;
      if (mx > m_ref + kAtLazy || (m_ref == -INFINITY && mx > -INFINITY)) {
        factor = m_ref == -INFINITY ? 0.0f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      // O holds chunks 0..i-1 and this chunk's P goes where S(i-1)'s neighbour buffer was: wait for the previous
      // chunk's P V in every chunk, so the barrier's phases are followed one by one (its waits tell only
      // consecutive phases apart) and a rescale below never meets an MMA in flight on O.
      if (i > 0) {
        if (!at_wait(o_done, (i - 1) & 1)) {
          if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            float o[32];
            tmem_ld32_wait(tl + L::kOCol0 + c0, o);
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(o[j] * factor);
            tmem_st16(tl + L::kOCol0 + c0, r);
            tmem_st16(tl + L::kOCol0 + c0 + 16, r + 16);
          }
        }
      }
      l_run *= factor;
      // p = 2^(s - m): masked scores are -inf and give 0; while the row has seen nothing m stands in as 0.
      const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
      float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t pk[kAtChunk / 2];
#pragma unroll
      for (int j = 0; j < kAtChunk; j += 4) {
        const float4 v4 = vs4[j / 4];
        const float p0 = ex2_approx(s[j] - m_use), p1 = ex2_approx(s[j + 1] - m_use);
        const float p2 = ex2_approx(s[j + 2] - m_use), p3 = ex2_approx(s[j + 3] - m_use);
        ps4[0] += p0, ps4[1] += p1, ps4[2] += p2, ps4[3] += p3;
        const __half2 h0 = __floats2half2_rn(p0 * v4.x, p1 * v4.y), h1 = __floats2half2_rn(p2 * v4.z, p3 * v4.w);
        pk[j / 2] = *reinterpret_cast<const uint32_t *>(&h0);
        pk[j / 2 + 1] = *reinterpret_cast<const uint32_t *>(&h1);
      }
      l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      tmem_st16(tl + L::kSCol0 + b * kAtChunk, pk);
      tmem_st16(tl + L::kSCol0 + b * kAtChunk + 16, pk + 16);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }
    // Partials of this split: the row of O once the last P V has completed.
    if (ok && n > 0 && !at_wait(o_done, (n - 1) & 1)) {
      if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
      ok = false;
    }
    tc_fence_after_sync();
    {
      float *po = p.partials + ((size_t(kvh) * p.splits + split) * kMaxFused + min(f, uint32_t(kMaxFused - 1))) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float o[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = 0.0f;
        if (ok && n > 0) tmem_ld32_wait(tl + L::kOCol0 + c0, o);  // the whole warp, also lanes past the fused rows
        if (f < F)
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(po + c0 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
      }
      if (f < F) {
        float *ps = p.stats + ((size_t(kvh) * p.splits + split) * kMaxFused + f) * 2;
        ps[0] = m_ref;
        ps[1] = l_run;
      }
    }
  } else if (warp < kAtMmaWarp) {
    // ---- converter warps; their first thread also keeps the raw ring full ----
    const uint32_t ctid = tid - 128;
    uint8_t *ring = smem + L::kRaw;
    auto issue = [&](uint32_t i) {  // chunk c_begin + i -> raw slot i % kAtRaw, as runs of 32 tokens inside a page
      const uint32_t slot = i % kAtRaw;
      uint8_t *dst = ring + slot * L::kRawBytes;
      fence_proxy_async();
      uint32_t bytes = 0;
      for (uint32_t h = 0; h < kAtChunk / 32; ++h)
        if ((c_begin + i) * kAtChunk + 32 * h < visible) bytes += 2 * 32 * D + 2 * 32 * sbytes;
      mbar_arrive_expect_tx(&raw_full[slot], bytes);
      for (uint32_t h = 0; h < kAtChunk / 32; ++h) {
        const uint32_t tk = (c_begin + i) * kAtChunk + 32 * h;
        if (tk >= visible) continue;  // nothing stored there yet: the converters' stale codes are masked
        const uint32_t page = p.page_table[tk / p.cache.page_tokens], pt = tk % p.cache.page_tokens;
        const size_t at = (size_t(page) * p.cache.kv_heads + kvh) * p.cache.page_tokens + pt;
        bulk_g2s(dst + 32 * h * D, static_cast<const int8_t *>(p.cache.k) + at * D, 32 * D, &raw_full[slot]);
        bulk_g2s(dst + kAtChunk * D + 32 * h * D, static_cast<const int8_t *>(p.cache.v) + at * D, 32 * D, &raw_full[slot]);
        bulk_g2s(dst + 2 * kAtChunk * D + 32 * h * sbytes, static_cast<const uint8_t *>(p.cache.k_scale) + at * sbytes, 32 * sbytes, &raw_full[slot]);
        bulk_g2s(dst + 2 * kAtChunk * D + kAtChunk * 4 + 32 * h * sbytes, static_cast<const uint8_t *>(p.cache.v_scale) + at * sbytes, 32 * sbytes, &raw_full[slot]);
      }
    };
    if (ctid == 0)
      for (uint32_t i = 0; i < n && i < kAtRaw; ++i) issue(i);
    for (uint32_t i = 0; i < n; ++i) {
      const uint32_t b = i & 1, slot = i % kAtRaw;
      bool ok = at_wait(&raw_full[slot], (i / kAtRaw) & 1);
      if (ok && i >= 2) ok = at_wait(&kv_empty[b], ((i >> 1) - 1) & 1);
      if (!ok) {
        if (ctid == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
        break;
      }
      const uint8_t *src = ring + slot * L::kRawBytes;
      uint8_t *kb = smem + L::kK + b * L::kConvBytes, *vb = smem + L::kV + b * L::kConvBytes;
      // Unit (token, part = 16 dimensions). A thread keeps one token (consecutive threads, consecutive tokens)
      // and walks the parts diagonally, so neither the 16-byte reads nor the 16-byte writes of a quarter warp
      // share a bank.
      static_assert(kAtConvThreads % kAtChunk == 0, "a converter thread keeps its token");
      const uint32_t tok = ctid % kAtChunk, pb0 = ctid / kAtChunk;
      const uint8_t *ksrc = src + tok * D, *vsrc = ksrc + kAtChunk * D;
      uint8_t *kdst = kb + (tok >> 3) * 256 + (tok & 7) * 16, *vdst = vb + (tok >> 3) * (D / 8 * 128) + (tok & 7) * 16;
#pragma unroll
      for (uint32_t it = 0; it < (D / 16) / (kAtConvThreads / kAtChunk); ++it) {
        const uint32_t pb = pb0 + it * (kAtConvThreads / kAtChunk);
        const uint32_t part = (pb & ~7u) | ((pb + tok) & 7u);
        uint4 lo, hi;
        int8x16_to_half(*reinterpret_cast<const uint4 *>(ksrc + part * 16), lo, hi);
        *reinterpret_cast<uint4 *>(kdst + part * (kAtChunk * 32)) = lo;
        *reinterpret_cast<uint4 *>(kdst + part * (kAtChunk * 32) + 128) = hi;
        int8x16_to_half(*reinterpret_cast<const uint4 *>(vsrc + part * 16), lo, hi);
        *reinterpret_cast<uint4 *>(vdst + part * 256) = lo;
        *reinterpret_cast<uint4 *>(vdst + part * 256 + 128) = hi;
      }
      if (ctid < kAtChunk) {
        // Tokens past the visible ones share the page but hold nothing: their scales read as zero.
        const bool live = (c_begin + i) * kAtChunk + ctid < visible;
        float ksc, vsc;
        if (p.cache.scale_f16) {
          ksc = __half2float(reinterpret_cast<const __half *>(src + 2 * kAtChunk * D)[ctid]);
          vsc = __half2float(reinterpret_cast<const __half *>(src + 2 * kAtChunk * D + kAtChunk * 4)[ctid]);
        } else {
          ksc = reinterpret_cast<const float *>(src + 2 * kAtChunk * D)[ctid];
          vsc = reinterpret_cast<const float *>(src + 2 * kAtChunk * D + kAtChunk * 4)[ctid];
        }
        scales[b * 2 * kAtChunk + ctid] = live ? ksc * score_scale : 0.0f;
        scales[b * 2 * kAtChunk + kAtChunk + ctid] = live ? vsc : 0.0f;
      }
      fence_proxy_async();      // the MMAs read these shared-memory writes through the async proxy
      named_bar_sync(1, kAtConvThreads);  // every converter warp has written the chunk and read the raw slot
      if (ctid == 0) {
        mbar_arrive(&kv_full[b]);
        if (i + kAtRaw < n) issue(i + kAtRaw);
      }
    }
  } else if (lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc_qk = umma_idesc_f16(128, kAtChunk), idesc_pv = umma_idesc_f16(128, D, true);
    bool ok = mbar_wait(q_ready, 0);
    tc_fence_after_sync();
    auto issue_qk = [&](uint32_t i) {  // S[i & 1] = Q K(i)^T
      const uint32_t b = i & 1;
      const uint64_t kd = umma_smem_desc(smem_u32(smem + L::kK + b * L::kConvBytes), 128, 256);
#pragma unroll
      for (uint32_t s = 0; s < D / 16; ++s)
        umma_f16_ts(tmem + L::kSCol0 + b * kAtChunk, tmem + 8 * s, kd + s * (kAtChunk * 32 / 16), idesc_qk, s > 0);
      umma_commit(&s_full[b]);
    };
    if (ok && n > 0) {
      ok = mbar_wait(&kv_full[0], 0);
      tc_fence_after_sync();
      if (ok) issue_qk(0);
    }
    for (uint32_t i = 0; i < n && ok; ++i) {
      const uint32_t b = i & 1;
      if (i + 1 < n) {
        ok = mbar_wait(&kv_full[b ^ 1], ((i + 1) >> 1) & 1);
        if (!ok) break;
        tc_fence_after_sync();
        issue_qk(i + 1);  // its S buffer held P(i - 1), consumed by the P V issued before this point
      }
      ok = mbar_wait(&p_full[b], (i >> 1) & 1);
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t vd = umma_smem_desc(smem_u32(smem + L::kV + b * L::kConvBytes), D / 8 * 128, 128);
#pragma unroll
      for (uint32_t s = 0; s < kAtChunk / 16; ++s)
        umma_f16_ts(tmem + L::kOCol0, tmem + L::kSCol0 + b * kAtChunk + 8 * s, vd + s * (2 * (D / 8 * 128) / 16), idesc_pv, i > 0 || s > 0);
      umma_commit(&kv_empty[b]);
      umma_commit(o_done);
    }
    if (!ok) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
  }

  // Everyone meets here, also after a wait that gave up, so tensor memory is always returned.
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kAtMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
  attention_merge<D>(p, split, kvh, s_last);
}

int launch_attention_tc(cudaStream_t stream, AttnParams &p, uint32_t visible, uint32_t lanes) {
  Context &cx = ctx();
  const uint32_t D = p.cache.head_dim, chunks = (visible + kAtChunk - 1) / kAtChunk;
  // Splits: about one CTA per SM over all KV heads and lanes (the whole grid is resident at once), at least 2 chunks each.
  uint32_t splits = std::max(1u, uint32_t(cx.sm_count) / (p.cache.kv_heads * lanes));
  splits = std::min(splits, std::max(1u, chunks / 2));
  const uint32_t cps = (chunks + splits - 1) / splits;
  splits = (chunks + cps - 1) / cps;
  SB_REQUIRE(size_t(lanes) * p.cache.kv_heads * splits <= size_t(cx.sm_count), "sb_attn_verify: %u lanes x %u KV heads exceed the %d SMs one launch fills",
             lanes, p.cache.kv_heads, cx.sm_count);
  const size_t need = size_t(lanes) * p.cache.kv_heads * splits * kMaxFused * (D + 2) * sizeof(float);
  SB_REQUIRE(need <= cx.attn_workspace_bytes && p.cache.kv_heads <= 64, "sb_attn_verify: workspace too small (%zu bytes needed)", need);
  p.stats = cx.attn_workspace + size_t(lanes) * p.cache.kv_heads * splits * kMaxFused * D;
  p.splits = splits, p.chunks_per_split = cps;
  const size_t smem = D == 256 ? AtLayout<256>::kBytes : AtLayout<128>::kBytes;
  void (*kernel)(const AttnParams) = D == 256 ? attention_tc_kernel<256> : attention_tc_kernel<128>;
  static bool attr_set[64][2] = {};  // a function attribute is per device
  const int dev = ctx().device >= 0 && ctx().device < 64 ? ctx().device : 0;
  if (!attr_set[dev][D == 256]) {
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    attr_set[dev][D == 256] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, p.cache.kv_heads, lanes);
  cfg.blockDim = dim3(kAtThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // Cooperative: every CTA is resident before any runs, which the shared merge's wait relies on.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return SB_OK;
}

}  // namespace sb
