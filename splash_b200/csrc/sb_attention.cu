// INT8 paged-KV attention over the verify block, one kernel: split-KV page loop with online softmax,
// then the split merge, bf16 rounding and the output gate in the CTA that arrives last for its KV head.
//
// Takes the place of the reference's split + reduce kernels (attention_q8_split*, attention_reduce*,
// runtime/metal/kernels/shared/paged_attention.metal:13-78; tile math
// runtime/metal/kernels/common/paged_attention_tile.h:178-285,339-471; merge :498-535; gate
// runtime/metal/kernels/common/attention_gate.h:19-45).
//
//   grid      (splits, kv_heads); 256 threads. The step's rows x the KV head's query heads form the
//             fused rows (row-major: fused = row * group + head_in_group, at most 128); warp w owns fused
//             rows 16w..16w+15 as one m16 MMA tile, warps without rows only help loading.
//   split     a contiguous run of 32-token chunks of the visible tokens [0, committed + rows)
//   chunk     K and V rows (token-major int8, 32 x D bytes contiguous inside a page) and their scales arrive
//             through a ring of bulk async copies three chunks ahead, are converted exactly to fp16 ((q ^ 0x80 | 0x6400) - 1152) and
//             stored in shared memory; S = Q K^T and O += P V run on mma.sync m16n8k16 (fp16 operands,
//             fp32 accumulators) with ldmatrix fragments; score = S * k_scale[token] / sqrt(D); row r sees
//             tokens <= committed + r (and, with a tree, only its ancestors inside the block);
//             P = fp16(p * v_scale[token]) (the reference rounds this product to bf16)
//   merge     fp32 partial O and (max, sum) per split go to the context's workspace; once every split of a KV
//             head has arrived (cooperative launch, bounded wait) the head's CTAs share its fused rows, each
//             adding a row's splits in split order with weights exp(max_s - max), dividing, rounding to bf16
//             and multiplying by sigmoid(gate)
#include <algorithm>

#include "sb_attention_internal.cuh"

namespace sb {

constexpr int kAttnThreads = 256;
constexpr int kChunk = 32;       // tokens per step of the page loop
constexpr int kRing = 3;         // raw chunks in flight per CTA
constexpr int kConv = 3;         // converted chunks (fp16) buffered for the multiplying warps

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1) attention_kernel(const AttnParams p_in) {
  const AttnParams p = attn_lane_view(p_in);  // (one lane: p_in itself)
  constexpr int PITCH = D + 8;             // halves per shared row: 16-byte rows shifted by 4 banks
  constexpr int KSTEPS = D / 16, NT_O = D / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half *q_s = reinterpret_cast<__half *>(smem_raw);              // [128][PITCH]
  __half *kv_s = q_s + kMaxFused * PITCH;                           // [kConv][K: 32 x PITCH, V: 32 x PITCH]
  float *sc_s = reinterpret_cast<float *>(kv_s + kConv * 2 * kChunk * PITCH);  // [kConv][ks: 32, vs: 32]; ks = scale / sqrt(D) * log2(e)
  uint8_t *ring = reinterpret_cast<uint8_t *>(sc_s + kConv * 2 * kChunk);      // [kRing][2 * 32 * D + 256] raw chunks
  uint64_t *full = reinterpret_cast<uint64_t *>(ring + kRing * (2 * kChunk * D + 256));
  uint64_t *conv_full = full + kRing, *conv_empty = conv_full + kConv;
  __shared__ uint32_t s_last;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kRing; ++i) mbar_init(&full[i], 1);
    for (int i = 0; i < kConv; ++i) {
      mbar_init(&conv_full[i], 1);
      mbar_init(&conv_empty[i], (p.fused + 15) / 16);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();

  const uint32_t split = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t F = p.fused, G = p.group;
  const uint32_t committed = p.committed_dev ? min(*p.committed_dev, p.committed) : p.committed;
  const uint32_t visible = committed + p.rows;
  const uint32_t chunks = (visible + kChunk - 1) / kChunk;
  const uint32_t c_begin = split * p.chunks_per_split, c_end = min(chunks, c_begin + p.chunks_per_split);

  // Queries of this KV head -> fp16 in shared memory (bounded by the q norm, so the conversion is exact
  // down to fp16's subnormals); rows past the fused rows are zero.
  for (uint32_t i = tid; i < kMaxFused * (D / 8); i += kAttnThreads) {
    const uint32_t f = i / (D / 8), c8 = i % (D / 8);
    uint4 o = make_uint4(0, 0, 0, 0);
    if (f < F) {
      const uint32_t row = f / G, hg = f % G;
      const uint4 raw = *reinterpret_cast<const uint4 *>(p.queries + (size_t(row) * p.q_heads + kvh * G + hg) * D + c8 * 8);
      const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 hv = __floats2half2_rn(bf16_bits_to_float(u[j] & 0xffffu), bf16_bits_to_float(u[j] >> 16));
        h[j] = *reinterpret_cast<const uint32_t *>(&hv);
      }
      o = make_uint4(h[0], h[1], h[2], h[3]);
    }
    *reinterpret_cast<uint4 *>(q_s + f * PITCH + c8 * 8) = o;
  }

  __syncthreads();  // the queries are staged before any warp multiplies
  const bool computes = warp * 16 < F;
  float o_acc[NT_O][4];
#pragma unroll
  for (int n = 0; n < NT_O; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o_acc[n][c] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  // Rows of this thread's two fused rows and what they may see.
  uint32_t limit[2], anc[2];
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const uint32_t f = warp * 16 + g + 8 * hrow, row = min(f / G, p.rows - 1);
    limit[hrow] = committed + row + 1;  // tokens below this are visible to a chain row
    anc[hrow] = 0xffffffffu;
    if (p.tree) {
      limit[hrow] = visible;
      anc[hrow] = p.tree[row].x;
    }
  }

  // Chunk ring: thread 0 keeps kRing - 1 chunks in flight with bulk async copies (a chunk's 32 tokens are
  // contiguous inside a page: D x 32 bytes of keys, of values, and their 32 scales each), completing on
  // one mbarrier per slot. Every thread then converts its share of the landed chunk to fp16.
  const uint32_t sbytes = p.cache.scale_f16 ? 2u : 4u;
  const uint32_t slot_bytes = 2 * kChunk * D + 256;
  auto issue = [&](uint32_t chunk) {
    const uint32_t s = (chunk - c_begin) % kRing, tk = chunk * kChunk;
    const uint32_t page = p.page_table[tk / p.cache.page_tokens], pt = tk % p.cache.page_tokens;
    const size_t slot = (size_t(page) * p.cache.kv_heads + kvh) * p.cache.page_tokens + pt;
    uint8_t *dst = ring + s * slot_bytes;
    fence_proxy_async();
    mbar_arrive_expect_tx(&full[s], 2 * kChunk * D + 2 * kChunk * sbytes);
    bulk_g2s(dst, static_cast<const int8_t *>(p.cache.k) + slot * D, kChunk * D, &full[s]);
    bulk_g2s(dst + kChunk * D, static_cast<const int8_t *>(p.cache.v) + slot * D, kChunk * D, &full[s]);
    bulk_g2s(dst + 2 * kChunk * D, static_cast<const uint8_t *>(p.cache.k_scale) + slot * sbytes, kChunk * sbytes, &full[s]);
    bulk_g2s(dst + 2 * kChunk * D + 128, static_cast<const uint8_t *>(p.cache.v_scale) + slot * sbytes, kChunk * sbytes, &full[s]);
  };
  const float score_scale = (D == 256 ? 0.0625f : 0.08838834764831845f) * 1.44269504089f;  // 1/sqrt(D) * log2(e)
  auto stage_into = [&](uint32_t chunk, __half *k_s, float *ks_s, uint32_t wtid, uint32_t wthreads) {
    const uint8_t *src = ring + ((chunk - c_begin) % kRing) * slot_bytes;
    __half *v_s = k_s + kChunk * PITCH;
    float *vs_s = ks_s + kChunk;
    for (uint32_t idx = wtid; idx < kChunk * (D / 16); idx += wthreads) {
      const uint32_t tok = idx / (D / 16), part = idx % (D / 16);
      uint4 lo, hi;
      int8x16_to_half(*reinterpret_cast<const uint4 *>(src + tok * D + part * 16), lo, hi);
      *reinterpret_cast<uint4 *>(k_s + tok * PITCH + part * 16) = lo;
      *reinterpret_cast<uint4 *>(k_s + tok * PITCH + part * 16 + 8) = hi;
      int8x16_to_half(*reinterpret_cast<const uint4 *>(src + kChunk * D + tok * D + part * 16), lo, hi);
      *reinterpret_cast<uint4 *>(v_s + tok * PITCH + part * 16) = lo;
      *reinterpret_cast<uint4 *>(v_s + tok * PITCH + part * 16 + 8) = hi;
    }
    if (wtid < kChunk) {
      // Tokens past the visible ones share the page but hold nothing: their scales read as zero.
      const bool live = chunk * kChunk + wtid < visible;
      float ksc, vsc;
      if (p.cache.scale_f16) {
        ksc = __half2float(reinterpret_cast<const __half *>(src + 2 * kChunk * D)[wtid]);
        vsc = __half2float(reinterpret_cast<const __half *>(src + 2 * kChunk * D + 128)[wtid]);
      } else {
        ksc = reinterpret_cast<const float *>(src + 2 * kChunk * D)[wtid];
        vsc = reinterpret_cast<const float *>(src + 2 * kChunk * D + 128)[wtid];
      }
      ks_s[wtid] = live ? ksc * score_scale : 0.0f;
      vs_s[wtid] = live ? vsc : 0.0f;
    }
  };

  auto compute_chunk = [&](uint32_t chunk, const __half *k_s, const __half *v_s, const float *ks_s, const float *vs_s) {
    const uint32_t tok0 = chunk * kChunk;
    // S = Q K^T for 16 fused rows x 32 tokens.
    float s_acc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s_acc[n][c] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, k_s + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_f16(s_acc[2 * np], a[0], a[1], a[2], a[3], b[0], b[1]);
        mma_f16(s_acc[2 * np + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
      }
    }
    // Scores (in log2 units), masks, online softmax. Accumulator c: row g + 8 (c >> 1), token 8 n + 2 t + (c & 1).
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t tl = 8 * n + 2 * t + (c & 1), tk = tok0 + tl;
        const int hrow = c >> 1;
        bool seen = tk < limit[hrow];
        if (p.tree && tk >= committed) seen = seen && ((anc[hrow] >> min(tk - committed, 31u)) & 1u);
        const float sc = seen ? s_acc[n][c] * ks_s[tl] : -INFINITY;
        s_acc[n][c] = sc;
        mx[hrow] = fmaxf(mx[hrow], sc);
      }
    float corr[2];
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 1));
      mx[hrow] = fmaxf(mx[hrow], __shfl_xor_sync(0xffffffffu, mx[hrow], 2));
      const float m_new = fmaxf(m_run[hrow], mx[hrow]);
      corr[hrow] = (m_new == -INFINITY || m_new == m_run[hrow]) ? 1.0f : exp2f(m_run[hrow] - m_new);
      m_run[hrow] = m_new;
    }
    float psum[2] = {0.0f, 0.0f};
    uint32_t pa[2][4];  // P as A fragments for the two 16-token k-steps
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      float pv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int hrow = c >> 1;
        const float pr = s_acc[n][c] == -INFINITY ? 0.0f : exp2f(s_acc[n][c] - m_run[hrow]);
        psum[hrow] += pr;
        pv[c] = pr * vs_s[8 * n + 2 * t + (c & 1)];
      }
      const __half2 r0 = __floats2half2_rn(pv[0], pv[1]), r1 = __floats2half2_rn(pv[2], pv[3]);
      // n-tile n covers tokens 8n..8n+7: k-step n / 2, low (n even) or high (n odd) half of its 16 tokens.
      pa[n >> 1][(n & 1) * 2 + 0] = *reinterpret_cast<const uint32_t *>(&r0);  // row g
      pa[n >> 1][(n & 1) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&r1);  // row g + 8
    }
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      psum[hrow] += __shfl_xor_sync(0xffffffffu, psum[hrow], 1);
      psum[hrow] += __shfl_xor_sync(0xffffffffu, psum[hrow], 2);
      l_run[hrow] = l_run[hrow] * corr[hrow] + psum[hrow];
    }
    if (corr[0] != 1.0f || corr[1] != 1.0f) {
#pragma unroll
      for (int n = 0; n < NT_O; ++n) {
        o_acc[n][0] *= corr[0], o_acc[n][1] *= corr[0];
        o_acc[n][2] *= corr[1], o_acc[n][3] *= corr[1];
      }
    }
    // O += P V.
#pragma unroll
    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_s + (kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + np * 16 + ((lane >> 4) & 1) * 8);
        mma_f16(o_acc[2 * np], pa[kt][0], pa[kt][1], pa[kt][2], pa[kt][3], b[0], b[1]);
        mma_f16(o_acc[2 * np + 1], pa[kt][0], pa[kt][1], pa[kt][2], pa[kt][3], b[2], b[3]);
      }
  };

  const uint32_t ncw = (F + 15) / 16;  // warps with an m-tile
  if (ncw + 2 <= kAttnThreads / 32) {
    // ---- specialised: warps 0..ncw-1 multiply, the last two warps convert chunks into a ring of three
    // converted buffers and keep the raw ring full. Buffers are handed over through mbarriers, so the
    // multiplying warps drift apart and keep the tensor pipe busy while others are in their softmax. ----
    const uint32_t nchunks = c_end > c_begin ? c_end - c_begin : 0;
    if (warp >= kAttnThreads / 32 - 2) {
      const uint32_t ctid = tid - (kAttnThreads - 64);
      if (ctid == 0)
        for (uint32_t c = c_begin; c < c_end && c < c_begin + kRing; ++c) issue(c);
      for (uint32_t i = 0; i < nchunks; ++i) {
        const uint32_t chunk = c_begin + i, buf = i % kConv;
        bool ok = mbar_wait(&full[i % kRing], (i / kRing) & 1);
        if (ok && i >= kConv) ok = mbar_wait(&conv_empty[buf], (i / kConv - 1) & 1);
        if (!ok) {
          if (ctid == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
          break;
        }
        stage_into(chunk, kv_s + buf * 2 * kChunk * PITCH, sc_s + buf * 2 * kChunk, ctid, 64);
        named_bar_sync(1, 64);  // both converter warps have written the buffer and read the raw slot
        if (ctid == 0) {
          mbar_arrive(&conv_full[buf]);
          if (chunk + kRing < c_end) issue(chunk + kRing);
        }
      }
    } else if (computes) {
      for (uint32_t i = 0; i < nchunks; ++i) {
        const uint32_t buf = i % kConv;
        if (!mbar_wait(&conv_full[buf], (i / kConv) & 1)) {
          if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
          break;
        }
        const __half *k_s = kv_s + buf * 2 * kChunk * PITCH;
        compute_chunk(c_begin + i, k_s, k_s + kChunk * PITCH, sc_s + buf * 2 * kChunk, sc_s + buf * 2 * kChunk + kChunk);
        __syncwarp();
        if (lane == 0) mbar_arrive(&conv_empty[buf]);
      }
    }
  } else {
    // ---- every warp has an m-tile: all warps convert chunk i + 1, then multiply chunk i; one barrier a chunk ----
    if (tid == 0)
      for (uint32_t c = c_begin; c < c_end && c < c_begin + kRing - 1; ++c) issue(c);
    bool alive = true;
    auto convert = [&](uint32_t chunk) {  // waits for the raw chunk, then converts this thread's share
      if (!mbar_wait(&full[(chunk - c_begin) % kRing], ((chunk - c_begin) / kRing) & 1)) {
        if (tid == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
        alive = false;
        return;
      }
      const uint32_t buf = (chunk - c_begin) & 1;
      stage_into(chunk, kv_s + buf * 2 * kChunk * PITCH, sc_s + buf * 2 * kChunk, tid, kAttnThreads);
    };
    if (c_begin < c_end) convert(c_begin);
    for (uint32_t chunk = c_begin; chunk < c_end && alive; ++chunk) {
      __syncthreads();  // chunk is converted; the buffer chunk + 1 goes to and the raw slot refilled below are free
      if (tid == 0 && chunk + kRing - 1 < c_end) issue(chunk + kRing - 1);
      if (chunk + 1 < c_end) convert(chunk + 1);
      const uint32_t buf = (chunk - c_begin) & 1;
      const __half *k_s = kv_s + buf * 2 * kChunk * PITCH;
      if (computes) compute_chunk(chunk, k_s, k_s + kChunk * PITCH, sc_s + buf * 2 * kChunk, sc_s + buf * 2 * kChunk + kChunk);
    }
  }

  // Partials of this split.
  if (computes) {
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const uint32_t f = warp * 16 + g + 8 * hrow;
      if (f < F) {
        float *po = p.partials + ((size_t(kvh) * p.splits + split) * kMaxFused + f) * D;
#pragma unroll
        for (int n = 0; n < NT_O; ++n)
          *reinterpret_cast<float2 *>(po + 8 * n + 2 * t) = make_float2(o_acc[n][2 * hrow], o_acc[n][2 * hrow + 1]);
        if (t == 0) {
          float *ps = p.stats + ((size_t(kvh) * p.splits + split) * kMaxFused + f) * 2;
          ps[0] = m_run[hrow];
          ps[1] = l_run[hrow];
        }
      }
    }
  }
  attention_merge<D>(p, split, kvh, &s_last);
}

}  // namespace sb

using namespace sb;

extern "C" int sb_set_attention_kernel(int kind) {
  SB_REQUIRE(kind == SB_ATTENTION_TCGEN05 || kind == SB_ATTENTION_WARP_MMA, "sb_set_attention_kernel: unknown kernel %d", kind);
  ctx().attention_kernel = kind;
  return SB_OK;
}

extern "C" int sb_attn_verify(void *stream, const SbAttnArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->queries && a->page_table && a->out, "sb_attn_verify: null pointer");
  const SbKvLayer &c = a->cache;
  SB_REQUIRE(c.k && c.v && c.k_scale && c.v_scale, "sb_attn_verify: null cache pointer");
  SB_REQUIRE(c.head_dim == 128 || c.head_dim == 256, "sb_attn_verify: head_dim %u is not 128 or 256", c.head_dim);
  SB_REQUIRE(c.kv_heads >= 1 && c.page_tokens >= 32 && (c.page_tokens & (c.page_tokens - 1)) == 0,
             "sb_attn_verify: page_tokens %u is not a power of two >= 32", c.page_tokens);
  SB_REQUIRE(a->rows >= 1 && a->rows <= 32 && a->q_heads % c.kv_heads == 0, "sb_attn_verify: rows %u outside 1..32 or q_heads not a multiple of kv_heads", a->rows);
  const uint32_t group = a->q_heads / c.kv_heads, fused = a->rows * group;
  SB_REQUIRE(fused <= kMaxFused, "sb_attn_verify: rows x group = %u exceeds %d fused rows", fused, kMaxFused);
  SB_REQUIRE(!a->gated || a->qkv, "sb_attn_verify: a gated layer needs the packed rows");
  SB_REQUIRE(a->out_stride >= a->q_heads * c.head_dim, "sb_attn_verify: out_stride below the row");
  Context &cx = ctx();
  const uint32_t lanes = std::max(1u, a->lanes);
  SB_REQUIRE(lanes == 1 || (a->rows <= 16 && a->committed_dev && lanes <= 64), "sb_attn_verify: %u lanes need rows <= 16 and the lanes' positions on the device", lanes);
  if (cx.attention_kernel == SB_ATTENTION_TCGEN05) {
    AttnParams p{};
    p.queries = static_cast<const uint16_t *>(a->queries);
    p.qkv = static_cast<const uint16_t *>(a->qkv);
    p.page_table = a->page_table;
    p.tree = static_cast<const uint2 *>(a->tree);
    p.out = static_cast<uint16_t *>(a->out);
    p.cache = c;
    p.partials = cx.attn_workspace;
    p.counters = cx.attn_counters;
    p.status = cx.status_dev;
    p.committed_dev = a->committed_dev;
    p.rows = a->rows, p.q_heads = a->q_heads, p.group = group, p.gated = a->gated, p.qkv_stride = a->qkv_stride;
    p.out_stride = a->out_stride, p.committed = a->committed, p.fused = fused, p.page_table_stride = a->page_table_stride;
    return launch_attention_tc(as_stream(stream), p, a->committed + a->rows, lanes);
  }
  const uint32_t D = c.head_dim, visible = a->committed + a->rows, chunks = (visible + kChunk - 1) / kChunk;
  // Splits: about one CTA per SM over all KV heads, at least 4 chunks each.
  uint32_t splits = std::max(1u, uint32_t(cx.sm_count) / (c.kv_heads * lanes));  // the whole grid is resident at once
  splits = std::min(splits, std::max(1u, chunks / 4));
  const uint32_t cps = (chunks + splits - 1) / splits;
  splits = (chunks + cps - 1) / cps;
  SB_REQUIRE(size_t(lanes) * c.kv_heads * splits <= size_t(cx.sm_count), "sb_attn_verify: %u lanes x %u KV heads exceed the %d SMs one launch fills", lanes,
             c.kv_heads, cx.sm_count);
  const size_t need = size_t(lanes) * c.kv_heads * splits * kMaxFused * (D + 2) * sizeof(float);
  SB_REQUIRE(need <= cx.attn_workspace_bytes && c.kv_heads <= 64, "sb_attn_verify: workspace too small (%zu bytes needed)", need);
  AttnParams p{};
  p.queries = static_cast<const uint16_t *>(a->queries);
  p.qkv = static_cast<const uint16_t *>(a->qkv);
  p.page_table = a->page_table;
  p.tree = static_cast<const uint2 *>(a->tree);
  p.out = static_cast<uint16_t *>(a->out);
  p.cache = c;
  p.partials = cx.attn_workspace;
  p.stats = cx.attn_workspace + size_t(lanes) * c.kv_heads * splits * kMaxFused * D;
  p.page_table_stride = a->page_table_stride;
  p.counters = cx.attn_counters;
  p.status = cx.status_dev;
  p.committed_dev = a->committed_dev;
  p.rows = a->rows, p.q_heads = a->q_heads, p.group = group, p.gated = a->gated, p.qkv_stride = a->qkv_stride;
  p.out_stride = a->out_stride, p.committed = a->committed, p.splits = splits, p.chunks_per_split = cps, p.fused = fused;
  const size_t smem = size_t(kMaxFused + kConv * 2 * kChunk) * (D + 8) * 2 + kConv * 2 * kChunk * sizeof(float) +
                      size_t(kRing) * (2 * kChunk * D + 256) + (kRing + 2 * kConv) * sizeof(uint64_t);
  void (*kernel)(const AttnParams) = D == 256 ? attention_kernel<256> : attention_kernel<128>;
  static bool attr_set[64][2] = {};  // a function attribute is per device
  const int dev = ctx().device >= 0 && ctx().device < 64 ? ctx().device : 0;
  if (!attr_set[dev][D == 256]) {
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    attr_set[dev][D == 256] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, c.kv_heads, lanes);
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = as_stream(stream);
  // Cooperative: every CTA is resident before any runs, which the shared merge's wait relies on.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return SB_OK;
}
