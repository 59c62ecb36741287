// Glue operators of the verify step: RMSNorm, embedding gather, RoPE tables, the fp32 projection of
// plain fp32 rows, q/k norm + RoPE + INT8 KV store, path commit, selection and acceptance.
// Each replaces the reference operator named at its entry point in include/splash_b200.h.
#include <algorithm>

#include "sb_dequant.cuh"
#include "sb_dot.cuh"

namespace sb {

// Sum over a block of `warps` warps in a fixed order: a butterfly within each warp, then the warps'
// values in index order. Every thread receives the total.
template <int WARPS>
__device__ __forceinline__ float block_sum(float v, float *scratch) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.0f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) r += scratch[w];
  return r;
}

// ---- RMSNorm: one block of 256 threads per row ----
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t *x, uint32_t width, uint32_t x_stride, const float *w,
                                                      uint16_t *out, uint32_t out_stride) {
  __shared__ float scratch[8];
  pdl_launch_dependents();
  pdl_wait();
  const uint16_t *row = x + size_t(blockIdx.x) * x_stride;
  float ss = 0.0f;
  for (uint32_t c = threadIdx.x; c < width; c += 256) {
    const float v = bf16_bits_to_float(row[c]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum<8>(ss, scratch);
  const float inv = rsqrtf(ss / float(width) + 1e-6f);
  for (uint32_t c = threadIdx.x; c < width; c += 256)
    out[size_t(blockIdx.x) * out_stride + c] = float_to_bf16_bits((bf16_bits_to_float(row[c]) * inv) * w[c]);
}

// ---- embedding gather ----
__global__ void __launch_bounds__(256) embed_kernel(uint32_t format, const uint8_t *table, uint64_t row_bytes, uint32_t vocab,
                                                    uint32_t width, const uint32_t *tokens, uint16_t *out,
                                                    uint32_t out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t r = blockIdx.y;
  uint32_t t = tokens[r];
  if (t >= vocab) t = 0;
  const uint8_t *row = table + size_t(t) * row_bytes;
  const uint32_t c = blockIdx.x * 256 + threadIdx.x;
  if (c >= width) return;
  float v;
  if (format == SB_FMT_BF16) v = bf16_bits_to_float(reinterpret_cast<const uint16_t *>(row)[c]);
  else if (format == SB_FMT_F16) v = __half2float(reinterpret_cast<const __half *>(row)[c]);
  else if (format == SB_FMT_F32) v = reinterpret_cast<const float *>(row)[c];
  else v = weight_value(format, row, c);
  out[size_t(r) * out_stride + c] = float_to_bf16_bits(v);
}

// ---- the same projection for many rows (the rows of several lanes): warp-level MMA with the fp32 weights split into three
// bf16 terms (hi + mid + lo carry the 24 bits of an fp32 significand), so every product with a bf16 input is exact and the
// sums run in fp32. ----
__device__ __forceinline__ void split3_bf16(float a, float b, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
  const uint32_t ah = float_to_bf16_bits(a), bh = float_to_bf16_bits(b);
  const float ar = a - bf16_bits_to_float(ah), br = b - bf16_bits_to_float(bh);
  const uint32_t am = float_to_bf16_bits(ar), bm = float_to_bf16_bits(br);
  const uint32_t al = float_to_bf16_bits(ar - bf16_bits_to_float(am)), bl = float_to_bf16_bits(br - bf16_bits_to_float(bm));
  hi = ah | (bh << 16), mid = am | (bm << 16), lo = al | (bl << 16);
}
// grid (n / 16, rows / 16): a CTA takes 16 rows x 16 columns; its 8 warps divide k (every warp's loads are in flight at once)
// and their sums are added in warp order.
__global__ void __launch_bounds__(256) linear_f32_rows_kernel(const float *w, const uint16_t *x, uint32_t rows, uint32_t n, uint32_t k,
                                                              uint32_t x_stride, void *out, uint32_t out_stride, uint32_t out_f32) {
  __shared__ float part_s[8][16][17];
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t r0 = blockIdx.y * 16, c0 = blockIdx.x * 16;
  const uint32_t kw = k / 8, kb = warp * kw;  // this warp's inputs
  const uint16_t *xa = x + size_t(min(r0 + g, rows - 1)) * x_stride + kb + 2 * t, *xb = x + size_t(min(r0 + g + 8, rows - 1)) * x_stride + kb + 2 * t;
  const float *w0 = w + size_t(c0 + g) * k + kb + 2 * t, *w1 = w + size_t(c0 + 8 + g) * k + kb + 2 * t;
  // The tensor cores' fp32 additions truncate; sums of 64 inputs are kept short and added up with rounded additions.
  float acc[2][4] = {}, total[2][4] = {};
#pragma unroll 4
  for (uint32_t k0 = 0; k0 < kw; k0 += 16) {
    if (k0 && k0 % 64 == 0) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[j][i] += acc[j][i], acc[j][i] = 0.0f;
    }
    const uint32_t a0 = *reinterpret_cast<const uint32_t *>(xa + k0), a1 = *reinterpret_cast<const uint32_t *>(xb + k0);
    const uint32_t a2 = *reinterpret_cast<const uint32_t *>(xa + k0 + 8), a3 = *reinterpret_cast<const uint32_t *>(xb + k0 + 8);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float *wr = j ? w1 : w0;
      const float2 p = *reinterpret_cast<const float2 *>(wr + k0), q = *reinterpret_cast<const float2 *>(wr + k0 + 8);
      uint32_t h0, m0, l0, h1, m1, l1;
      split3_bf16(p.x, p.y, h0, m0, l0);
      split3_bf16(q.x, q.y, h1, m1, l1);
      mma_bf16(acc[j], a0, a1, a2, a3, l0, l1);  // the small terms first
      mma_bf16(acc[j], a0, a1, a2, a3, m0, m1);
      mma_bf16(acc[j], a0, a1, a2, a3, h0, h1);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) part_s[warp][g + (i >> 1) * 8][8 * j + 2 * t + (i & 1)] = total[j][i] + acc[j][i];
  __syncthreads();
  const uint32_t r = threadIdx.x >> 4, c = threadIdx.x & 15;
  float v = 0.0f;
#pragma unroll
  for (int wv = 0; wv < 8; ++wv) v += part_s[wv][r][c];
  if (r0 + r >= rows) return;
  if (out_f32) static_cast<float *>(out)[size_t(r0 + r) * out_stride + c0 + c] = v;
  else static_cast<uint16_t *>(out)[size_t(r0 + r) * out_stride + c0 + c] = float_to_bf16_bits(v);
}

// ---- RoPE tables ----
__global__ void rope_kernel(const uint32_t *positions, uint32_t rows, const float *inv_freq, uint32_t pairs, float scale,
                            float *cosine, float *sine) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * pairs) return;
  const float angle = float(positions[i / pairs]) * inv_freq[i % pairs];
  float s, c;
  sincosf(angle, &s, &c);
  cosine[i] = c * scale;
  sine[i] = s * scale;
}

// ---- fp32 projection of plain fp32 rows: grid (columns, 2); a warp per (column, row), lanes over k ----
constexpr int kF32Rows = 1024;  // (a warp per (column, row): the rows of several lanes too)
__global__ void __launch_bounds__(256) linear_f32_kernel(const float *w, const uint16_t *x, uint32_t rows, uint32_t n,
                                                         uint32_t k, uint32_t x_stride, void *out, uint32_t out_stride,
                                                         uint32_t out_f32, const float *norm_w) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t col = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t r = blockIdx.y * 8 + warp;
  if (r >= rows) return;
  const float *wr = w + size_t(col) * k;
  const uint16_t *xr = x + size_t(r) * x_stride;
  float inv = 1.0f;
  if (norm_w) {
    float ss = 0.0f;
#pragma unroll 4
    for (uint32_t c = 8 * lane; c < k; c += 256) {
      const uint4 v = *reinterpret_cast<const uint4 *>(xr + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = bf16_bits_to_float(u[j] & 0xffffu), b = bf16_bits_to_float(u[j] >> 16);
        ss = fmaf(a, a, fmaf(b, b, ss));
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = rsqrtf(ss / float(k) + 1e-6f);
  }
  // Lane-strided groups of 8 inputs, then a butterfly over the lanes.
  float acc = 0.0f;
  if (!norm_w) {
    acc = warp_dot_f32_bf16(wr, xr, k, lane);
  } else {
#pragma unroll 5
  for (uint32_t c = 8 * lane; c < k; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4 *>(xr + c);
    const float4 w0 = *reinterpret_cast<const float4 *>(wr + c), w1 = *reinterpret_cast<const float4 *>(wr + c + 4);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float xv = bf16_bits_to_float((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xffffu));
      if (norm_w) xv = round_bf16((xv * inv) * norm_w[c + j]);
      acc = fmaf(xv, wv[j], acc);
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  }
  if (lane == 0) {
    if (out_f32) static_cast<float *>(out)[size_t(r) * out_stride + col] = acc;
    else static_cast<uint16_t *>(out)[size_t(r) * out_stride + col] = float_to_bf16_bits(acc);
  }
}

constexpr uint32_t kLaneRows = 16;  // row slots of a lane in a step of several lanes (the verify block's most rows)

// ---- q/k norm + RoPE + INT8 KV store: grid (q_heads + kv_heads, rows, lanes), head_dim threads ----
struct StoreParams {
  const uint16_t *qkv;
  const float *q_norm, *k_norm, *cos_tab, *sin_tab;
  const uint32_t *page_table;
  uint16_t *queries;
  SbKvLayer cache;
  const uint32_t *committed_dev;
  uint32_t rows, q_heads, gated, pairs, qkv_stride, committed;
  uint32_t page_table_stride;  // lanes (blockIdx.z): page-table entries between consecutive lanes' tables
};

__device__ __forceinline__ int8_t kv_code(float v, float m) {
  if (m == 0.0f) return 0;
  const float q = rintf(__fdiv_rn(__fmul_rn(v, 127.0f), m));
  return int8_t(fminf(fmaxf(q, -127.0f), 127.0f));
}

template <int D>
__global__ void __launch_bounds__(D) attn_store_kernel(const StoreParams p) {
  constexpr int W = D / 32;
  __shared__ float part[W], part2[W];
  __shared__ float normed[D];
  pdl_launch_dependents();
  pdl_wait();
  // Lanes (blockIdx.z): a lane's rows are rows 16 z .. of the row-indexed buffers; its position and page table are its own.
  const uint32_t lane_index = blockIdx.z;
  const uint32_t head = blockIdx.x, row = kLaneRows * lane_index + blockIdx.y, d = threadIdx.x, lane = d & 31, warp = d >> 5;
  const bool query = head < p.q_heads;
  const uint32_t kvh = query ? 0 : head - p.q_heads, qs = p.gated ? 2 * D : D;
  const uint16_t *prow = p.qkv + size_t(row) * p.qkv_stride;
  const uint16_t *src = query ? prow + head * qs : prow + p.q_heads * qs + kvh * D;
  const float x = bf16_bits_to_float(src[d]);
  // Sum of squares: 32 dimensions per warp added in dimension order, then the warps in order.
  float sq = x * x;
  // in-order sum within the warp: lane 0 accumulates lanes 0..31 (a sequential chain, as the oracle's)
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, sq, i));
  if (lane == 0) part[warp] = acc;
  __syncthreads();
  float ss = 0.0f;
#pragma unroll
  for (int w = 0; w < W; ++w) ss = __fadd_rn(ss, part[w]);
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(D)), 1e-6f)));
  const float wn = (query ? p.q_norm : p.k_norm)[d];
  normed[d] = round_bf16(__fmul_rn(__fmul_rn(x, inv), wn));
  __syncthreads();
  float r = normed[d];
  if (d < 2 * p.pairs) {
    const uint32_t pr = d % p.pairs;
    const float a = normed[pr], b = normed[pr + p.pairs];
    const float c = p.cos_tab[size_t(row) * p.pairs + pr], s = p.sin_tab[size_t(row) * p.pairs + pr];
    r = d < p.pairs ? round_bf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)))
                    : round_bf16(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s)));
  }
  if (query) {
    p.queries[(size_t(row) * p.q_heads + head) * D + d] = float_to_bf16_bits(r);
    return;
  }
  const float v = bf16_bits_to_float(prow[p.q_heads * qs + p.cache.kv_heads * D + kvh * D + d]);
  float km = fabsf(r), vm = fabsf(v);
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    km = fmaxf(km, __shfl_xor_sync(0xffffffffu, km, o));
    vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, o));
  }
  __syncthreads();
  if (lane == 0) part[warp] = km, part2[warp] = vm;
  __syncthreads();
  km = 0.0f, vm = 0.0f;
#pragma unroll
  for (int w = 0; w < W; ++w) km = fmaxf(km, part[w]), vm = fmaxf(vm, part2[w]);
  const uint32_t tok = (p.committed_dev ? p.committed_dev[lane_index] : p.committed) + blockIdx.y;
  const uint32_t page = p.page_table[size_t(lane_index) * p.page_table_stride + tok / p.cache.page_tokens], pt = tok % p.cache.page_tokens;
  const size_t slot = (size_t(page) * p.cache.kv_heads + kvh) * p.cache.page_tokens + pt;
  static_cast<int8_t *>(p.cache.k)[slot * D + d] = kv_code(r, km);
  static_cast<int8_t *>(p.cache.v)[slot * D + d] = kv_code(v, vm);
  if (d == 0) {
    const float ks = km == 0.0f ? 0.0f : __fdiv_rn(km, 127.0f), vs = vm == 0.0f ? 0.0f : __fdiv_rn(vm, 127.0f);
    if (p.cache.scale_f16) {
      static_cast<__half *>(p.cache.k_scale)[slot] = __float2half_rn(ks);
      static_cast<__half *>(p.cache.v_scale)[slot] = __float2half_rn(vs);
    } else {
      static_cast<float *>(p.cache.k_scale)[slot] = ks;
      static_cast<float *>(p.cache.v_scale)[slot] = vs;
    }
  }
}

// ---- path commit: grid (kv_heads), head_dim threads; rows move in depth order ----
// Several lanes: grid (kv_heads, lanes); lane l's position at committed_dev[l], its page table page_table_stride entries
// further on, its path mask mask_stride words further on.
__global__ void kv_path_commit_kernel(SbKvLayer c, const uint32_t *page_table, uint32_t committed, const uint32_t *committed_dev,
                                      const uint32_t *path_mask, uint32_t page_table_stride, uint32_t mask_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t lane_of_step = blockIdx.y;
  page_table += size_t(lane_of_step) * page_table_stride, path_mask += size_t(lane_of_step) * mask_stride;
  if (committed_dev) committed = committed_dev[lane_of_step];
  const uint32_t mask = *path_mask, h = blockIdx.x, d = threadIdx.x, D = c.head_dim;
  uint32_t depth = 0;
  for (uint32_t row = 0; row < 32; ++row) {
    if (!((mask >> row) & 1u)) continue;
    if (row != depth) {
      const uint32_t s = committed + row, t = committed + depth;
      const size_t ss = (size_t(page_table[s / c.page_tokens]) * c.kv_heads + h) * c.page_tokens + s % c.page_tokens;
      const size_t ts = (size_t(page_table[t / c.page_tokens]) * c.kv_heads + h) * c.page_tokens + t % c.page_tokens;
      static_cast<int8_t *>(c.k)[ts * D + d] = static_cast<int8_t *>(c.k)[ss * D + d];
      static_cast<int8_t *>(c.v)[ts * D + d] = static_cast<int8_t *>(c.v)[ss * D + d];
      if (d == 0) {
        if (c.scale_f16) {
          static_cast<uint16_t *>(c.k_scale)[ts] = static_cast<uint16_t *>(c.k_scale)[ss];
          static_cast<uint16_t *>(c.v_scale)[ts] = static_cast<uint16_t *>(c.v_scale)[ss];
        } else {
          static_cast<float *>(c.k_scale)[ts] = static_cast<float *>(c.k_scale)[ss];
          static_cast<float *>(c.v_scale)[ts] = static_cast<float *>(c.v_scale)[ss];
        }
      }
    }
    ++depth;
    __syncthreads();  // a later row may read the slot this one wrote
  }
}

// ---- selection: one block of 1024 threads per row ----
constexpr uint32_t kSentinel = 0xFFFFFFFFu;
constexpr uint32_t kShard = 256;
constexpr uint32_t kDrawCandidates = 16, kNoDraw = 0xff;  // a row's draft candidates; "no child drawn" (runtime/metal/abi/ExecutionGeometry.h:63)
constexpr int kSampleThreads = 1024;

__device__ __forceinline__ bool selectable(float x) { return !(isnan(x) || x == -INFINITY); }

// ---- the end of a row's distribution: min-p, then top-k, then the top-p nucleus (sampling.metal:604-668) ----
// A token stays iff its key (order-preserving bits of its logit, -0 as +0) is above cut.key, or equal to it with an id
// up to cut.id. Every search walks the 32 key bits from the top with one block-wide measurement per bit; masses are the
// shard sums (256 ids in id order) added in shard order by one thread, as everywhere in this kernel.
constexpr uint32_t kMaxFilterShards = 1024;  // vocabulary up to 262144 with filters
struct RowCut {
  uint32_t key, id;
};
__device__ __forceinline__ uint32_t logit_key(float x) {
  if (x == 0.0f) x = 0.0f;
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_logit(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ bool cut_keeps(const RowCut c, float x, uint32_t v) {
  if (!selectable(x)) return false;
  const uint32_t k = logit_key(x);
  return k > c.key || (k == c.key && v <= c.id);
}
struct FilterScratch {
  float shard_mass[kMaxFilterShards];
  uint32_t counts[kSampleThreads];
  uint32_t warp_counts[32];
  uint32_t count, pick_thread, pick_rank, id;
  float mass;
};
// Count and mass of the kept tokens whose key is at least `key` (above it when `strict`); every thread gets both.
__device__ void block_measure(const float *l, uint32_t vocab, RowCut cut, uint32_t key, bool strict, bool want_mass, float mx, float inv_t,
                              FilterScratch &fs, uint32_t &count, float &mass) {
  const uint32_t tid = threadIdx.x, shards = (vocab + kShard - 1) / kShard;
  uint32_t mine = 0;
  for (uint32_t s = tid; s < shards; s += kSampleThreads) {
    float sum = 0.0f;
    const uint32_t end = min(vocab, (s + 1) * kShard);
    for (uint32_t v = s * kShard; v < end; ++v) {
      const float x = l[v];
      if (!cut_keeps(cut, x, v)) continue;
      const uint32_t k = logit_key(x);
      if (strict ? k > key : k >= key) {
        ++mine;
        if (want_mass) sum = __fadd_rn(sum, expf(__fmul_rn(__fsub_rn(x, mx), inv_t)));
      }
    }
    fs.shard_mass[s] = sum;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if ((tid & 31) == 0) fs.warp_counts[tid >> 5] = mine;
  __syncthreads();
  if (tid == 0) {
    uint32_t c = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) c += fs.warp_counts[w];
    float m = 0.0f;
    if (want_mass)
      for (uint32_t s = 0; s < shards; ++s) m = __fadd_rn(m, fs.shard_mass[s]);
    fs.count = c, fs.mass = m;
  }
  __syncthreads();
  count = fs.count, mass = fs.mass;
  __syncthreads();
}
// The id of the n-th (1-based) kept token whose key equals `key`, in id order.
__device__ uint32_t block_nth_tie(const float *l, uint32_t vocab, RowCut cut, uint32_t key, uint32_t n, FilterScratch &fs) {
  const uint32_t tid = threadIdx.x, chunk = (vocab + kSampleThreads - 1) / kSampleThreads;
  const uint32_t v0 = min(vocab, tid * chunk), v1 = min(vocab, v0 + chunk);
  uint32_t mine = 0;
  for (uint32_t v = v0; v < v1; ++v) mine += cut_keeps(cut, l[v], v) && logit_key(l[v]) == key;
  fs.counts[tid] = mine;
  if (tid == 0) fs.id = kSentinel;
  __syncthreads();
  if (tid == 0) {
    uint32_t before = 0, t = 0;
    for (; t < kSampleThreads && before + fs.counts[t] < n; ++t) before += fs.counts[t];
    fs.pick_thread = t, fs.pick_rank = n - before;
  }
  __syncthreads();
  if (tid == fs.pick_thread) {
    uint32_t rank = fs.pick_rank;
    for (uint32_t v = v0; v < v1; ++v)
      if (cut_keeps(cut, l[v], v) && logit_key(l[v]) == key && --rank == 0) {
        fs.id = v;
        break;
      }
  }
  __syncthreads();
  const uint32_t id = fs.id;
  __syncthreads();
  return id;
}
__device__ RowCut distribution_end(const float *l, uint32_t vocab, float mx, float temperature, float inv_t, float min_p, uint32_t top_k,
                                   float top_p, FilterScratch &fs) {
  RowCut cut{0u, kSentinel};
  uint32_t kept_count, count;
  float kept_mass, mass;
  block_measure(l, vocab, cut, 0u, false, true, mx, inv_t, fs, kept_count, kept_mass);
  if (min_p > 0.0f) {
    const float t = fminf(__fadd_rn(mx, __fmul_rn(temperature, logf(min_p))), mx);
    block_measure(l, vocab, cut, logit_key(t), false, true, mx, inv_t, fs, count, mass);
    if (count < kept_count) cut = RowCut{logit_key(t), kSentinel}, kept_count = count, kept_mass = mass;
  }
  if (top_k > 0 && top_k < kept_count) {
    uint32_t key = 0;  // the largest key with at least top_k kept tokens at or above it
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = key | (1u << bit);
      block_measure(l, vocab, cut, cand, false, false, mx, inv_t, fs, count, mass);
      if (count >= top_k) key = cand;
    }
    block_measure(l, vocab, cut, key, true, true, mx, inv_t, fs, count, mass);
    const uint32_t need = top_k - count;
    const uint32_t id = block_nth_tie(l, vocab, cut, key, need, fs);
    cut = RowCut{key, id};
    kept_count = top_k;
    kept_mass = __fadd_rn(mass, __fmul_rn(float(need), expf(__fmul_rn(__fsub_rn(key_logit(key), mx), inv_t))));
  }
  if (top_p > 0.0f && top_p < 1.0f) {
    const float nucleus = __fmul_rn(top_p, kept_mass);
    uint32_t key = 0;  // the largest key whose kept tokens at or above it weigh more than the nucleus
    bool found = false;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = key | (1u << bit);
      block_measure(l, vocab, cut, cand, false, true, mx, inv_t, fs, count, mass);
      if (mass > nucleus) key = cand, found = true;
    }
    if (!found) {
      block_measure(l, vocab, cut, 0u, false, true, mx, inv_t, fs, count, mass);
      found = mass > nucleus;
    }
    if (found) {  // rounding may leave the nucleus unreached: then everything kept so far stays
      uint32_t above_count, at_count;
      float above_mass, at_mass;
      block_measure(l, vocab, cut, key, true, true, mx, inv_t, fs, above_count, above_mass);
      block_measure(l, vocab, cut, key, false, false, mx, inv_t, fs, at_count, at_mass);
      const uint32_t ties = at_count - above_count;
      if (ties > 0) {
        const float w = expf(__fmul_rn(__fsub_rn(key_logit(key), mx), inv_t));
        const float q = fminf(fmaxf(__fdiv_rn(__fsub_rn(nucleus, above_mass), w), 0.0f), float(ties - 1));
        const uint32_t keep = 1u + uint32_t(q);
        const uint32_t id = block_nth_tie(l, vocab, cut, key, keep, fs);
        cut = RowCut{key, id};
      }
    }
  }
  return cut;
}

// One row's selection by one block (row blockIdx.x of lane blockIdx.y).
__device__ __forceinline__ void sample_row(const SbSampleArgs &a_in) {
  __shared__ FilterScratch fs;
  __shared__ float best_v[32];
  __shared__ uint32_t best_i[32];
  __shared__ float s_max;
  __shared__ uint32_t s_top;
  // Lanes (blockIdx.y): lane z's rows are rows 16 z .. of every row-indexed buffer, its uniforms the 80 from 80 z on.
  SbSampleArgs a = a_in;
  {
    const uint32_t z = blockIdx.y, r0 = kLaneRows * z;
    a.logits += size_t(r0) * a.logit_stride, a.input_tokens += r0, a.selected += r0;
    if (a.uniforms) a.uniforms += 80 * z;
    if (a.workspace) a.workspace += size_t(r0) * (2 * ((a.vocab + kShard - 1) / kShard) + 8);
    if (a.cut_out) a.cut_out += 2 * r0;
    if (a.candidate_ids) a.candidate_ids += kDrawCandidates * r0, a.candidate_q += kDrawCandidates * r0, a.draws += 4 * r0;
    if (a.lane_policies) {  // the lane's own policy
      const SbLanePolicy q = a.lane_policies[z];
      a.temperature = q.temperature, a.min_p = q.min_p, a.top_k = q.top_k, a.top_p = q.top_p;
    }
  }
  const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float *l = a.logits + size_t(r) * a.logit_stride;
  // Greedy: value descending, id ascending.
  float bv = -INFINITY;
  uint32_t bi = kSentinel;
  for (uint32_t v = tid; v < a.vocab; v += kSampleThreads) {
    const float x = l[v];
    if (selectable(x) && (bi == kSentinel || x > bv)) bv = x, bi = v;
  }
  auto better = [](float v1, uint32_t i1, float v2, uint32_t i2) {
    if (i2 == kSentinel) return true;
    if (i1 == kSentinel) return false;
    return v1 > v2 || (v1 == v2 && i1 < i2);
  };
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (!better(bv, bi, ov, oi)) bv = ov, bi = oi;
  }
  if (lane == 0) best_v[warp] = bv, best_i[warp] = bi;
  __syncthreads();
  if (tid == 0) {
    float v = best_v[0];
    uint32_t i = best_i[0];
    for (int w = 1; w < kSampleThreads / 32; ++w)
      if (!better(v, i, best_v[w], best_i[w])) v = best_v[w], i = best_i[w];
    s_max = v, s_top = i;
  }
  __syncthreads();
  const uint32_t top = s_top;
  if (a.temperature == 0.0f || !a.uniforms || top == kSentinel) {
    if (tid == 0) a.selected[r] = top;
    return;
  }
  // Temperature weights; each shard of 256 ids summed by one thread in id order.
  const float mx = s_max, inv_t = __fdiv_rn(1.0f, a.temperature);
  const uint32_t shards = (a.vocab + kShard - 1) / kShard;
  float *shard = a.workspace + size_t(r) * (2 * shards + 8), *shard2 = shard + shards;
  const bool has_child = !a.candidate_ids && r + 1 < a.rows;  // (with the draft's candidates given, the children are the rows' draws)
  const uint32_t child = has_child ? a.input_tokens[r + 1] : kSentinel;
  RowCut cut{0u, kSentinel};
  if (a.min_p > 0.0f || (a.top_k > 0 && a.top_k < a.vocab) || (a.top_p > 0.0f && a.top_p < 1.0f))
    cut = distribution_end(l, a.vocab, mx, a.temperature, inv_t, a.min_p, a.top_k, a.top_p, fs);
  if (a.cut_out && tid == 0) a.cut_out[2 * r] = cut.key, a.cut_out[2 * r + 1] = cut.id;
  auto weight = [&](uint32_t v) {
    const float x = l[v];
    return cut_keeps(cut, x, v) ? expf(__fmul_rn(__fsub_rn(x, mx), inv_t)) : 0.0f;
  };
  for (uint32_t s = tid; s < shards; s += kSampleThreads) {
    float sum = 0.0f, sum2 = 0.0f;
    const uint32_t end = min(a.vocab, (s + 1) * kShard);
    for (uint32_t v = s * kShard; v < end; ++v) {
      const float w = weight(v);
      sum = __fadd_rn(sum, w);
      sum2 = __fadd_rn(sum2, v == child ? 0.0f : w);
    }
    shard[s] = sum;
    shard2[s] = sum2;
  }
  __syncthreads();
  if (tid != 0) return;
  float z = 0.0f;
  for (uint32_t s = 0; s < shards; ++s) z = __fadd_rn(z, shard[s]);
  if (a.candidate_ids) {
    // Recursive rejection sampling without replacement over the children the draft drew for this row
    // (runtime/metal/kernels/decode/sampling.metal:693-885): child i of the row's kDrawCandidates candidates, of
    // probability p_i under the target and q_i under the draft, is taken when u_i q_i < p_i; after a rejection the
    // target becomes its residual max(p - q, 0), renormalised, and the draft loses the rejected child, renormalised; a
    // row that takes none draws from the last residual, its candidates first, then the tokens outside them. A row
    // without drawn children draws from its whole distribution.
    const uint32_t *ids = a.candidate_ids + kDrawCandidates * r;
    const float *cq = a.candidate_q + kDrawCandidates * r;
    const uint8_t *draws = a.draws + 4 * r;
    float target = __fmul_rn(a.uniforms[r], z);
    bool excluding = false;
    if (draws[0] != kNoDraw && z > 0.0f) {
      float pc[kDrawCandidates], qc[kDrawCandidates];
      for (uint32_t i = 0; i < kDrawCandidates; ++i) {
        const uint32_t id = ids[i];
        const float w = id < a.vocab ? weight(id) : 0.0f;
        if (id < a.vocab) shard[id / kShard] = fmaxf(__fsub_rn(shard[id / kShard], w), 0.0f);  // the shards without the candidates
        pc[i] = __fdiv_rn(w, z);
        qc[i] = cq[i];
      }
      float outside_weight = 0.0f;
      for (uint32_t s = 0; s < shards; ++s) outside_weight = __fadd_rn(outside_weight, shard[s]);
      float outside = __fdiv_rn(outside_weight, z);
      for (uint32_t c = 0; c < 4; ++c) {
        const uint32_t dc = draws[c];
        if (dc >= kDrawCandidates) break;
        if (__fmul_rn(a.uniforms[16 + 4 * r + c], qc[dc]) < pc[dc]) {
          a.selected[r] = ids[dc];
          return;
        }
        float residual = outside;
        for (uint32_t i = 0; i < kDrawCandidates; ++i) residual = __fadd_rn(residual, fmaxf(__fsub_rn(pc[i], qc[i]), 0.0f));
        if (!(residual > 0.0f)) break;
        for (uint32_t i = 0; i < kDrawCandidates; ++i) pc[i] = __fdiv_rn(fmaxf(__fsub_rn(pc[i], qc[i]), 0.0f), residual);
        outside = __fdiv_rn(outside, residual);
        qc[dc] = 0.0f;
        float rest = 0.0f;
        for (uint32_t i = 0; i < kDrawCandidates; ++i) rest = __fadd_rn(rest, qc[i]);
        for (uint32_t i = 0; rest > 0.0f && i < kDrawCandidates; ++i) qc[i] = __fdiv_rn(qc[i], rest);
      }
      float inside = 0.0f;
      for (uint32_t i = 0; i < kDrawCandidates; ++i) inside = __fadd_rn(inside, pc[i]);
      const float point = __fmul_rn(a.uniforms[r], __fadd_rn(inside, outside));
      float cumulative = 0.0f;
      uint32_t last = kDrawCandidates;
      for (uint32_t i = 0; i < kDrawCandidates && !(point < cumulative); ++i)
        if (pc[i] > 0.0f) last = i, cumulative = __fadd_rn(cumulative, pc[i]);
      if (last < kDrawCandidates && (point < cumulative || !(outside > 0.0f))) {
        a.selected[r] = ids[last];
        return;
      }
      excluding = true;
      target = __fmul_rn(__fdiv_rn(__fsub_rn(point, inside), outside), outside_weight);
    }
    // By the target's own weights (outside the candidates after rejections): the shard the point falls in (the last one
    // with weight if rounding leaves it unreached), then its ids in order.
    auto excluded = [&](uint32_t v) {
      bool e = false;
      for (uint32_t i = 0; excluding && i < kDrawCandidates; ++i) e = e || ids[i] == v;
      return e;
    };
    float run = 0.0f, shard_target = 0.0f;
    uint32_t at = kSentinel;
    for (uint32_t s = 0; s < shards; ++s) {
      if (!(shard[s] > 0.0f)) continue;
      at = s, shard_target = __fsub_rn(target, run);
      run = __fadd_rn(run, shard[s]);
      if (run > target) break;
    }
    uint32_t pick = kSentinel;
    if (at != kSentinel) {
      float loc = 0.0f;
      const uint32_t end = min(a.vocab, (at + 1) * kShard);
      for (uint32_t v = at * kShard; v < end; ++v) {
        const float w = excluded(v) ? 0.0f : weight(v);
        if (w > 0.0f) pick = v;  // the last id weighed so far: where the walk ends if rounding leaves the target unreached
        loc = __fadd_rn(loc, w);
        if (w > 0.0f && loc > shard_target) break;
      }
    }
    a.selected[r] = pick;
    return;
  }
  bool drop = false;
  if (has_child && child < a.vocab) {
    const float u = a.uniforms[16 + 4 * r];
    if (__fmul_rn(u, z) < weight(child)) {
      a.selected[r] = child;
      return;
    }
    drop = true;
  }
  const float *sh = drop ? shard2 : shard;
  float zr = z;
  if (drop) {
    zr = 0.0f;
    for (uint32_t s = 0; s < shards; ++s) zr = __fadd_rn(zr, sh[s]);
  }
  const float target = __fmul_rn(a.uniforms[r], zr);
  float run = 0.0f;
  uint32_t pick = kSentinel;
  for (uint32_t s = 0; s < shards && pick == kSentinel; ++s) {
    if (__fadd_rn(run, sh[s]) > target) {
      float loc = 0.0f;
      const uint32_t end = min(a.vocab, (s + 1) * kShard);
      for (uint32_t v = s * kShard; v < end; ++v) {
        loc = __fadd_rn(loc, (drop && v == child) ? 0.0f : weight(v));
        if (__fadd_rn(run, loc) > target) {
          pick = v;
          break;
        }
      }
    }
    run = __fadd_rn(run, sh[s]);
  }
  if (pick == kSentinel)
    for (uint32_t v = a.vocab; v-- > 0;)
      if (weight(v) > 0.0f && !(drop && v == child)) {
        pick = v;
        break;
      }
  a.selected[r] = pick;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const SbSampleArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  sample_row(a);
}

// ---- acceptance: one thread ----
// Lane z: rows 16 z .., results 4 z ... The selections are read as other blocks of the same launch may have
// written them (volatile: from L2).
__device__ __forceinline__ void accept_lane(const SbAcceptArgs &a_in, uint32_t z) {
  SbAcceptArgs a = a_in;
  a.input_tokens += kLaneRows * z, a.tokens += kLaneRows * z, a.results += 4 * z;
  const uint2 *tree = static_cast<const uint2 *>(a.tree) + kLaneRows * z;  // {ancestors, parent | depth << 16}
  volatile uint32_t *tokens = a.tokens;
  uint32_t path[32];
  path[0] = 0;
  uint32_t accepted = 0;
  for (uint32_t row = 0;;) {
    const uint32_t token = tokens[row];
    uint32_t next = 0;
    for (uint32_t child = row + 1; child < a.rows && !next; ++child)
      next = ((tree[child].y & 0xffffu) == row && a.input_tokens[child] == token) ? child : 0;
    if (!next) break;
    path[++accepted] = next;
    row = next;
  }
  uint32_t kept = min(accepted + 1, a.remaining);
  for (uint32_t i = 0; i < kept; ++i) {
    const uint32_t token = tokens[path[i]];
    tokens[i] = token;
    for (uint32_t s = 0; s < a.n_stop; ++s)
      if (a.stop_tokens[s] == token) kept = i + 1;
  }
  a.results[0] = kept;
  a.results[1] = min(accepted, kept);
  a.results[2] = tree[path[kept - 1]].x;
  a.results[3] = 0;
}
__global__ void accept_kernel(const SbAcceptArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) accept_lane(a, blockIdx.x);
}

// The lane's commit after acceptance (mode as the step's end takes it: 0 hold and clear the pending rows, 1 commit the
// retained rows, 2 hold and keep the pending rows, 3 | rows << 8 commit every row).
__device__ __forceinline__ void commit_lane(const SbSelectAcceptArgs &c, uint32_t lane) {
  uint32_t *results = c.accept.results + 4 * lane;
  const uint32_t mode = c.advance & 0xffu, rows = c.advance >> 8;
  if (mode == 3) {
    results[0] = rows, results[1] = rows - 1, results[2] = (2u << (rows - 1)) - 1u;
    c.committed[lane] += rows;
    c.pending_rows[lane] = rows;
    c.pending_path[lane] = 0;
  } else if (mode == 1) {
    c.committed[lane] += results[0];
    c.pending_rows[lane] = results[0];
    c.pending_path[lane] = results[2];
  } else if (mode == 0) {
    c.pending_rows[lane] = 0;
    c.pending_path[lane] = 0;
  }
}

// Selection, acceptance and the lane's commit in one launch: a block per row selects (sample_row), and the block of a
// lane that finishes last (a ticket per lane, drawn after the block's selection is visible) walks the accepted path
// and commits the lane. The ticket word returns to zero for the next launch.
__global__ void __launch_bounds__(kSampleThreads) select_accept_kernel(const SbSelectAcceptArgs c_in) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t lane = blockIdx.y;
  // The lane's own rows (blocks of different lengths step together): the blocks of the slots past them select nothing.
  const uint32_t lane_rows = c_in.lane_rows ? min(c_in.lane_rows[lane], c_in.sample.rows) : c_in.sample.rows;
  if (blockIdx.x < lane_rows) {
    SbSampleArgs s = c_in.sample;
    s.rows = lane_rows;
    sample_row(s);
  }
  if (threadIdx.x != 0) return;
  __threadfence();
  if (atomicAdd(c_in.tickets + lane, 1u) != c_in.sample.rows - 1) return;
  __threadfence();
  c_in.tickets[lane] = 0;
  SbSelectAcceptArgs c = c_in;
  c.accept.rows = lane_rows;
  if (c.lane_remaining) c.accept.remaining = min(c.accept.remaining, max(c.lane_remaining[lane], 1u));
  if ((c.advance & 0xffu) == 3) c.advance = 3u | lane_rows << 8;
  if (!lane_rows) {  // the lane sits the step out
    uint32_t *results = c.accept.results + 4 * lane;
    results[0] = results[1] = results[2] = results[3] = 0;
    if (c.committed && (c.advance & 0xffu) != 2) c.pending_rows[lane] = 0, c.pending_path[lane] = 0;
    return;
  }
  accept_lane(c.accept, lane);
  if (c.committed) commit_lane(c, lane);
}

// The tokens a lane's rows may select (TargetRow::admits, runtime/metal/kernels/decode/sampling.metal:33-46): a row's
// constraint mask, a bit a token, and the tokens the lane never selects (the stop tokens of a lane that ignores
// end-of-sequence). A token a row does not admit gets the logit -inf in place, which every selection reads as not
// selectable; a row that admits nothing selects the sentinel. One thread per vocabulary token.
__global__ void admit_kernel(const SbAdmitArgs a_in) {
  pdl_launch_dependents();
  pdl_wait();
  SbAdmitArgs a = a_in;  // lane blockIdx.y: rows 16 z ..
  a.logits += size_t(kLaneRows) * blockIdx.y * a.logit_stride;
  if (a.masks) a.masks += size_t(kLaneRows) * blockIdx.y * a.mask_words;
  const uint32_t token = blockIdx.x * blockDim.x + threadIdx.x;
  if (token >= a.vocab) return;
  bool excluded = false;
  for (uint32_t i = 0; i < a.n_excluded; ++i) excluded |= a.excluded[i] == token;
  for (uint32_t row = 0; row < a.rows; ++row) {
    const bool masked = a.masks && !((a.masks[size_t(row) * a.mask_words + token / 32] >> (token % 32)) & 1u);
    if (excluded || masked) a.logits[size_t(row) * a.logit_stride + token] = -INFINITY;
  }
}

// One thread per vocabulary token: the token's count in every row's context, then the penalty on the rows that
// hold it (runtime/metal/kernels/decode/sampling.metal:997-1048). Products and sums are single IEEE operations in
// the reference's order, so the result equals the CPU statement bit for bit.
__global__ void penalize_kernel(const SbPenaltyArgs a_in) {
  pdl_launch_dependents();
  pdl_wait();
  SbPenaltyArgs a = a_in;  // lane blockIdx.y: rows 16 z .., its own table of the vocabulary
  a.logits += size_t(kLaneRows) * blockIdx.y * a.logit_stride, a.input_tokens += kLaneRows * blockIdx.y;
  a.words += size_t(blockIdx.y) * a.vocab, a.tree = static_cast<const uint2 *>(a.tree) + kLaneRows * blockIdx.y;
  const uint32_t token = blockIdx.x * blockDim.x + threadIdx.x;
  if (token >= a.vocab) return;
  uint32_t drafted = 0;
  for (uint32_t row = 1; row < a.rows; ++row) drafted |= uint32_t(a.input_tokens[row] == token) << row;
  const uint32_t word = a.words[token];
  if (!word && !drafted) return;
  const float inverse = fminf(__fdiv_rn(1.0f, a.repetition), 3.402823466e+38f);
  const uint2 *tree = static_cast<const uint2 *>(a.tree);
  for (uint32_t row = 0; row < a.rows; ++row) {
    const uint32_t count = (word & 0x7fffffffu) + __popc(drafted & tree[row].x & ~1u);
    if (!count && !(word & 0x80000000u)) continue;
    float *logit = a.logits + size_t(row) * a.logit_stride + token;
    float v = *logit;
    const uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7fffffffu) > 0x7f800000u || bits == 0xff800000u) continue;  // NaN and -inf stay unselectable
    v = __fmul_rn(v, v > 0.0f ? inverse : a.repetition);
    if (count) v = __fsub_rn(v, __fadd_rn(__fmul_rn(a.frequency, float(count)), a.presence));
    *logit = fminf(fmaxf(v, -3.402823466e+38f), 3.402823466e+38f);
  }
}

// ---- MoE routing: one block of 256 threads per row (runtime/metal/kernels/shared/moe.metal:22-111) ----
__global__ void __launch_bounds__(256) moe_route_kernel(const SbMoeRouteArgs a) {
  __shared__ float row_scores[256], ordered[32], partials[8];
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t routes = a.top_k + (a.shared_gate ? 1u : 0u);
  row_scores[tid] = tid < a.experts ? a.scores[size_t(row) * a.slots + tid] : -INFINITY;
  if (a.shared_gate) {
    const uint16_t *x = static_cast<const uint16_t *>(a.input) + size_t(row) * a.input_size;
    float s = 0.0f;
    for (uint32_t d = tid; d < a.input_size; d += 256) s = __fadd_rn(s, __fmul_rn(bf16_bits_to_float(x[d]), a.shared_gate[d]));
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) partials[warp] = s;
  }
  __syncthreads();
  if (a.shared_gate && tid == 0) {
    float total = 0.0f;
    for (int g = 0; g < 8; ++g) total += partials[g];
    a.selected[size_t(row) * routes + a.top_k] = a.experts;
    a.weights[size_t(row) * routes + a.top_k] = 1.0f / (1.0f + exp2f(-1.44269504089f * total));
  }
  if (warp != 0) return;
  // Lane l holds experts l, l + 32, ...; each rank takes the highest remaining score and the lowest id among ties.
  float mine[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) mine[s] = row_scores[lane + 32 * s];
  for (uint32_t rank = 0; rank < a.top_k; ++rank) {
    float best = -INFINITY;
    uint32_t slot = 0;
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (mine[s] > best) best = mine[s], slot = s;
    float row_best = best;
#pragma unroll
    for (int o = 16; o; o >>= 1) row_best = fmaxf(row_best, __shfl_xor_sync(0xffffffffu, row_best, o));
    const uint32_t candidate = best == row_best ? lane + 32 * slot : 0xFFFFFFFFu;
    uint32_t winner = candidate;
#pragma unroll
    for (int o = 16; o; o >>= 1) winner = min(winner, __shfl_xor_sync(0xffffffffu, winner, o));
    if (candidate == winner) {
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (uint32_t(s) == slot) mine[s] = -INFINITY;
    }
    if (lane == 0) {
      ordered[rank] = row_best;
      a.selected[size_t(row) * routes + rank] = winner == 0xFFFFFFFFu ? 0u : winner;
    }
  }
  __syncwarp();
  if (lane < a.top_k) {
    float den = 0.0f;
    for (uint32_t o = 0; o < a.top_k; ++o)
      den += a.sigmoid_normalized ? 1.0f / (1.0f + exp2f(-1.44269504089f * ordered[o])) : exp2f((ordered[o] - ordered[0]) * 1.44269504089f);
    a.weights[size_t(row) * routes + lane] = a.sigmoid_normalized ? (1.0f / (1.0f + exp2f(-1.44269504089f * ordered[lane]))) / (den + 1e-20f)
                                                                   : exp2f((ordered[lane] - ordered[0]) * 1.44269504089f) / den;
  }
}

template <class... Args>
static int launch(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx().pdl ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return SB_OK;
}

}  // namespace sb

using namespace sb;

extern "C" {

int sb_rmsnorm(void *stream, const void *x, uint32_t rows, uint32_t width, uint32_t x_stride, const void *weight, void *out,
               uint32_t out_stride) {
  SB_NEED_DEVICE();
  SB_REQUIRE(x && weight && out && rows && width, "sb_rmsnorm: null pointer or empty shape");
  SB_REQUIRE(x_stride >= width && out_stride >= width, "sb_rmsnorm: stride below width");
  return launch(rmsnorm_kernel, dim3(rows), dim3(256), as_stream(stream), static_cast<const uint16_t *>(x), width, x_stride,
                static_cast<const float *>(weight), static_cast<uint16_t *>(out), out_stride);
}

int sb_embed(void *stream, uint32_t format, const void *table, uint32_t vocab, uint32_t width, const uint32_t *tokens_dev,
             uint32_t rows, void *out, uint32_t out_stride) {
  SB_NEED_DEVICE();
  SB_REQUIRE(table && tokens_dev && out && rows && vocab, "sb_embed: null pointer or empty shape");
  const uint64_t rb = sb_row_bytes(format, width);
  SB_REQUIRE(rb != 0 && format != SB_FMT_NVFP4, "sb_embed: width %u is not whole blocks of format %u", width, format);
  SB_REQUIRE(out_stride >= width, "sb_embed: out_stride below width");
  return launch(embed_kernel, dim3((width + 255) / 256, rows), dim3(256), as_stream(stream), format,
                static_cast<const uint8_t *>(table), rb, vocab, width, tokens_dev, static_cast<uint16_t *>(out), out_stride);
}

int sb_rope_tables(void *stream, const uint32_t *positions_dev, uint32_t rows, const float *inv_freq_dev, uint32_t pairs,
                   float scale, float *cos_dev, float *sin_dev) {
  SB_NEED_DEVICE();
  SB_REQUIRE(positions_dev && inv_freq_dev && cos_dev && sin_dev && rows && pairs, "sb_rope_tables: null pointer or empty shape");
  return launch(rope_kernel, dim3((rows * pairs + 127) / 128), dim3(128), as_stream(stream), positions_dev, rows, inv_freq_dev,
                pairs, scale, cos_dev, sin_dev);
}

int sb_linear_f32(void *stream, const float *w_dev, const void *x, uint32_t rows, uint32_t n, uint32_t k, uint32_t x_stride,
                  void *out, uint32_t out_stride, uint32_t out_f32, const void *norm_weight) {
  SB_NEED_DEVICE();
  SB_REQUIRE(w_dev && x && out, "sb_linear_f32: null pointer");
  SB_REQUIRE(rows >= 1 && rows <= kF32Rows && n && k, "sb_linear_f32: rows = %u outside 1..%d, or empty shape", rows, kF32Rows);
  SB_REQUIRE(x_stride >= k && out_stride >= n && k % 8 == 0 && x_stride % 8 == 0, "sb_linear_f32: stride below extent, or k not a multiple of 8");
  if (rows > 16 && !norm_weight && n % 16 == 0 && k % 128 == 0)  // many rows: on the tensor cores
    return launch(linear_f32_rows_kernel, dim3(n / 16, (rows + 15) / 16), dim3(256), as_stream(stream), w_dev, static_cast<const uint16_t *>(x), rows, n, k,
                  x_stride, out, out_stride, out_f32);
  return launch(linear_f32_kernel, dim3(n, (rows + 7) / 8), dim3(256), as_stream(stream), w_dev, static_cast<const uint16_t *>(x), rows, n, k,
                x_stride, out, out_stride, out_f32, static_cast<const float *>(norm_weight));
}

static int check_cache(const SbKvLayer &c, const char *who) {
  SB_REQUIRE(c.k && c.v && c.k_scale && c.v_scale, "%s: null cache pointer", who);
  SB_REQUIRE(c.head_dim == 128 || c.head_dim == 256, "%s: head_dim %u is not 128 or 256", who, c.head_dim);
  SB_REQUIRE(c.kv_heads >= 1 && c.page_tokens >= 16 && (c.page_tokens & (c.page_tokens - 1)) == 0,
             "%s: kv_heads %u / page_tokens %u (a power of two >= 16)", who, c.kv_heads, c.page_tokens);
  return SB_OK;
}

int sb_attn_store(void *stream, const SbAttnStoreArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->qkv && a->q_norm && a->k_norm && a->page_table && a->queries, "sb_attn_store: null pointer");
  int st = check_cache(a->cache, "sb_attn_store");
  if (st != SB_OK) return st;
  const uint32_t D = a->cache.head_dim, qs = a->gated ? 2 * D : D;
  SB_REQUIRE(a->rows >= 1 && a->rows <= 32 && a->q_heads >= 1 && a->q_heads % a->cache.kv_heads == 0,
             "sb_attn_store: rows %u outside 1..32 or q_heads %u not a multiple of kv_heads", a->rows, a->q_heads);
  SB_REQUIRE(a->qkv_stride >= a->q_heads * qs + 2 * a->cache.kv_heads * D, "sb_attn_store: qkv_stride %u below the packed row", a->qkv_stride);
  SB_REQUIRE(2 * a->pairs <= D && (a->pairs == 0 || (a->cos_tab && a->sin_tab)), "sb_attn_store: %u rotary pairs exceed the head, or no tables", a->pairs);
  const uint32_t lanes = std::max(1u, a->lanes);
  SB_REQUIRE(lanes == 1 || (a->rows <= kLaneRows && a->committed_dev && lanes <= 64), "sb_attn_store: %u lanes need rows <= 16 and the lanes' positions on the device", lanes);
  StoreParams p{static_cast<const uint16_t *>(a->qkv), a->q_norm, a->k_norm, a->cos_tab, a->sin_tab, a->page_table,
                static_cast<uint16_t *>(a->queries), a->cache, a->committed_dev, a->rows, a->q_heads, a->gated, a->pairs, a->qkv_stride, a->committed,
                a->page_table_stride};
  const dim3 grid(a->q_heads + a->cache.kv_heads, a->rows, lanes);
  if (D == 256) return launch(attn_store_kernel<256>, grid, dim3(256), as_stream(stream), p);
  return launch(attn_store_kernel<128>, grid, dim3(128), as_stream(stream), p);
}

int sb_kv_path_commit(void *stream, const SbKvLayer *cache, const uint32_t *page_table, uint32_t committed,
                      const uint32_t *path_mask_dev) {
  SB_NEED_DEVICE();
  SB_REQUIRE(cache && page_table && path_mask_dev, "sb_kv_path_commit: null pointer");
  int st = check_cache(*cache, "sb_kv_path_commit");
  if (st != SB_OK) return st;
  return launch(kv_path_commit_kernel, dim3(cache->kv_heads), dim3(cache->head_dim), as_stream(stream), *cache, page_table,
                committed, static_cast<const uint32_t *>(nullptr), path_mask_dev, 0u, 0u);
}

int sb_kv_path_commit_lanes(void *stream, const SbKvLayer *cache, const uint32_t *page_table, uint32_t page_table_stride,
                            const uint32_t *committed_dev, const uint32_t *path_mask_dev, uint32_t mask_stride, uint32_t lanes) {
  SB_NEED_DEVICE();
  SB_REQUIRE(cache && page_table && committed_dev && path_mask_dev && lanes >= 1 && lanes <= 64, "sb_kv_path_commit_lanes: null pointer, or %u lanes (1..64)", lanes);
  int st = check_cache(*cache, "sb_kv_path_commit_lanes");
  if (st != SB_OK) return st;
  return launch(kv_path_commit_kernel, dim3(cache->kv_heads, lanes), dim3(cache->head_dim), as_stream(stream), *cache, page_table, 0u, committed_dev,
                path_mask_dev, page_table_stride, mask_stride);
}

int sb_kv_path_commit_at(void *stream, const SbKvLayer *cache, const uint32_t *page_table, const uint32_t *committed_dev,
                         const uint32_t *path_mask_dev) {
  SB_NEED_DEVICE();
  SB_REQUIRE(cache && page_table && committed_dev && path_mask_dev, "sb_kv_path_commit_at: null pointer");
  int st = check_cache(*cache, "sb_kv_path_commit_at");
  if (st != SB_OK) return st;
  return launch(kv_path_commit_kernel, dim3(cache->kv_heads), dim3(cache->head_dim), as_stream(stream), *cache, page_table, 0u, committed_dev,
                path_mask_dev, 0u, 0u);
}

uint64_t sb_sample_workspace_bytes(uint32_t rows, uint32_t vocab) {
  return uint64_t(rows) * (2 * ((vocab + kShard - 1) / kShard) + 8) * sizeof(float);
}

int sb_sample_verify(void *stream, const SbSampleArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->logits && a->selected && a->input_tokens, "sb_sample_verify: null pointer");
  SB_REQUIRE(a->rows >= 1 && a->rows <= 16 && a->vocab >= 1 && a->logit_stride >= a->vocab, "sb_sample_verify: rows %u outside 1..16 or bad vocabulary extent", a->rows);
  SB_REQUIRE(a->temperature >= 0.0f, "sb_sample_verify: negative temperature");
  SB_REQUIRE(a->temperature == 0.0f || (a->uniforms && a->workspace), "sb_sample_verify: a sampled policy needs uniforms and a workspace");
  SB_REQUIRE(a->min_p >= 0.0f && a->min_p <= 1.0f && a->top_p >= 0.0f, "sb_sample_verify: min_p %g outside 0..1 or negative top_p", double(a->min_p));
  const bool filtered = a->min_p > 0.0f || (a->top_k > 0 && a->top_k < a->vocab) || (a->top_p > 0.0f && a->top_p < 1.0f);
  SB_REQUIRE(!filtered || a->vocab <= kMaxFilterShards * kShard, "sb_sample_verify: min-p / top-k / top-p support vocabularies up to %u", kMaxFilterShards * kShard);
  SB_REQUIRE(!a->candidate_ids || (a->candidate_q && a->draws), "sb_sample_verify: candidates come with their draft probabilities and the rows' draws");
  SB_REQUIRE(a->lanes <= 64, "sb_sample_verify: %u lanes (up to 64)", a->lanes);
  SB_REQUIRE(!a->lane_policies || (a->uniforms && a->workspace && a->vocab <= kMaxFilterShards * kShard), "sb_sample_verify: policies a lane need uniforms, the workspace and a vocabulary the filters take");
  return launch(sample_kernel, dim3(a->rows, std::max(1u, a->lanes)), dim3(kSampleThreads), as_stream(stream), *a);
}

int sb_sample_admit(void *stream, const SbAdmitArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->logits && (a->masks || a->n_excluded), "sb_sample_admit: null logits, or neither masks nor excluded tokens");
  SB_REQUIRE(a->rows >= 1 && a->rows <= 32 && a->vocab >= 1 && a->logit_stride >= a->vocab, "sb_sample_admit: rows %u outside 1..32 or bad vocabulary extent", a->rows);
  SB_REQUIRE(!a->masks || a->mask_words >= (a->vocab + 31) / 32, "sb_sample_admit: %u mask words a row do not cover %u tokens", a->mask_words, a->vocab);
  SB_REQUIRE(a->n_excluded <= 16 && (!a->n_excluded || a->excluded), "sb_sample_admit: up to 16 excluded tokens, with their ids");
  SB_REQUIRE(a->lanes <= 64 && (a->lanes <= 1 || a->rows <= kLaneRows), "sb_sample_admit: %u lanes (up to 64, of up to 16 rows)", a->lanes);
  return launch(admit_kernel, dim3((a->vocab + 255) / 256, std::max(1u, a->lanes)), dim3(256), as_stream(stream), *a);
}

int sb_sample_penalize(void *stream, const SbPenaltyArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->logits && a->words && a->input_tokens && a->tree, "sb_sample_penalize: null pointer");
  SB_REQUIRE(a->rows >= 1 && a->rows <= 32 && a->vocab >= 1 && a->logit_stride >= a->vocab, "sb_sample_penalize: rows %u outside 1..32 or bad vocabulary extent",
             a->rows);
  SB_REQUIRE(a->repetition > 0.0f, "sb_sample_penalize: repetition %g is not positive", double(a->repetition));
  SB_REQUIRE(a->lanes <= 64 && (a->lanes <= 1 || a->rows <= kLaneRows), "sb_sample_penalize: %u lanes (up to 64, of up to 16 rows)", a->lanes);
  return launch(penalize_kernel, dim3((a->vocab + 255) / 256, std::max(1u, a->lanes)), dim3(256), as_stream(stream), *a);
}

int sb_moe_route(void *stream, const SbMoeRouteArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->scores && a->selected && a->weights, "sb_moe_route: null pointer");
  SB_REQUIRE(a->rows >= 1 && a->experts >= 1 && a->experts <= 256 && a->slots >= a->experts, "sb_moe_route: %u experts in %u slots (up to 256)", a->experts, a->slots);
  SB_REQUIRE(a->top_k >= 1 && a->top_k <= 32 && a->top_k <= a->experts, "sb_moe_route: top_k = %u outside 1..min(32, experts)", a->top_k);
  SB_REQUIRE(!a->shared_gate || (a->input && a->input_size), "sb_moe_route: a gated shared expert needs the rows' input");
  return launch(moe_route_kernel, dim3(a->rows), dim3(256), as_stream(stream), *a);
}

int sb_select_accept(void *stream, const SbSelectAcceptArgs *c) {
  SB_NEED_DEVICE();
  SB_REQUIRE(c && c->tickets, "sb_select_accept: null pointer");
  const SbSampleArgs *a = &c->sample;
  const SbAcceptArgs *b = &c->accept;
  SB_REQUIRE(a->logits && a->selected && a->input_tokens, "sb_select_accept: null pointer");
  SB_REQUIRE(a->rows >= 1 && a->rows <= 16 && a->vocab >= 1 && a->logit_stride >= a->vocab, "sb_select_accept: rows %u outside 1..16 or bad vocabulary extent", a->rows);
  SB_REQUIRE(a->temperature >= 0.0f, "sb_select_accept: negative temperature");
  SB_REQUIRE(a->temperature == 0.0f || (a->uniforms && a->workspace), "sb_select_accept: a sampled policy needs uniforms and a workspace");
  SB_REQUIRE(a->min_p >= 0.0f && a->min_p <= 1.0f && a->top_p >= 0.0f, "sb_select_accept: min_p %g outside 0..1 or negative top_p", double(a->min_p));
  const bool filtered = a->min_p > 0.0f || (a->top_k > 0 && a->top_k < a->vocab) || (a->top_p > 0.0f && a->top_p < 1.0f);
  SB_REQUIRE(!filtered || a->vocab <= kMaxFilterShards * kShard, "sb_select_accept: min-p / top-k / top-p support vocabularies up to %u", kMaxFilterShards * kShard);
  SB_REQUIRE(!a->candidate_ids || (a->candidate_q && a->draws), "sb_select_accept: candidates come with their draft probabilities and the rows' draws");
  SB_REQUIRE(a->lanes <= 64, "sb_select_accept: %u lanes (up to 64)", a->lanes);
  SB_REQUIRE(!a->lane_policies || (a->uniforms && a->workspace && a->vocab <= kMaxFilterShards * kShard), "sb_select_accept: policies a lane need uniforms, the workspace and a vocabulary the filters take");
  SB_REQUIRE(b->input_tokens == a->input_tokens && b->tokens == a->selected && b->tree && b->results, "sb_select_accept: acceptance reads the selection's rows: same input tokens, tokens = selected");
  SB_REQUIRE(b->rows == a->rows && b->remaining >= 1 && std::max(1u, b->lanes) == std::max(1u, a->lanes), "sb_select_accept: selection and acceptance disagree on rows or lanes");
  SB_REQUIRE(b->n_stop == 0 || b->stop_tokens, "sb_select_accept: stop tokens missing");
  SB_REQUIRE(!c->committed || (c->pending_rows && c->pending_path), "sb_select_accept: the commit needs the lanes' pending words");
  SB_REQUIRE((c->advance & 0xffu) <= 3 && ((c->advance & 0xffu) != 3 || c->advance >> 8 == a->rows), "sb_select_accept: advance = 0x%x", c->advance);
  return launch(select_accept_kernel, dim3(a->rows, std::max(1u, a->lanes)), dim3(kSampleThreads), as_stream(stream), *c);
}

int sb_accept(void *stream, const SbAcceptArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a && a->input_tokens && a->tree && a->tokens && a->results, "sb_accept: null pointer");
  SB_REQUIRE(a->rows >= 1 && a->rows <= 32 && a->remaining >= 1, "sb_accept: rows %u outside 1..32 or nothing remaining", a->rows);
  SB_REQUIRE(a->n_stop == 0 || a->stop_tokens, "sb_accept: stop tokens missing");
  SB_REQUIRE(a->lanes <= 64 && (a->lanes <= 1 || a->rows <= kLaneRows), "sb_accept: %u lanes (up to 64, of up to 16 rows)", a->lanes);
  return launch(accept_kernel, dim3(std::max(1u, a->lanes)), dim3(32), as_stream(stream), *a);
}

/* Programmatic dependent launch for the glue kernels of this context (on by default). */
int sb_set_pdl(int enabled) {
  ctx().pdl = enabled != 0;
  return SB_OK;
}

}  // extern "C"
