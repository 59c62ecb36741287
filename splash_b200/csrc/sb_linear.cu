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
//   grid      one persistent CTA per SM (a multiple of the k-slice count), 288 threads:
//             warps 0..7 consume, warp 8 produces
//   k-slices  K's super-blocks are cut into S contiguous slices; a CTA owns one slice for the whole
//             launch and keeps its 16 x slice activations resident in shared memory, converted
//             once to fp16 with a per-row power-of-two scale (exact for bf16 inputs within 2^-27
//             of the row's largest magnitude) in the order the MMA fragments read them
//   tiles     64 weight rows x slice; the producer warp streams each tile's rows into a ring of
//             stages (64 rows x 4 super-blocks) with 1-D bulk async copies completing on
//             mbarriers; consumer warp (rg, kg) multiplies rows 32 rg..32 rg+31 of super-block kg
//             of each stage: mma.sync m16n8k16 (A = 16 weight rows, B = 8 tokens) into fp32
//   Q4_K      operand = sc*q (exact integer <= 945 in fp16, built as (1024+q)*sc - 1024*sc with one
//             LOP3 and one HFMA2 per two weights); per super-block y += d*Aq - dmin*Am, where Am is
//             one more MMA of the 6-bit mins against the sub-block sums of x (split hi + lo fp16)
//   Q6_K      operand = fp16(sc*(q-32)) (one rounding when |.| > 2048); y += d*Aq per super-block
//   Q8_0      operand = fp16(d*q), the value the reference's staged tile rounds to
//   reduce    the 4 k-group warps of a tile add their sums in order through shared memory; with
//             S > 1 the slices publish fp32 partials and the last arriver adds them in slice order
//             (runtime/metal/kernels/common/split_reduce.h:24-55), then applies the epilogue
//             (runtime/metal/kernels/common/gguf_tile.h:8-14, gguf_linear.metal:38)
#include "sb_internal.h"
#include "sb_ptx.cuh"

namespace sb {

constexpr int kTokens = 16;         // rows of X one launch multiplies
constexpr int kConsumerWarps = 8;
constexpr int kThreads = 32 * (kConsumerWarps + 1);
constexpr int kRG = 2, kKG = 4, kMT = 2;  // row groups x k groups of consumer warps; m-tiles per warp
constexpr int kTileRows = kRG * kMT * 16; // 64
constexpr int kStageSb = kKG;             // super-blocks per ring stage
constexpr int kMaxStages = 8;
constexpr int kMaxSliceSb = 10;           // super-blocks of activations a CTA keeps resident (80 KiB)
constexpr int kRedPitch = 17;
constexpr uint32_t kXsbBytes = kTokens * 256 * 2;  // fp16 activations of one super-block
constexpr uint32_t kSxSbBytes = 512;               // hi/lo sub-block sums of one super-block

struct LinearParams {
  const uint8_t *w, *w2;
  const uint16_t *x, *aux;
  void *out;
  const float *norm_w;
  float *partials;
  uint32_t *counters, *status;
  uint32_t n, k, rows, x_stride, aux_stride, out_stride, epilogue, out_f32;
  uint32_t nsb, slices, tiles, stages, row_bytes, pitch, stage_bytes;
  uint32_t x_off, sx_off, red_off, ring_off;  // shared memory offsets
};

template <int FMT> struct WFmt;
template <> struct WFmt<SB_FMT_Q4K> { static constexpr uint32_t kSbBytes = 144; static constexpr bool kPairLayout = true; };
template <> struct WFmt<SB_FMT_Q6K> { static constexpr uint32_t kSbBytes = 210; static constexpr bool kPairLayout = false; };
template <> struct WFmt<SB_FMT_Q80> { static constexpr uint32_t kSbBytes = 272; static constexpr bool kPairLayout = false; };

__device__ __forceinline__ void slice_range(uint32_t nsb, uint32_t slices, uint32_t s, uint32_t &b0, uint32_t &b1) {
  b0 = s * nsb / slices;
  b1 = (s + 1) * nsb / slices;
}

// ---- activations: bf16 global -> scaled fp16 fragments in shared memory ----
// Each consumer warp converts tokens 2w and 2w+1 of the CTA's slice. A unit is the 16 bytes one
// lane of an MMA reads: 8 consecutive inputs in the order [0,2,1,3,4,6,5,7].
template <bool PAIR>
__device__ void stage_activations(const LinearParams &p, uint8_t *smem, uint32_t sb0, uint32_t sb1, float *scale_back,
                                  uint32_t warp, uint32_t lane) {
  uint8_t *xs = smem + p.x_off;
  __half *sx = reinterpret_cast<__half *>(smem + p.sx_off);
  const uint32_t k0 = sb0 * 256, k1 = sb1 * 256;
  for (uint32_t tok = 2 * warp; tok < 2 * warp + 2; ++tok) {
    const bool live = tok < p.rows;
    const uint16_t *row = p.x + size_t(tok) * p.x_stride;
    float inv = 1.0f;
    if (live && p.norm_w) {
      // Sum of squares over the whole row in a fixed order: lane-strided 8-element groups, then a
      // butterfly over the lanes.
      float ss = 0.0f;
      for (uint32_t k = 8 * lane; k < p.k; k += 256) {
        const uint4 v = *reinterpret_cast<const uint4 *>(row + k);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = bf16_bits_to_float(u[i] & 0xffffu), b = bf16_bits_to_float(u[i] >> 16);
          ss = fmaf(a, a, ss);
          ss = fmaf(b, b, ss);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = rsqrtf(ss / float(p.k) + 1e-6f);
    }
    auto load8 = [&](uint32_t k, float (&f)[8]) {
      if (!live) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.0f;
        return;
      }
      const uint4 v = *reinterpret_cast<const uint4 *>(row + k);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = bf16_bits_to_float(u[i] & 0xffffu);
        f[2 * i + 1] = bf16_bits_to_float(u[i] >> 16);
      }
      if (p.norm_w) {
        const float4 w0 = *reinterpret_cast<const float4 *>(p.norm_w + k);
        const float4 w1 = *reinterpret_cast<const float4 *>(p.norm_w + k + 4);
        const float wn[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = round_bf16((f[i] * inv) * wn[i]);
      }
    };
    // Pass 1: the slice's largest magnitude -> power-of-two scale keeping every value below 2^10.
    float mx = 0.0f;
    for (uint32_t k = k0 + 8 * lane; k < k1; k += 256) {
      float f[8];
      load8(k, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));  // NaN is ignored here; it survives in the values
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    int e = 0;
    if (mx > 0.0f && mx <= 3.0e38f) {
      (void)frexpf(mx, &e);  // mx = f * 2^e, f in [0.5, 1)
      e -= 10;
    }
    const float down = ldexpf(1.0f, -e);
    if (lane == 0) scale_back[tok] = ldexpf(1.0f, e);
    // Pass 2: convert and store in fragment order; lane L of an iteration holds inputs 8L..8L+7 of
    // one super-block.
    const uint32_t h = tok >> 3, g = tok & 7;
    for (uint32_t sb = sb0; sb < sb1; ++sb) {
      float f[8];
      load8(sb * 256 + 8 * lane, f);
      __half hv[8];
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        hv[i] = __float2half_rn(f[i] * down);
        sum += __half2float(hv[i]);
      }
      const uint32_t j = lane >> 2, q = lane & 3, lsb = sb - sb0;
      uint32_t unit;
      if (PAIR) unit = ((((lsb * 4 + q) * 2 + (j & 1)) * 2 + h) * 8 + g) * 4 + (j >> 1);
      else unit = (((lsb * 8 + j) * 2 + h) * 8 + g) * 4 + q;
      const __half2 p0 = __halves2half2(hv[0], hv[2]), p1 = __halves2half2(hv[1], hv[3]);
      const __half2 p2 = __halves2half2(hv[4], hv[6]), p3 = __halves2half2(hv[5], hv[7]);
      uint4 o;
      o.x = *reinterpret_cast<const uint32_t *>(&p0);
      o.y = *reinterpret_cast<const uint32_t *>(&p1);
      o.z = *reinterpret_cast<const uint32_t *>(&p2);
      o.w = *reinterpret_cast<const uint32_t *>(&p3);
      *reinterpret_cast<uint4 *>(xs + size_t(unit) * 16) = o;
      if (PAIR) {
        // Sub-block sums (32 inputs = 4 lanes), split into hi + lo halves for the mins' MMA.
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (q == 0) {
          const __half hi = __float2half_rn(sum);
          const __half lo = __float2half_rn(sum - __half2float(hi));
          const uint32_t at = (((lsb * 2 + h) * 8 + g) * 4 + (j >> 1)) * 4 + (j & 1) * 2;
          sx[at] = hi;
          sx[at + 1] = lo;
        }
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

template <int FMT>
__device__ __forceinline__ void multiply_super_block(const uint8_t *wbase, const uint32_t (&roff)[kMT][2],
                                                     const uint8_t *xs_sb, const uint8_t *sx_sb, uint32_t lane,
                                                     float (&y)[kMT][2][4]);

template <>
__device__ __forceinline__ void multiply_super_block<SB_FMT_Q4K>(const uint8_t *wbase, const uint32_t (&roff)[kMT][2],
                                                                 const uint8_t *xs_sb, const uint8_t *sx_sb,
                                                                 uint32_t lane, float (&y)[kMT][2][4]) {
  const uint32_t t = lane & 3;
  uint32_t q[kMT][2][8];
  Q4Scales sc[kMT][2];
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint8_t *row = wbase + roff[mt][r];
      sc[mt][r] = q4_scales(*reinterpret_cast<const uint4 *>(row), t);
      const uint4 lo = *reinterpret_cast<const uint4 *>(row + 16 + 32 * t);
      const uint4 hi = *reinterpret_cast<const uint4 *>(row + 32 + 32 * t);
      q[mt][r][0] = lo.x, q[mt][r][1] = lo.y, q[mt][r][2] = lo.z, q[mt][r][3] = lo.w;
      q[mt][r][4] = hi.x, q[mt][r][5] = hi.y, q[mt][r][6] = hi.z, q[mt][r][7] = hi.w;
    }
  float aq[kMT][2][4];
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 4; ++c) aq[mt][h][c] = 0.0f;
  const uint32_t kMagic = 0x64006400u;
#pragma unroll
  for (int i2 = 0; i2 < 4; ++i2) {
    uint4 bx[2][2];
#pragma unroll
    for (int p = 0; p < 2; ++p)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        bx[p][h] = *reinterpret_cast<const uint4 *>(xs_sb + ((((i2 * 2 + p) * 2 + h) * 32 + lane) << 4));
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
      for (int wi = 0; wi < 2; ++wi) {
        const uint32_t w0 = q[mt][0][2 * i2 + wi], w1 = q[mt][1][2 * i2 + wi];
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
    for (int mt = 0; mt < kMT; ++mt) {
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

template <>
__device__ __forceinline__ void multiply_super_block<SB_FMT_Q6K>(const uint8_t *wbase, const uint32_t (&roff)[kMT][2],
                                                                 const uint8_t *xs_sb, const uint8_t *,
                                                                 uint32_t lane, float (&y)[kMT][2][4]) {
  // Lane t of a row multiplies inputs 8t..8t+7 of each of the 8 groups of 32: for half n of the
  // block, ql[64n+8t..] (groups 4n, 4n+2 in its nibbles), ql[64n+32+8t..] (4n+1, 4n+3) and
  // qh[32n+8t..] (two bits per group). The 6-bit code lands in bits 4..9 of a half whose value is
  // 64 + code/... : 0x5400 | code << 4 = 64 + code, so (64 + code) * sc - 96 * sc = sc * (code - 32).
  const uint32_t t = lane & 3;
  const uint32_t kMagic = 0x54005400u, kLow = 0x00f000f0u, kHigh = 0x03000300u;
  float aq[kMT][2][4];
#pragma unroll
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 4; ++c) aq[mt][h][c] = 0.0f;
  float dscale[kMT][2];
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    uint2 qa[kMT][2], qb[kMT][2], qh[kMT][2];
    uint32_t ms[kMT][2][4], bs[kMT][2][4];
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
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
      for (int mt = 0; mt < kMT; ++mt)
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
  for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      y[mt][h][0] = fmaf(dscale[mt][0], aq[mt][h][0], y[mt][h][0]);
      y[mt][h][1] = fmaf(dscale[mt][0], aq[mt][h][1], y[mt][h][1]);
      y[mt][h][2] = fmaf(dscale[mt][1], aq[mt][h][2], y[mt][h][2]);
      y[mt][h][3] = fmaf(dscale[mt][1], aq[mt][h][3], y[mt][h][3]);
    }
}

template <>
__device__ __forceinline__ void multiply_super_block<SB_FMT_Q80>(const uint8_t *wbase, const uint32_t (&roff)[kMT][2],
                                                                 const uint8_t *xs_sb, const uint8_t *,
                                                                 uint32_t lane, float (&y)[kMT][2][4]) {
  // A "super-block" is 8 consecutive Q8_0 blocks {half d, 32 int8}. Lane t multiplies bytes
  // 8t..8t+7 of each block; the operand is fp16(d * q), the product rounded once.
  const uint32_t t = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 bx[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) bx[h] = *reinterpret_cast<const uint4 *>(xs_sb + (((j * 2 + h) * 32 + lane) << 4));
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt) {
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

// ---- the kernel ----
template <int FMT>
__global__ void __launch_bounds__(kThreads, 1) linear_kernel(const LinearParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + kMaxStages;
  float *scale_back = reinterpret_cast<float *>(smem + 128);      // 16 floats
  uint32_t *flags = reinterpret_cast<uint32_t *>(smem + 192);     // [0] arrival, [1] failed
  constexpr uint32_t kSb = WFmt<FMT>::kSbBytes;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t slice = blockIdx.x % p.slices;
  uint32_t sb0, sb1;
  slice_range(p.nsb, p.slices, slice, sb0, sb1);
  const uint32_t slice_sb = sb1 - sb0, chunks = (slice_sb + kStageSb - 1) / kStageSb;
  const uint32_t items = p.tiles * p.slices;
  const bool gate_up = p.epilogue == SB_EPILOGUE_GATE_UP;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    flags[0] = 0;
    flags[1] = 0;
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kConsumerWarps) {
    // ---- producer: weights do not depend on the previous kernel, so no dependency wait here ----
    const uint64_t policy = policy_evict_first();
    uint32_t fill = 0;  // stages issued so far
    bool ok = true;
    for (uint32_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const uint32_t tile = item / p.slices;
      for (uint32_t c = 0; c < chunks && ok; ++c, ++fill) {
        const uint32_t slot = fill % p.stages, round = fill / p.stages;
        if (round > 0) ok = mbar_wait(&empty[slot], (round - 1) & 1);
        if (!ok) break;
        const uint32_t csb0 = sb0 + c * kStageSb, nsb_c = min(uint32_t(kStageSb), sb1 - csb0);
        // Per row: [src, src + nsb_c * kSb) widened to 16-byte boundaries.
        uint32_t bytes[2];
        const uint8_t *src[2];
        uint32_t total = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t r = lane + 32 * i;
          uint32_t wrow;
          const uint8_t *wb;
          if (gate_up) {
            wrow = min(tile * 32 + (r & 31), p.n - 1);
            wb = r < 32 ? p.w : p.w2;
          } else {
            wrow = min(tile * kTileRows + r, p.n - 1);
            wb = p.w;
          }
          const uint8_t *s = wb + size_t(wrow) * p.row_bytes + size_t(csb0) * kSb;
          const uint32_t lead = uint32_t(reinterpret_cast<uintptr_t>(s) & 15u);
          src[i] = s - lead;
          bytes[i] = (lead + nsb_c * kSb + 15u) & ~15u;
          total += bytes[i];
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) mbar_arrive_expect_tx(&full[slot], total);
        __syncwarp();
        uint8_t *dst = smem + p.ring_off + slot * p.stage_bytes;
#pragma unroll
        for (int i = 0; i < 2; ++i)
          bulk_g2s_stream(dst + (lane + 32 * i) * p.pitch, src[i], bytes[i], &full[slot], policy);
      }
    }
    if (!ok && lane == 0) {
      atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
      flags[1] = 1;
    }
    // Do not leave while copies are in flight: wait (bounded) until the consumers have released the
    // last fill of every stage, which they do only after its bytes have landed.
    for (uint32_t f = fill > p.stages ? fill - p.stages : 0; f < fill; ++f)
      if (!mbar_wait(&empty[f % p.stages], (f / p.stages) & 1)) break;
    return;
  }

  // ---- consumers ----
  pdl_wait();
  if (WFmt<FMT>::kPairLayout) stage_activations<true>(p, smem, sb0, sb1, scale_back, warp, lane);
  else stage_activations<false>(p, smem, sb0, sb1, scale_back, warp, lane);
  named_bar_sync(1, 32 * kConsumerWarps);

  const uint32_t rg = warp / kKG, kg = warp % kKG;
  const uint32_t g = lane >> 2, t = lane & 3;
  (void)t;
  float *red = reinterpret_cast<float *>(smem + p.red_off);
  const uint32_t ctid = threadIdx.x;  // 0..255
  uint32_t drained = 0;
  for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
    const uint32_t tile = item / p.slices;
    float y[kMT][2][4];
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 4; ++c) y[mt][h][c] = 0.0f;
    for (uint32_t c = 0; c < chunks; ++c, ++drained) {
      const uint32_t slot = drained % p.stages, round = drained / p.stages;
      if (!mbar_wait(&full[slot], round & 1)) {
        if (lane == 0) atomicExch(p.status, SB_DEV_WAIT_EXPIRED);
        return;  // the launch has failed; the status word says so
      }
      const uint32_t csb0 = sb0 + c * kStageSb, nsb_c = min(uint32_t(kStageSb), sb1 - csb0);
      if (kg < nsb_c) {
        const uint8_t *stage = smem + p.ring_off + slot * p.stage_bytes;
        // Row r of the stage starts `lead` bytes into its slot: its global address modulo 16 (always 0
        // for Q4_K, whose rows are 16-byte multiples).
        const uint32_t lsb = csb0 + kg - sb0;
        uint32_t roff[kMT][2];
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t tr = rg * 32 + mt * 16 + r * 8 + g;
            uint32_t lead = 0;
            if (FMT != SB_FMT_Q4K) {
              const uint32_t wrow = gate_up ? min(tile * 32 + (tr & 31), p.n - 1) : min(tile * kTileRows + tr, p.n - 1);
              const uint8_t *wb = (gate_up && tr >= 32) ? p.w2 : p.w;
              lead = uint32_t((reinterpret_cast<uintptr_t>(wb) + size_t(wrow) * p.row_bytes + size_t(csb0) * kSb) & 15u);
            }
            roff[mt][r] = tr * p.pitch + lead + kg * kSb;
          }
        multiply_super_block<FMT>(stage, roff, smem + p.x_off + lsb * kXsbBytes, smem + p.sx_off + lsb * kSxSbBytes,
                                  lane, y);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[slot]);
    }
    // ---- tile reduce over the k-group warps, in order ----
    named_bar_sync(2, 32 * kConsumerWarps);  // the previous tile's readers are done with `red`
    float *mine = red + warp * (32 * kRedPitch);
#pragma unroll
    for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mine[(mt * 16 + g) * kRedPitch + h * 8 + 2 * t] = y[mt][h][0];
        mine[(mt * 16 + g) * kRedPitch + h * 8 + 2 * t + 1] = y[mt][h][1];
        mine[(mt * 16 + g + 8) * kRedPitch + h * 8 + 2 * t] = y[mt][h][2];
        mine[(mt * 16 + g + 8) * kRedPitch + h * 8 + 2 * t + 1] = y[mt][h][3];
      }
    named_bar_sync(1, 32 * kConsumerWarps);
    // Thread -> (token, 4 consecutive tile rows).
    const uint32_t tok = ctid >> 4, r4 = (ctid & 15) * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t r = r4 + i, wrg = r >> 5, rl = r & 31;
      float s = 0.0f;
#pragma unroll
      for (int k = 0; k < kKG; ++k) s += red[((wrg * kKG + k) * 32 + rl) * kRedPitch + tok];
      v[i] = s * scale_back[tok];
    }
    const uint32_t pcols = gate_up ? 2 * p.n : p.n;
    // Partial / output column of tile row r: plain tiles map rows to columns; a gate/up tile holds
    // 32 gate rows then 32 up rows of the same 32 columns.
    const uint32_t col0 = gate_up ? (r4 < 32 ? tile * 32 + r4 : p.n + tile * 32 + (r4 - 32)) : tile * kTileRows + r4;
    const bool col_ok = gate_up ? (tile * 32 + (r4 & 31) < p.n) : (col0 < p.n);  // n is a multiple of 4
    bool finish = true;
    if (p.slices > 1) {
      if (col_ok)
        *reinterpret_cast<float4 *>(p.partials + (size_t(slice) * kTokens + tok) * pcols + col0) =
            make_float4(v[0], v[1], v[2], v[3]);
      __threadfence();
      named_bar_sync(2, 32 * kConsumerWarps);
      if (ctid == 0) flags[0] = atomicAdd(&p.counters[tile], 1u);
      named_bar_sync(1, 32 * kConsumerWarps);
      finish = flags[0] == p.slices - 1;
      if (finish) {
        __threadfence();
        if (col_ok) {
          float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
          for (uint32_t sl = 0; sl < p.slices; ++sl) {
            const float4 q = __ldcg(reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * pcols + col0));
            s.x += q.x, s.y += q.y, s.z += q.z, s.w += q.w;
          }
          v[0] = s.x, v[1] = s.y, v[2] = s.z, v[3] = s.w;
        }
        if (ctid == 0) p.counters[tile] = 0;
      }
    }
    if (finish && tok < p.rows && col_ok) {
      if (!gate_up) {
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float a = v[i];
          if (p.epilogue == SB_EPILOGUE_RESIDUAL)
            a += bf16_bits_to_float(p.aux[size_t(tok) * p.aux_stride + col0 + i]);
          else if (p.epilogue == SB_EPILOGUE_UP_WITH_GATE)
            a = round_bf16(a) * silu_f(bf16_bits_to_float(p.aux[size_t(tok) * p.aux_stride + col0 + i]));
          o[i] = a;
        }
        if (p.out_f32) {
          *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + size_t(tok) * p.out_stride + col0) =
              make_float4(o[0], o[1], o[2], o[3]);
        } else {
          uint2 pk;
          pk.x = uint32_t(float_to_bf16_bits(o[0])) | (uint32_t(float_to_bf16_bits(o[1])) << 16);
          pk.y = uint32_t(float_to_bf16_bits(o[2])) | (uint32_t(float_to_bf16_bits(o[3])) << 16);
          *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(p.out) + size_t(tok) * p.out_stride + col0) = pk;
        }
      } else {
        // The up rows' threads (r4 >= 32) hold `up`; the gate sums sit 32 rows earlier in `red` or in
        // the partials: fetch them again so one thread owns both.
        if (r4 >= 32) {
          float gsum[4];
          if (p.slices > 1) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t sl = 0; sl < p.slices; ++sl) {
              const float4 q = __ldcg(reinterpret_cast<const float4 *>(p.partials + (size_t(sl) * kTokens + tok) * pcols + (col0 - p.n)));
              s.x += q.x, s.y += q.y, s.z += q.z, s.w += q.w;
            }
            gsum[0] = s.x, gsum[1] = s.y, gsum[2] = s.z, gsum[3] = s.w;
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t rl = (r4 - 32) + i;
              float s = 0.0f;
#pragma unroll
              for (int k = 0; k < kKG; ++k) s += red[((0 * kKG + k) * 32 + rl) * kRedPitch + tok];
              gsum[i] = s * scale_back[tok];
            }
          }
          const uint32_t oc = col0 - p.n;
          uint32_t ob[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) ob[i] = float_to_bf16_bits(round_bf16(v[i]) * silu_f(round_bf16(gsum[i])));
          uint2 pk;
          pk.x = ob[0] | (ob[1] << 16);
          pk.y = ob[2] | (ob[3] << 16);
          *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(p.out) + size_t(tok) * p.out_stride + oc) = pk;
        }
      }
    }
  }
}

// ---- host side ----
static uint32_t pick_slices(uint32_t nsb, int sms) {
  uint32_t s = (nsb + kMaxSliceSb - 1) / kMaxSliceSb;
  return s < 1 ? 1 : s;
}

static int make_plan(uint32_t format, uint32_t n, uint32_t k, uint32_t epilogue, LinearParams &p, SbLinearPlan &plan) {
  FmtInfo fi;
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80,
             "sb_linear: format %u is not a quantized block format of this kernel", format);
  fmt_info(format, fi);
  SB_REQUIRE(k && k % 256 == 0, "sb_linear: k = %u is not a multiple of 256", k);
  SB_REQUIRE(n && n % 4 == 0, "sb_linear: n = %u is not a multiple of 4", n);
  const bool gate_up = epilogue == SB_EPILOGUE_GATE_UP;
  const uint32_t sb_bytes = format == SB_FMT_Q4K ? 144 : format == SB_FMT_Q6K ? 210 : 272;
  p.nsb = k / 256;
  p.slices = pick_slices(p.nsb, ctx().sm_count);
  p.tiles = gate_up ? (n + 31) / 32 : (n + kTileRows - 1) / kTileRows;
  p.row_bytes = uint32_t(sb_row_bytes(format, k));
  // Row pitch of a stage: the widened copy of kStageSb super-blocks, with the pitch congruent to 16
  // modulo 32 so the 16-byte reads of 8 rows x 4 lanes spread over all banks.
  uint32_t pitch = (kStageSb * sb_bytes + 15 + 15) & ~15u;
  if (format == SB_FMT_Q4K) pitch = kStageSb * sb_bytes;
  if (pitch % 32 != 16) pitch += 16;
  p.pitch = pitch;
  p.stage_bytes = (kTileRows * pitch + 127) & ~127u;
  const uint32_t slice_max = (p.nsb + p.slices - 1) / p.slices;
  p.x_off = 256;
  p.sx_off = p.x_off + slice_max * kXsbBytes;
  p.red_off = p.sx_off + slice_max * kSxSbBytes;
  p.ring_off = (p.red_off + kConsumerWarps * 32 * kRedPitch * 4 + 127) & ~127u;
  const uint32_t budget = 227 * 1024;
  SB_REQUIRE(p.ring_off + 2 * p.stage_bytes <= budget, "sb_linear: shared memory plan does not fit (k = %u)", k);
  p.stages = min(uint32_t(kMaxStages), (budget - p.ring_off) / p.stage_bytes);
  const uint32_t sms = uint32_t(ctx().sm_count ? ctx().sm_count : 148);
  uint32_t ctas = sms / p.slices * p.slices;
  const uint32_t items = p.tiles * p.slices;
  if (ctas > items) ctas = items;
  plan = {p.slices, ctas, uint32_t(kTileRows), p.stages, p.ring_off + p.stages * p.stage_bytes, uint32_t(kStageSb),
          slice_max, p.tiles};
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

extern "C" int sb_linear(void *stream, const SbLinearArgs *a) {
  SB_NEED_DEVICE();
  SB_REQUIRE(a, "sb_linear: null arguments");
  SB_REQUIRE(a->weights && a->x && a->out, "sb_linear: null weights, x or out");
  SB_REQUIRE(a->rows >= 1 && a->rows <= kTokens, "sb_linear: rows = %u outside 1..%d", a->rows, kTokens);
  SB_REQUIRE(a->epilogue <= SB_EPILOGUE_GATE_UP, "sb_linear: unknown epilogue %u", a->epilogue);
  SB_REQUIRE((a->epilogue == SB_EPILOGUE_GATE_UP) == (a->weights2 != nullptr),
             "sb_linear: weights2 is given exactly with SB_EPILOGUE_GATE_UP");
  SB_REQUIRE((a->epilogue == SB_EPILOGUE_RESIDUAL || a->epilogue == SB_EPILOGUE_UP_WITH_GATE) == (a->aux != nullptr),
             "sb_linear: aux is given exactly with the residual and up-with-gate epilogues");
  SB_REQUIRE(a->x_stride >= a->k && a->x_stride % 8 == 0, "sb_linear: x_stride %u < k or not a multiple of 8", a->x_stride);
  SB_REQUIRE(a->out_stride >= a->n && a->out_stride % 4 == 0, "sb_linear: out_stride %u < n or not a multiple of 4", a->out_stride);
  SB_REQUIRE(!a->aux || a->aux_stride >= a->n, "sb_linear: aux_stride %u < n", a->aux_stride);
  SB_REQUIRE(!(a->out_f32 && a->epilogue != SB_EPILOGUE_NONE), "sb_linear: an fp32 destination takes no epilogue");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(a->x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->out) & 15) == 0,
             "sb_linear: x and out must be 16-byte aligned");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(a->weights) & 1) == 0, "sb_linear: weights must be 2-byte aligned");
  LinearParams p{};
  SbLinearPlan plan;
  const int st = make_plan(a->format, a->n, a->k, a->epilogue, p, plan);
  if (st != SB_OK) return st;
  if (a->format == SB_FMT_Q4K)
    SB_REQUIRE((reinterpret_cast<uintptr_t>(a->weights) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a->weights2) & 15) == 0,
               "sb_linear: Q4_K weights must be 16-byte aligned");
  Context &c = ctx();
  const uint32_t pcols = a->epilogue == SB_EPILOGUE_GATE_UP ? 2 * a->n : a->n;
  SB_REQUIRE(p.slices == 1 || size_t(p.slices) * kTokens * pcols * 4 <= c.linear_partials_bytes,
             "sb_linear: split-K scratch too small for n = %u with %u slices", a->n, p.slices);
  SB_REQUIRE(p.tiles <= c.linear_counter_count, "sb_linear: too many tiles (%u)", p.tiles);
  p.w = static_cast<const uint8_t *>(a->weights);
  p.w2 = static_cast<const uint8_t *>(a->weights2);
  p.x = static_cast<const uint16_t *>(a->x);
  p.aux = static_cast<const uint16_t *>(a->aux);
  p.out = a->out;
  p.norm_w = static_cast<const float *>(a->norm_weight);
  p.partials = c.linear_partials;
  p.counters = c.linear_counters;
  p.status = c.status_dev;
  p.n = a->n, p.k = a->k, p.rows = a->rows;
  p.x_stride = a->x_stride, p.aux_stride = a->aux_stride, p.out_stride = a->out_stride;
  p.epilogue = a->epilogue, p.out_f32 = a->out_f32;

  void (*kernel)(const LinearParams) = a->format == SB_FMT_Q4K   ? linear_kernel<SB_FMT_Q4K>
                                       : a->format == SB_FMT_Q6K ? linear_kernel<SB_FMT_Q6K>
                                                                 : linear_kernel<SB_FMT_Q80>;
  static bool attr_set[3] = {false, false, false};
  const int ki = a->format == SB_FMT_Q4K ? 0 : a->format == SB_FMT_Q6K ? 1 : 2;
  if (!attr_set[ki]) {
    SB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[ki] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan.ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = plan.smem_bytes;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (a->flags & SB_LINEAR_PDL) ? 1 : 0;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return SB_OK;
}
