// Inline-PTX helpers for the 5th-generation tensor cores of sm_100a: tensor memory (TMEM)
// allocation, register <-> TMEM moves, the single-thread tcgen05.mma with its A operand in TMEM and
// its B operand described in shared memory, and the commit that turns completion of the issued MMAs
// into an mbarrier arrival.
#pragma once
#include <stdint.h>

#include "sb_ptx.cuh"

namespace sb {

// TMEM addresses are {lane[31:16], column[15:0]}; a warp reaches only the 32 lanes of its quadrant,
// 32 * (warp index % 4).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t column) {
  return base + (lane << 16) + column;
}

// Whole-warp calls. `columns` is a power of two >= 32; the base address lands in *slot (shared).
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Lane i of the warp writes r[0..15] to columns c..c+15 of TMEM lane (quadrant base + i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t r4,
                                         uint32_t r5, uint32_t r6, uint32_t r7) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r0), "r"(r1),
               "r"(r2), "r"(r3), "r"(r4), "r"(r5), "r"(r6), "r"(r7)
               : "memory");
}
// Lane i of the warp reads columns c..c+31 of TMEM lane (quadrant base + i) as fp32. The wait is part of
// the same statement, so no use of the values can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld32_wait(uint32_t taddr, float *v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same for 16 columns.
__device__ __forceinline__ void tmem_ld16_wait(uint32_t taddr, float *v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 48 columns (32 + 16) in one statement with the wait.
__device__ __forceinline__ void tmem_ld48_wait(uint32_t taddr, float *v) {
  uint32_t r[48];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%48];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47}, [%49];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47])
      : "r"(taddr), "r"(taddr + 32)
      : "memory");
#pragma unroll
  for (int i = 0; i < 48; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor, K-major, no swizzle: the operand is a grid of 8-row x 16-byte
// core matrices (128 contiguous bytes each); `lbo` is the byte distance between the two core matrices
// of one K = 16 step, `sbo` the distance between consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return uint64_t((smem_addr >> 4) & 0x3fffu) | (uint64_t((lbo >> 4) & 0x3fffu) << 16) | (uint64_t((sbo >> 4) & 0x3fffu) << 32) |
         (uint64_t(1) << 46);
}
// Instruction descriptor of kind::f16: fp16 A (K-major) and B (K-major, or MN-major = N contiguous), fp32
// accumulator, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n, bool b_mn_major = false) {
  return (1u << 4) | (b_mn_major ? 1u << 16 : 0u) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[tmem] * B[smem]^T for one K = 16 step; issued by one thread.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// One Q4_K super-block in a single statement, so the issuing thread spends three instructions per MMA. The 16
// K-steps (A columns a + 8 i, B tiles 512 i bytes on) alternate between two accumulators, D (even steps) and
// D + 16 (odd steps), so that consecutive MMAs do not wait for each other's result; a 17th MMA (A columns
// a + 128, B tile 16) writes the mins' sums to D + 32.
__device__ __forceinline__ void umma_q4k_super_block(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred pf, pt;\n\t"
      ".reg .b32 a, d1, dm;\n\t"
      ".reg .b64 b;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u32 d1, %0, 16;\n\t"
      "add.u32 dm, %0, 32;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
      "add.u32 a, %1, 8;\n\t"
      "add.u64 b, %2, 32;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pf;\n\t"
      "add.u32 a, %1, 128;\n\t"
      "add.u64 b, %2, 512;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [dm], [a], b, %3, pf;\n\t"
      "add.u32 a, %1, 16;\n\t"
      "add.u64 b, %2, 64;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 24;\n\t"
      "add.u64 b, %2, 96;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 32;\n\t"
      "add.u64 b, %2, 128;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 40;\n\t"
      "add.u64 b, %2, 160;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 48;\n\t"
      "add.u64 b, %2, 192;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 56;\n\t"
      "add.u64 b, %2, 224;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 64;\n\t"
      "add.u64 b, %2, 256;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 72;\n\t"
      "add.u64 b, %2, 288;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 80;\n\t"
      "add.u64 b, %2, 320;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 88;\n\t"
      "add.u64 b, %2, 352;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 96;\n\t"
      "add.u64 b, %2, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 104;\n\t"
      "add.u64 b, %2, 416;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 112;\n\t"
      "add.u64 b, %2, 448;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 120;\n\t"
      "add.u64 b, %2, 480;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d1], [a], b, %3, pt;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}
// The same super-block issued by two threads: thread `half` issues the K-steps of its parity into its own
// accumulator (D + 16 half); thread 0 also issues the mins' MMA into D + 32. The threads' MMAs are independent,
// so neither waits for the other's issue slot.
__device__ __forceinline__ void umma_q4k_super_block_half(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t half) {
  if (half == 0)
    asm volatile(
      "{\n\t"
      ".reg .pred pf, pt;\n\t"
      ".reg .b32 a, d;\n\t"
      ".reg .b64 b;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u32 d, %0, 0;\n\t"
      "add.u32 a, %1, 0;\n\t"
      "add.u64 b, %2, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pf;\n\t"
      "add.u32 a, %1, 16;\n\t"
      "add.u64 b, %2, 64;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 32;\n\t"
      "add.u64 b, %2, 128;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 48;\n\t"
      "add.u64 b, %2, 192;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 64;\n\t"
      "add.u64 b, %2, 256;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 80;\n\t"
      "add.u64 b, %2, 320;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 96;\n\t"
      "add.u64 b, %2, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 112;\n\t"
      "add.u64 b, %2, 448;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 128;\n\t"
      "add.u32 d, %0, 32;\n\t"
      "add.u64 b, %2, 512;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pf;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
  else
    asm volatile(
      "{\n\t"
      ".reg .pred pf, pt;\n\t"
      ".reg .b32 a, d;\n\t"
      ".reg .b64 b;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u32 d, %0, 16;\n\t"
      "add.u32 a, %1, 8;\n\t"
      "add.u64 b, %2, 32;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pf;\n\t"
      "add.u32 a, %1, 24;\n\t"
      "add.u64 b, %2, 96;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 40;\n\t"
      "add.u64 b, %2, 160;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 56;\n\t"
      "add.u64 b, %2, 224;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 72;\n\t"
      "add.u64 b, %2, 288;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 88;\n\t"
      "add.u64 b, %2, 352;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 104;\n\t"
      "add.u64 b, %2, 416;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "add.u32 a, %1, 120;\n\t"
      "add.u64 b, %2, 480;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [d], [a], b, %3, pt;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}
// The mbarrier receives one arrival when every MMA this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

}  // namespace sb
