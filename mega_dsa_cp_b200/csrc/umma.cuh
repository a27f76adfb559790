// tcgen05 (5th-generation tensor core) primitives for sm_100a, as inline PTX:
// tensor-memory allocation, UMMA issue with the A operand in tensor memory and
// the B operand in shared memory, commit-to-mbarrier, and 32-lane x 32-bit
// tensor-memory loads / stores.
#pragma once

#include "common.cuh"

namespace mdc {
namespace umma {

// ---- tensor memory ---------------------------------------------------------
// A TMEM address is (lane << 16) | column; a warp may only touch the 32 lanes
// of its quadrant (warp index % 4).
__device__ inline void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
  // The allocation permit is NOT relinquished: a persistent block allocates again for its next
  // task, and an allocation after a relinquish is an error.  One block owns the SM anyway.
}
__device__ inline void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ inline void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ inline void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 16 consecutive 32-bit columns, one row per thread of the warp
__device__ inline void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
          taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ inline void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// true in exactly one lane of the (converged) warp
__device__ inline bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " elect.sync _|p, 0xffffffff;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ---- descriptors -------------------------------------------------------------
// Shared-memory operand, K-major, 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart, 16-byte chunk j of row r stored at chunk j ^ (r % 8).
// `addr` = shared address of the first row (+ 32 bytes per K step of 16 halves).
__device__ inline uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);        // start address
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16: fp16 (fmt 0) or bf16 (fmt 1) operands,
// fp32 accumulator, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, int ab_fmt) {
  return (1u << 4) | (static_cast<uint32_t>(ab_fmt) << 7) | (static_cast<uint32_t>(ab_fmt) << 10) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// D[tmem] (+)= A[tmem] * B[smem]^T ; issued by one thread.
__device__ inline void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// One 128-token stage of the indexer: eight K=16 steps into one accumulator,
// A = 64 consecutive tensor-memory columns (8 per step), B = eight prepared
// shared-memory descriptors.  A single asm block keeps the issuing thread's
// instruction count at the minimum (two predicates, then eight MMAs).
__device__ inline void mma_f16_ts_x8(uint32_t d_tmem, uint32_t a_tmem, const uint64_t (&b)[8], uint32_t idesc) {
  asm volatile(
      "{\n"
      " .reg .pred pf, pt;\n"
      " .reg .b32 a1, a2, a3, a4, a5, a6, a7;\n"
      " setp.ne.b32 pf, 0, 0;\n"
      " setp.eq.b32 pt, 0, 0;\n"
      " add.u32 a1, %1, 8;\n"
      " add.u32 a2, %1, 16;\n"
      " add.u32 a3, %1, 24;\n"
      " add.u32 a4, %1, 32;\n"
      " add.u32 a5, %1, 40;\n"
      " add.u32 a6, %1, 48;\n"
      " add.u32 a7, %1, 56;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %2, pf;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %4, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %5, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %6, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a4], %7, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a5], %8, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a6], %9, %2, pt;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [a7], %10, %2, pt;\n"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(idesc), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7])
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T
__device__ inline void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Arrive on `bar` once every tcgen05 operation issued so far by this thread has completed.
__device__ inline void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

}  // namespace umma
}  // namespace mdc
