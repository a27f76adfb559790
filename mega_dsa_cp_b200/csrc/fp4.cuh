// E2M1 (FP4) block-scaled decode helpers for sm_100a.
//
// Packed layout: two codes per byte, even element in the low nibble.  The
// conversions below are exact: an E2M1 value times a UE4M3 or (in-range) UE8M0
// scale has at most 6 significant bits and fits fp16 without rounding as long
// as the scale exponent stays inside [-23, 13]; scales outside that range
// saturate to 0 / inf like any fp16 conversion.
#pragma once

#include "common.cuh"

namespace mdc {

// 8 packed E2M1 codes -> 4 x f16x2 (element 2i in the low half of out[i]).
__device__ inline void e2m1x8_to_f16x2(uint32_t w, uint32_t (&out)[4]) {
  asm("{\n"
      " .reg .b8 b0, b1, b2, b3;\n"
      " mov.b32 {b0, b1, b2, b3}, %4;\n"
      " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      " cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}"
      : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
      : "r"(w));
}

// two UE4M3 scale bytes -> f16x2 (byte 0 in the low half)
__device__ inline uint32_t e4m3x2_to_f16x2(uint16_t two) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(two));
  return r;
}

// UE8M0 byte -> fp16 bits of 2^(e-127), replicated in both halves
__device__ inline uint32_t ue8m0_to_f16x2(uint32_t e) {
  __half h = __float2half_rn(__uint_as_float(e << 23));
  uint32_t b = __half_as_ushort(h);
  return b | (b << 16);
}

__device__ inline uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

__device__ inline uint32_t bcast_lo(uint32_t x) { return __byte_perm(x, x, 0x1010); }
__device__ inline uint32_t bcast_hi(uint32_t x) { return __byte_perm(x, x, 0x3232); }

// fp32 value of one E2M1 code (sign in bit 3)
__device__ inline float e2m1_to_float(uint32_t code) {
  const uint32_t m = code & 7u;
  // 0, .5, 1, 1.5, 2, 3, 4, 6
  float v = (m < 2u) ? 0.5f * static_cast<float>(m)
                     : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -v : v;
}

__device__ inline void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ inline void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace mdc

namespace mdc {
// packed fp32 pair multiply-add of sm_100: d = a * b + c on both halves
__device__ inline void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  unsigned long long a, b, c;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(d0), "f"(d1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(c));
}
}  // namespace mdc
