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

// 8 packed E2M1 codes -> 4 x f16x2 holding value * 2^-14, element i in the low
// half and element i+4 in the high half of out[i].  Integer-only: the 3-bit
// magnitude code placed at bits 11..9 of an fp16 IS value * 2^-14 (codes 0 and 1
// land on fp16 subnormals 0 and 2^-15), the sign goes to bit 15; nibbles i and
// i+4 are 16 bits apart, so one shift serves both halves.  The caller
// multiplies by (block scale * 2^7), which yields value * scale * 2^-7 exactly
// in fp16 (at most 6 significant bits, magnitudes between 2^-17 and 21) for any
// UE4M3 scale; the remaining 2^7 is folded into the head weights.
constexpr uint32_t kF16x2_2p14 = 0x74007400u;
constexpr uint32_t kF16x2_2p7 = 0x58005800u;
__device__ inline void e2m1x8_pairs_f16(uint32_t w, uint32_t (&out)[4]) {
  out[0] = ((w << 12) & 0x80008000u) | ((w << 9) & 0x0E000E00u);
  out[1] = ((w << 8) & 0x80008000u) | ((w << 5) & 0x0E000E00u);
  out[2] = ((w << 4) & 0x80008000u) | ((w << 1) & 0x0E000E00u);
  out[3] = (w & 0x80008000u) | ((w >> 3) & 0x0E000E00u);
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

// UE8M0 byte -> fp16 bits of 2^(e-127+7), replicated in both halves
__device__ inline uint32_t ue8m0_to_f16x2_2p7(uint32_t e) {
  __half h = __float2half_rn(__uint_as_float(min(e + 7u, 254u) << 23));
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
