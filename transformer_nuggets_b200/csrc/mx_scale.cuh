// MXFP8 scale arithmetic shared by the tile quantizer and the fused producer kernels:
// E8M0 byte and power-of-two multiplier from a block's bf16 amax bits, and the exact
// widen-and-scale of packed bf16 pairs.
#pragma once

#include "common.cuh"

namespace tnq {

__device__ __forceinline__ uint32_t abs_pk_bf16(uint32_t a) {
  uint32_t r;
  asm("abs.bf16x2 %0, %1;" : "=r"(r) : "r"(a));
  return r;
}

// amax bits (15-bit bf16 magnitude) -> scale byte and the multiplier 2^-e as a bf16 pair
// (same value in both halves).
template <int MODE>
__device__ __forceinline__ void e8m0_from_amax(uint32_t m16, uint32_t& byte, uint32_t& inv_pair) {
  const int bias = (MODE == TNQ_E8M0_CEIL) ? (0x1f - 1024) : -1024;  // (m + 0x1f) >> 7, minus 8
  byte = (uint32_t)max(((int)m16 + bias) >> 7, 1);
  inv_pair = 0x7f007f00u - byte * 0x00800080u;  // ((254 - byte) << 7) in both halves
}

// two scaled bf16 pairs -> four e4m3 bytes (a.lo, a.hi, b.lo, b.hi)
__device__ __forceinline__ uint32_t e4m3x4_from_pk(uint32_t a, uint32_t b) {
  return cvt_fp8x4<TNQ_FP8_E4M3>(bf16lo(a), bf16hi(a), bf16lo(b), bf16hi(b));
}

// Widen-and-scale in one step: fp32 = bf16 * bf16 + (-0.0) with the mixed-precision FMA
// of sm_100 (the product of a bf16 and a power of two is exact in fp32; adding -0.0
// keeps the sign of a zero product).  s16 = bf16 bits of the power-of-two multiplier.
__device__ __forceinline__ void widen_scale_pk(uint32_t w, uint16_t s16, float& lo, float& hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
      "fma.rn.f32.bf16 %0, l, %3, %4;\n\tfma.rn.f32.bf16 %1, h, %3, %4;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "r"(w), "h"(s16), "f"(-0.0f));
}
// the same with one multiplier per half (two adjacent columns with their own scales)
__device__ __forceinline__ void widen_scale_pk2(uint32_t w, uint16_t s_lo, uint16_t s_hi, float& lo, float& hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\t"
      "fma.rn.f32.bf16 %0, l, %3, %5;\n\tfma.rn.f32.bf16 %1, h, %4, %5;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "r"(w), "h"(s_lo), "h"(s_hi), "f"(-0.0f));
}
// two raw bf16 pairs and a power-of-two multiplier -> four e4m3 bytes
__device__ __forceinline__ uint32_t e4m3x4_scaled(uint32_t a, uint32_t b, uint16_t s16) {
  float a0, a1, b0, b1;
  widen_scale_pk(a, s16, a0, a1);
  widen_scale_pk(b, s16, b0, b1);
  return cvt_fp8x4<TNQ_FP8_E4M3>(a0, a1, b0, b1);
}

}  // namespace tnq
