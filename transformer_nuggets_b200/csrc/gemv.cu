// Block-scaled M = 1 GEMV on the quantizers' own output formats - the consumer that
// sits directly downstream of the casts:
//   MXFP8 : y[n] = sum_b 2^(sx[b]-127) * 2^(sw[n,b]-127) * sum_{k in b} x[k] * w[n,k]      (32-element blocks)
//   NVFP4 : y[n] = gx * gw * sum_b sx[b] * sw[n,b] * sum_{k in b} x[k] * w[n,k]            (16-element blocks)
// with e4m3 / packed e2m1 payloads, E8M0 / E4M3 block scales in raw row-major or
// swizzled 128x4 storage, fp32 accumulation, bf16 output.
//
// The weight matrix is read once from HBM (the kernel is bandwidth bound); x is decoded
// once per CTA into shared memory as fp16 together with its block factors.  A warp owns
// kRowsPerWarp output rows and walks K in 512-byte steps: each lane fetches one 16-byte
// weight chunk per row (all rows' loads in flight together), decodes it with the hardware
// cvt (e4m3x2 / e2m1x2 -> f16x2) and accumulates exact products in fp32 with the
// mixed-precision FMA (fma.rn.f32.f16); block scales are applied to the per-lane partial
// of each block, lanes are folded with shuffles at the end.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace tnq {

constexpr int kGemvThreads = 256;
constexpr int kRowsPerWarp = 4;
constexpr int kRowsPerCta = kRowsPerWarp * (kGemvThreads / 32);

// 2^(byte - 127) as fp32; byte 0 -> 2^-127 (subnormal), byte 255 -> NaN
__device__ __forceinline__ float e8m0_to_f32(uint32_t byte) {
  uint32_t bits = byte << 23;
  if (byte == 0u) bits = 0x00400000u;
  if (byte == 255u) bits = 0x7fc00000u;
  return __uint_as_float(bits);
}
__device__ __forceinline__ float e4m3_byte_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)byte));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
// d = a.lo * b.lo + c, then d = a.hi * b.hi + d   (fp16 products exact in fp32)
__device__ __forceinline__ float fma2_f16_f32(uint32_t a, uint32_t b, float c) {
  float d;
  asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t.reg .f32 t;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
      "fma.rn.f32.f16 t, al, bl, %3;\n\tfma.rn.f32.f16 %0, ah, bh, t;\n\t}"
      : "=f"(d)
      : "r"(a), "r"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((uint16_t)two_bytes));
  return r;
}
// four packed e2m1 codes (two bytes) -> two f16x2 words (codes 0,1 and 2,3)
__device__ __forceinline__ void cvt_e2m1x4_to_f16x2(uint32_t two_bytes, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b8 b0, b1;\n\t.reg .b16 h;\n\tcvt.u16.u32 h, %2;\n\tmov.b16 {b0, b1}, h;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(two_bytes));
}

__device__ __forceinline__ int64_t scale_index(int64_t r, int64_t c, int64_t w, int layout) {
  return layout == TNQ_SCALES_SWIZZLED ? swizzled_offset(r, c, (w + 3) / 4) : r * w + c;
}

// ---------------------------------------------------------------- MXFP8
// smem: x as fp16 [K] then block factors fp32 [K/32]
__global__ void __launch_bounds__(kGemvThreads)
    k_mxfp8_gemv(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, const uint8_t* __restrict__ x_sf,
                 const uint8_t* __restrict__ w_sf, int64_t n, int k, int layout, uint16_t* __restrict__ y) {
  extern __shared__ __align__(16) uint8_t tnq_gemv_smem[];
  uint32_t* xs = reinterpret_cast<uint32_t*>(tnq_gemv_smem);            // K/2 words of f16x2
  float* fx = reinterpret_cast<float*>(tnq_gemv_smem + (size_t)k * 2);  // K/32 factors
  const int kb = k / 32;
  for (int i = threadIdx.x; i < k / 2; i += kGemvThreads)
    xs[i] = cvt_e4m3x2_to_f16x2(reinterpret_cast<const uint16_t*>(x)[i]);
  for (int i = threadIdx.x; i < kb; i += kGemvThreads) fx[i] = e8m0_to_f32(x_sf[scale_index(0, i, kb, layout)]);
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int steps = k / 512;  // full 512-element steps; a ragged tail of whole 32-blocks follows
  for (int64_t row0 = ((int64_t)blockIdx.x * (kGemvThreads / 32) + warp) * kRowsPerWarp; row0 < n;
       row0 += (int64_t)gridDim.x * kRowsPerCta) {
    float acc[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) acc[r] = 0.0f;
    const int tail_chunks = (k - steps * 512) / 16;  // 16-element chunks after the full steps
    for (int s = 0; s <= steps; ++s) {
      const bool last = s == steps;
      if (last && lane >= tail_chunks) break;
      const int kc = s * 512 + lane * 16;  // this lane's 16 elements
      uint4 wv[kRowsPerWarp];
      uint32_t sb[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const int64_t row = row0 + r < n ? row0 + r : n - 1;
        wv[r] = ldg128(w + row * k + kc);
        sb[r] = w_sf[scale_index(row, kc >> 5, kb, layout)];
      }
      const uint4 xa = *reinterpret_cast<const uint4*>(xs + (kc >> 1));
      const uint4 xb = *reinterpret_cast<const uint4*>(xs + (kc >> 1) + 4);
      const float f = fx[kc >> 5];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        float p = 0.0f;
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].x & 0xffffu), xa.x, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].x >> 16), xa.y, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].y & 0xffffu), xa.z, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].y >> 16), xa.w, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].z & 0xffffu), xb.x, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].z >> 16), xb.y, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].w & 0xffffu), xb.z, p);
        p = fma2_f16_f32(cvt_e4m3x2_to_f16x2(wv[r].w >> 16), xb.w, p);
        acc[r] = __fmaf_rn(p, __fmul_rn(f, e8m0_to_f32(sb[r])), acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float v = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && row0 + r < n) y[row0 + r] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
  }
}

// ---------------------------------------------------------------- NVFP4
// smem: x as fp16 [K] then block factors fp32 [K/16] (e4m3 block scale * global input scale)
__global__ void __launch_bounds__(kGemvThreads)
    k_nvfp4_gemv(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, const uint8_t* __restrict__ x_sf,
                 const uint8_t* __restrict__ w_sf, const float* __restrict__ x_global, const float* __restrict__ w_global,
                 int64_t n, int k, int layout, uint16_t* __restrict__ y) {
  extern __shared__ __align__(16) uint8_t tnq_gemv_smem[];
  uint32_t* xs = reinterpret_cast<uint32_t*>(tnq_gemv_smem);
  float* fx = reinterpret_cast<float*>(tnq_gemv_smem + (size_t)k * 2);
  const int kb = k / 16;
  for (int i = threadIdx.x; i < k / 4; i += kGemvThreads) {  // two bytes = four codes per iteration
    uint32_t lo, hi;
    cvt_e2m1x4_to_f16x2(reinterpret_cast<const uint16_t*>(x)[i], lo, hi);
    xs[2 * i] = lo, xs[2 * i + 1] = hi;
  }
  for (int i = threadIdx.x; i < kb; i += kGemvThreads) fx[i] = e4m3_byte_to_f32(x_sf[scale_index(0, i, kb, layout)]);
  __syncthreads();
  const float g = (x_global ? *x_global : 1.0f) * (w_global ? *w_global : 1.0f);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int steps = k / 1024;  // a lane takes 16 bytes = 32 codes = two blocks per step
  for (int64_t row0 = ((int64_t)blockIdx.x * (kGemvThreads / 32) + warp) * kRowsPerWarp; row0 < n;
       row0 += (int64_t)gridDim.x * kRowsPerCta) {
    float acc[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) acc[r] = 0.0f;
    const int tail_chunks = (k - steps * 1024) / 32;
    for (int s = 0; s <= steps; ++s) {
      const bool last = s == steps;
      if (last && lane >= tail_chunks) break;
      const int kc = s * 1024 + lane * 32;  // this lane's 32 elements (two blocks)
      uint4 wv[kRowsPerWarp];
      uint32_t sb[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const int64_t row = row0 + r < n ? row0 + r : n - 1;
        wv[r] = ldg128(w + (row * k + kc) / 2);
        const uint32_t s0 = w_sf[scale_index(row, kc >> 4, kb, layout)];
        const uint32_t s1 = w_sf[scale_index(row, (kc >> 4) + 1, kb, layout)];
        sb[r] = s0 | (s1 << 8);
      }
      uint4 xv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) xv[q] = *reinterpret_cast<const uint4*>(xs + (kc >> 1) + 4 * q);
      const float f0 = fx[kc >> 4], f1 = fx[(kc >> 4) + 1];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const uint32_t wr[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
        float p[2] = {0.0f, 0.0f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // word q: 8 codes, block q / 2
          uint32_t a0, a1, a2, a3;
          cvt_e2m1x4_to_f16x2(wr[q] & 0xffffu, a0, a1);
          cvt_e2m1x4_to_f16x2(wr[q] >> 16, a2, a3);
          float t = p[q >> 1];
          t = fma2_f16_f32(a0, xv[q].x, t);
          t = fma2_f16_f32(a1, xv[q].y, t);
          t = fma2_f16_f32(a2, xv[q].z, t);
          t = fma2_f16_f32(a3, xv[q].w, t);
          p[q >> 1] = t;
        }
        acc[r] = __fmaf_rn(p[0], __fmul_rn(f0, e4m3_byte_to_f32(sb[r] & 0xffu)), acc[r]);
        acc[r] = __fmaf_rn(p[1], __fmul_rn(f1, e4m3_byte_to_f32(sb[r] >> 8)), acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float v = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && row0 + r < n) y[row0 + r] = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(v, g)));
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <auto Kernel>
static int gemv_grid(int64_t n, int smem) {
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) return -1;
    configured[dev] = 160 * 1024;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, kGemvThreads, smem) != cudaSuccess || per_sm < 1)
    return -1;
  const int64_t want = (n + kRowsPerCta - 1) / kRowsPerCta;
  const int64_t cap = (int64_t)per_sm * sm_count();
  return (int)(want < cap ? want : cap);
}

extern "C" int tnq_mxfp8_gemv(const void* x, const void* w, const void* x_sf, const void* w_sf, int64_t n, int64_t k,
                              int scale_layout, void* y_bf16, tnq_stream_t stream) {
  if (n < 0 || k < 0) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (n == 0) return TNQ_OK;
  if (!x || !w || !x_sf || !w_sf || !y_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 32 != 0) return TNQ_ESHAPE;
  if (k > 65536) return TNQ_EUNSUPPORTED;  // x is kept in shared memory as fp16
  if (!aligned16(x) || !aligned16(w)) return TNQ_EALIGN;
  const int smem = (int)(k * 2 + (k / 32) * 4);
  const int grid = gemv_grid<k_mxfp8_gemv>(n, smem);
  if (grid < 1) return cuda_fail(cudaGetLastError());
  k_mxfp8_gemv<<<grid, kGemvThreads, smem, stream>>>(static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(w),
                                                     static_cast<const uint8_t*>(x_sf), static_cast<const uint8_t*>(w_sf),
                                                     n, (int)k, scale_layout, static_cast<uint16_t*>(y_bf16));
  return check_launch();
}

extern "C" int tnq_nvfp4_gemv(const void* x_packed, const void* w_packed, const void* x_sf, const void* w_sf,
                              const float* x_global, const float* w_global, int64_t n, int64_t k, int scale_layout,
                              void* y_bf16, tnq_stream_t stream) {
  if (n < 0 || k < 0) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (n == 0) return TNQ_OK;
  if (!x_packed || !w_packed || !x_sf || !w_sf || !y_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 32 != 0) return TNQ_ESHAPE;  // a lane takes whole 16-byte chunks of packed codes
  if (k > 65536) return TNQ_EUNSUPPORTED;
  if (!aligned16(x_packed) || !aligned16(w_packed)) return TNQ_EALIGN;
  const int smem = (int)(k * 2 + (k / 16) * 4);
  const int grid = gemv_grid<k_nvfp4_gemv>(n, smem);
  if (grid < 1) return cuda_fail(cudaGetLastError());
  k_nvfp4_gemv<<<grid, kGemvThreads, smem, stream>>>(
      static_cast<const uint8_t*>(x_packed), static_cast<const uint8_t*>(w_packed), static_cast<const uint8_t*>(x_sf),
      static_cast<const uint8_t*>(w_sf), x_global, w_global, n, (int)k, scale_layout, static_cast<uint16_t*>(y_bf16));
  return check_launch();
}
