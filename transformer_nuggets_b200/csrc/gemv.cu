// Block-scaled M = 1 GEMV on the quantizers' own output formats - the consumer that
// sits directly downstream of the casts:
//   MXFP8 : y[n] = sum_b 2^(sx[b]-127) * 2^(sw[n,b]-127) * sum_{k in b} x[k] * w[n,k]      (32-element blocks)
//   NVFP4 : y[n] = gx * gw * sum_b sx[b] * sw[n,b] * sum_{k in b} x[k] * w[n,k]            (16-element blocks)
// with e4m3 / packed e2m1 payloads, E8M0 / E4M3 block scales in raw row-major or
// swizzled 128x4 storage, fp32 accumulation, bf16 output.
//
// The weight matrix is read once from HBM; x is decoded once per CTA into shared memory as
// fp16 together with its block factors.  A team of T warps owns four output rows at a time
// - rows i, i + 32, i + 64, i + 96 of a 128-row tile, whose swizzled scale bytes for four
// consecutive block columns are 16 contiguous bytes, so one 16-byte load per lane and step
// brings every scale the lane needs - and walks K together: in one step lane j of the team
// fetches the j-th 16-byte chunk of each row.  The next step's loads are issued into a
// second register buffer before the current one is consumed.
//
// The inner loop is sized by instruction issue, not by arithmetic: payload bytes feed the
// hardware converters straight from the loaded words (cvt.rn.f16x2.e2m1x2 / e4m3x2 take a
// byte / half of a register without an extract), scale bytes go through cvt as well
// (ue8m0x2 -> bf16x2, e4m3x2 -> f16x2), MXFP8 accumulates exact products in fp32 with the
// mixed-precision FMA (fma.rn.f32.f16), NVFP4 sums the eight products of a half block
// exactly in fp16x2 (|sum| <= 288) before widening, and all per-row address arithmetic is
// one 32 x 32 -> 64-bit multiply-add per load.  Lanes are folded with shuffles and the
// team's warps through shared memory in a fixed order, so results do not depend on the grid.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace tnq {

#ifndef TNQ_GEMV_THREADS
#define TNQ_GEMV_THREADS 128
#endif
#ifndef TNQ_GEMV_MIN_CTAS
#define TNQ_GEMV_MIN_CTAS 4
#endif
constexpr int kGemvThreads = TNQ_GEMV_THREADS;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvRows = 4;  // rows per team and step

// 2^(byte - 127) as fp32; byte 0 -> 2^-127 (subnormal), byte 255 -> NaN
__device__ __forceinline__ float e8m0_to_f32(uint32_t byte) {
  uint32_t r;
  asm("cvt.rn.bf16x2.ue8m0x2 %0, %1;" : "=r"(r) : "h"((uint16_t)byte));
  return __uint_as_float(r << 16);
}
__device__ __forceinline__ float e4m3_byte_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)byte));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
__device__ __forceinline__ __half2 u32_as_half2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t half2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((uint16_t)two_bytes));
  return r;
}
// one 32-bit word of four e4m3 bytes -> two f16x2 words
__device__ __forceinline__ void cvt_e4m3x4_to_f16x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 h0, h1;\n\tmov.b32 {h0, h1}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, h0;\n\tcvt.rn.f16x2.e4m3x2 %1, h1;\n\t}"
      : "=&r"(lo), "=&r"(hi)
      : "r"(w));
}
// one 32-bit word of eight packed e2m1 codes -> four f16x2 words (codes 0,1 / 2,3 / 4,5 / 6,7)
__device__ __forceinline__ void cvt_e2m1x8_to_f16x2(uint32_t w, uint32_t (&o)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\tcvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=&r"(o[0]), "=&r"(o[1]), "=&r"(o[2]), "=&r"(o[3])  // early clobber: never the input's register
      : "r"(w));
}
// c + a.lo * b.lo + a.hi * b.hi with both products exact in fp32 (a, b: f16x2)
__device__ __forceinline__ float fma2_f16_f32(uint32_t a, uint32_t b, float c) {
  float d;
  asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t.reg .f32 t;\n\tmov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
      "fma.rn.f32.f16 t, al, bl, %3;\n\tfma.rn.f32.f16 %0, ah, bh, t;\n\t}"
      : "=&f"(d)
      : "r"(a), "r"(b), "f"(c));
  return d;
}
// (a.lo * b.lo, a.hi * b.hi) as two fp32 values, both exact (a, b: f16x2)
__device__ __forceinline__ void mul2_f16_f32(uint32_t a, uint32_t b, float& lo, float& hi) {
  asm("{\n\t.reg .b16 al, ah, bl, bh;\n\tmov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
      "fma.rn.f32.f16 %0, al, bl, 0f00000000;\n\tfma.rn.f32.f16 %1, ah, bh, 0f00000000;\n\t}"
      : "=&f"(lo), "=&f"(hi)
      : "r"(a), "r"(b));
}

// The fp16 copy of x is written and read with explicit shared-space instructions: the
// writer stores 32-bit words, the readers fetch 16-byte pieces, and neither goes through a
// typed C++ pointer that the compiler could reason about separately.
__device__ __forceinline__ void sts32(uint32_t saddr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t saddr, uint32_t lo, uint32_t hi) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(saddr), "r"(lo), "r"(hi) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float2 lds64f(uint32_t saddr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(saddr));
  return v;
}
__device__ __forceinline__ float lds32f(uint32_t saddr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
  return v;
}

// Byte offset of block-scale column kb within one scale row, and the row's base offset:
// raw row-major [rows, W] or the swizzled 128x4 layout (a row's bytes sit in groups of
// four, 512 bytes apart).
__device__ __forceinline__ int sf_col_offset(int kb, int layout) {
  return layout == TNQ_SCALES_SWIZZLED ? ((kb >> 2) << 9) + (kb & 3) : kb;
}
__device__ __forceinline__ int64_t sf_row_base(int64_t r, int64_t w, int layout) {
  return layout == TNQ_SCALES_SWIZZLED ? (r >> 7) * ((w + 3) / 4) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 : r * w;
}

template <bool FP4>
struct GemvFmt;
template <>
struct GemvFmt<false> {  // MXFP8: a lane's 16-byte chunk is 16 elements (half a block)
  static constexpr int kElemsPerByte = 1, kBlock = 32;
};
template <>
struct GemvFmt<true> {  // NVFP4: a lane's 16-byte chunk is 32 elements (two blocks)
  static constexpr int kElemsPerByte = 2, kBlock = 16;
};

// Bytes of the fp16 copy of x in shared memory: whole warps of 16-byte chunks.
template <bool FP4>
__host__ __device__ constexpr int gemv_x_bytes(int k) {
  const int chunks = k / GemvFmt<FP4>::kElemsPerByte / 16;
  return ((chunks + 31) / 32) * 32 * (FP4 ? 64 : 32);
}

// One step of one lane: a 16-byte weight chunk of each row and the rows' scale bytes
// (component r of `sv`: row r's scale byte(s) for this chunk at bit `sh`).
struct GemvLoads {
  uint4 w[kGemvRows];
  uint4 sv;
};

template <bool FP4, int T>
__global__ void __launch_bounds__(kGemvThreads, TNQ_GEMV_MIN_CTAS)
    k_blockscaled_gemv(const uint8_t* __restrict__ w, const uint8_t* __restrict__ x, const uint8_t* __restrict__ x_sf,
                       const uint8_t* __restrict__ w_sf, const float* __restrict__ x_global,
                       const float* __restrict__ w_global, uint32_t n, uint32_t k, int layout,
                       uint16_t* __restrict__ y) {
  using F = GemvFmt<FP4>;
  constexpr int kTeams = kGemvWarps / T;
  constexpr int Q = FP4 ? 4 : 2;  // 16-byte pieces of fp16 x per 16-byte weight chunk
  extern __shared__ __align__(16) uint8_t tnq_gemv_smem[];
  const uint32_t xs = smem_u32(tnq_gemv_smem);       // x as f16x2 (padded to whole warps), shared-space address
  const uint32_t fx = xs + gemv_x_bytes<FP4>(k);     // x block factors (fp32), shared-space address
  const uint32_t kb = k / F::kBlock;
  float* partial = reinterpret_cast<float*>(tnq_gemv_smem + gemv_x_bytes<FP4>(k)) + ((kb + 3) & ~3u);  // [2][warps][rows]
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t team = warp / T, tlane = (warp % T) * 32 + lane;

  // ---- prologue: decode x once per CTA.  Piece q of chunk c is stored at uint4 index
  // (c / 32) * 32 * Q + q * 32 + (c % 32), so that the 32 lanes of a warp read consecutive
  // 16-byte pieces (no bank conflicts).
  if constexpr (FP4) {
    for (uint32_t i = threadIdx.x; i < k / 8; i += kGemvThreads) {  // one word = 8 codes = one 16-byte piece
      uint32_t o[4];
      cvt_e2m1x8_to_f16x2(reinterpret_cast<const uint32_t*>(x)[i], o);
      const uint32_t c = i >> 2, q = i & 3;
      sts128(xs + (((c >> 5) * Q + q) * 32 + (c & 31)) * 16, o[0], o[1], o[2], o[3]);
    }
    for (uint32_t i = threadIdx.x; i < kb; i += kGemvThreads)
      sts32(fx + i * 4, __float_as_uint(e4m3_byte_to_f32(x_sf[sf_row_base(0, kb, layout) + sf_col_offset(i, layout)])));
  } else {
    for (uint32_t i = threadIdx.x; i < k / 4; i += kGemvThreads) {  // one word = 4 bytes = half a piece
      uint32_t lo, hi;
      cvt_e4m3x4_to_f16x2(reinterpret_cast<const uint32_t*>(x)[i], lo, hi);
      const uint32_t c = i >> 2, q = (i >> 1) & 1, e = (i & 1) * 2;
      sts64(xs + ((((c >> 5) * Q + q) * 32 + (c & 31)) * 4 + e) * 4, lo, hi);
    }
    for (uint32_t i = threadIdx.x; i < kb; i += kGemvThreads)
      sts32(fx + i * 4, __float_as_uint(e8m0_to_f32(x_sf[sf_row_base(0, kb, layout) + sf_col_offset(i, layout)])));
  }
  __syncthreads();
  float g = 1.0f;
  if constexpr (FP4) g = (x_global ? *x_global : 1.0f) * (w_global ? *w_global : 1.0f);

  // ---- this CTA's work: a balanced contiguous range of row groups, kTeams groups per round;
  // every team runs the same number of rounds so that the CTA-wide barrier stays uniform.
  // Group g owns rows (g / 32) * 128 + (g % 32) + 32 * r, r = 0..3.
  const uint32_t row_bytes = k / F::kElemsPerByte;
  const uint32_t chunks = row_bytes / 16;                  // 16-byte chunks per row
  const uint32_t steps = (chunks + T * 32 - 1) / (T * 32);  // steps per round (the last may be ragged)
  const uint32_t groups = ((n + 127) / 128) * 32;
  const uint32_t g_begin = (uint32_t)((uint64_t)blockIdx.x * groups / gridDim.x);
  const uint32_t g_end = (uint32_t)((uint64_t)(blockIdx.x + 1) * groups / gridDim.x);
  const uint32_t rounds = (g_end - g_begin + kTeams - 1) / kTeams;
  const uint32_t items = rounds * steps;
  const bool swz = layout == TNQ_SCALES_SWIZZLED;
  const uint32_t kb0 = FP4 ? 2 * tlane : tlane >> 1;  // first block column of this lane's chunk in step 0
  const uint32_t kb_step = FP4 ? 2 * T * 32 : T * 16;  // block columns a step advances
  const uint32_t sh = swz ? (kb0 & 3) * 8 : 0;          // where this lane's scale byte(s) sit in a word of `sv`
  const uint32_t ktiles = (kb + 3) >> 2;

  // load cursor: the group's (clamped) rows and scale base, the lane's chunk and block column
  uint32_t l_group = g_begin + team, l_step = 0, l_c = tlane, l_kb = kb0, l_item = 0;
  uint32_t l_row[kGemvRows];
  const uint8_t* l_sf = w_sf;
  auto enter_group = [&]() {
    const uint32_t row0 = (l_group >> 5) * 128 + (l_group & 31);
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) l_row[r] = min(row0 + 32 * r, n - 1);  // rows past the end re-read the last row
    if (swz) l_sf = w_sf + ((uint64_t)(row0 >> 7) * ktiles) * 512 + (row0 & 31) * 16;
  };
  enter_group();
  auto load = [&](GemvLoads& b) {
    if (l_group < g_end && l_c < chunks) {
      const uint8_t* wp = w + (uint64_t)l_c * 16;
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) b.w[r] = ldg128(wp + (uint64_t)l_row[r] * row_bytes);
      if (swz) {  // one 16-byte piece: word r = row r's four block columns
        b.sv = *reinterpret_cast<const uint4*>(l_sf + (uint64_t)(l_kb >> 2) * 512);
      } else {
        const uint8_t* sp = w_sf + l_kb;
        uint32_t v[kGemvRows];
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
          if constexpr (FP4) v[r] = *reinterpret_cast<const uint16_t*>(sp + (uint64_t)l_row[r] * kb);
          else v[r] = sp[(uint64_t)l_row[r] * kb];
        }
        b.sv = make_uint4(v[0], v[1], v[2], v[3]);
      }
    }
    ++l_item, l_c += T * 32, l_kb += kb_step;
    if (++l_step == steps) {
      l_step = 0, l_c = tlane, l_kb = kb0, l_group += kTeams;
      enter_group();
    }
  };

  float acc[kGemvRows];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r) acc[r] = 0.0f;
  uint32_t c_group = g_begin + team, c_step = 0, c_c = tlane;
  uint32_t xi = (tlane >> 5) * Q * 32 + lane;  // uint4 index of this lane's first x piece
  auto consume = [&](const GemvLoads& b) {
    if (c_group >= g_end || c_c >= chunks) return;
    const uint32_t sw[kGemvRows] = {b.sv.x >> sh, b.sv.y >> sh, b.sv.z >> sh, b.sv.w >> sh};
    if constexpr (FP4) {
      uint4 xv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) xv[q] = lds128(xs + (xi + q * 32) * 16);
      const float2 fxv = lds64f(fx + c_c * 8);
      const uint32_t fxh = half2_as_u32(__floats2half2_rn(fxv.x, fxv.y));  // e4m3 values: exact in fp16
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        const uint32_t wr[4] = {b.w[r].x, b.w[r].y, b.w[r].z, b.w[r].w};
        float s0, s1;  // x factor * row scale of the two blocks, exact
        mul2_f16_f32(cvt_e4m3x2_to_f16x2(sw[r]), fxh, s0, s1);
        float p[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // block h: words 2h, 2h+1; each f16x2 half sums 8 exact products
          uint32_t a[4], c[4];
          cvt_e2m1x8_to_f16x2(wr[2 * h], a);
          cvt_e2m1x8_to_f16x2(wr[2 * h + 1], c);
          __half2 t = __hmul2(u32_as_half2(a[0]), u32_as_half2(xv[2 * h].x));
          __half2 u = __hmul2(u32_as_half2(c[0]), u32_as_half2(xv[2 * h + 1].x));
          t = __hfma2(u32_as_half2(a[1]), u32_as_half2(xv[2 * h].y), t);
          u = __hfma2(u32_as_half2(c[1]), u32_as_half2(xv[2 * h + 1].y), u);
          t = __hfma2(u32_as_half2(a[2]), u32_as_half2(xv[2 * h].z), t);
          u = __hfma2(u32_as_half2(c[2]), u32_as_half2(xv[2 * h + 1].z), u);
          t = __hfma2(u32_as_half2(a[3]), u32_as_half2(xv[2 * h].w), t);
          u = __hfma2(u32_as_half2(c[3]), u32_as_half2(xv[2 * h + 1].w), u);
          t = __hadd2(t, u);  // each half: eight products, |sum| <= 288, exact in fp16
          p[h] = fma2_f16_f32(half2_as_u32(t), 0x3c003c00u, 0.0f);  // t.lo + t.hi in fp32
        }
        acc[r] = __fmaf_rn(p[0], s0, acc[r]);
        acc[r] = __fmaf_rn(p[1], s1, acc[r]);
      }
    } else {
      const uint4 xa = lds128(xs + xi * 16), xb = lds128(xs + (xi + 32) * 16);
      const float f = lds32f(fx + (c_c >> 1) * 4);
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        cvt_e4m3x4_to_f16x2(b.w[r].x, a0, a1);
        cvt_e4m3x4_to_f16x2(b.w[r].y, a2, a3);
        cvt_e4m3x4_to_f16x2(b.w[r].z, b0, b1);
        cvt_e4m3x4_to_f16x2(b.w[r].w, b2, b3);
        float p = 0.0f, q = 0.0f;  // two chains per row
        p = fma2_f16_f32(a0, xa.x, p);
        q = fma2_f16_f32(b0, xb.x, q);
        p = fma2_f16_f32(a1, xa.y, p);
        q = fma2_f16_f32(b1, xb.y, q);
        p = fma2_f16_f32(a2, xa.z, p);
        q = fma2_f16_f32(b2, xb.z, q);
        p = fma2_f16_f32(a3, xa.w, p);
        q = fma2_f16_f32(b3, xb.w, q);
        acc[r] = __fmaf_rn(p + q, __fmul_rn(f, e8m0_to_f32(sw[r] & 0xffu)), acc[r]);
      }
    }
  };
  uint32_t par = 0;
  auto finish = [&]() {  // end of a round: fold lanes, then the team's warps, store
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      float v = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r] = v;
    }
    const uint32_t row = (c_group >> 5) * 128 + (c_group & 31) + 32 * lane;  // lane r stores row r
    const bool store = lane < kGemvRows && c_group < g_end && row < n;
    if constexpr (T == 1) {
      if (store) {
        float v = acc[0];
#pragma unroll
        for (int r = 1; r < kGemvRows; ++r) v = lane == r ? acc[r] : v;
        y[row] = __bfloat16_as_ushort(__float2bfloat16_rn(FP4 ? __fmul_rn(v, g) : v));
      }
    } else {
      float* mine = partial + (par * kGemvWarps + warp) * kGemvRows;
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) mine[r] = acc[r];
      }
      __syncthreads();
      if (warp % T == 0 && store) {
        float v = 0.0f;
#pragma unroll
        for (int j = 0; j < T; ++j) v += partial[(par * kGemvWarps + warp + j) * kGemvRows + lane];
        y[row] = __bfloat16_as_ushort(__float2bfloat16_rn(FP4 ? __fmul_rn(v, g) : v));
      }
      par ^= 1u;  // the other buffer is free again once every warp has passed the next barrier
    }
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) acc[r] = 0.0f;
  };
  auto step_done = [&]() {
    c_c += T * 32, xi += T * Q * 32;
    if (++c_step == steps) {
      finish();
      c_step = 0, c_c = tlane, xi = (tlane >> 5) * Q * 32 + lane, c_group += kTeams;
    }
  };

  // ---- the pipeline: the next step's loads are in flight while this one is consumed
  GemvLoads buf[2];
  if (items > 0) load(buf[0]);
  for (uint32_t it = 0; it < items; it += 2) {
    if (l_item < items) load(buf[1]);
    consume(buf[0]);
    step_done();
    if (it + 1 < items) {
      if (l_item < items) load(buf[0]);
      consume(buf[1]);
      step_done();
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <bool FP4, int T>
static int launch_gemv_t(const void* x, const void* w, const void* x_sf, const void* w_sf, const float* xg,
                         const float* wg, int64_t n, int64_t k, int layout, void* y, cudaStream_t stream) {
  using F = GemvFmt<FP4>;
  constexpr int kTeams = kGemvWarps / T;
  const int kb = (int)(k / F::kBlock);
  const int smem = gemv_x_bytes<FP4>((int)k) + ((kb + 3) & ~3) * 4 + 2 * kGemvWarps * kGemvRows * 4;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(k_blockscaled_gemv<FP4, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) !=
        cudaSuccess)
      return cuda_fail(cudaGetLastError());
    configured[dev] = 1;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_blockscaled_gemv<FP4, T>, kGemvThreads, smem) !=
          cudaSuccess ||
      per_sm < 1)
    return TNQ_EUNSUPPORTED;
  const int64_t groups = ((n + 127) / 128) * 32;
  const int64_t want = (groups + kTeams - 1) / kTeams;
  const int64_t cap = (int64_t)per_sm * sm_count();
  const int grid = (int)(want < cap ? want : cap);
  k_blockscaled_gemv<FP4, T><<<grid, kGemvThreads, smem, stream>>>(
      static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(x_sf),
      static_cast<const uint8_t*>(w_sf), xg, wg, (uint32_t)n, (uint32_t)k, layout, static_cast<uint16_t*>(y));
  return check_launch();
}

// Team size.  One warp per row group keeps every warp independent (no CTA barrier) and is
// the fastest once a row spans at least one 512-byte step; shorter rows share a warp's lanes
// poorly either way.
template <bool FP4>
static int launch_gemv(const void* x, const void* w, const void* x_sf, const void* w_sf, const float* xg, const float* wg,
                       int64_t n, int64_t k, int layout, void* y, cudaStream_t stream) {
#ifdef TNQ_GEMV_FORCE_T
  return launch_gemv_t<FP4, TNQ_GEMV_FORCE_T>(x, w, x_sf, w_sf, xg, wg, n, k, layout, y, stream);
#else
  return launch_gemv_t<FP4, 1>(x, w, x_sf, w_sf, xg, wg, n, k, layout, y, stream);
#endif
}

extern "C" int tnq_mxfp8_gemv(const void* x, const void* w, const void* x_sf, const void* w_sf, int64_t n, int64_t k,
                              int scale_layout, void* y_bf16, tnq_stream_t stream) {
  if (n < 0 || k < 0) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (n == 0) return TNQ_OK;
  if (!x || !w || !x_sf || !w_sf || !y_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 32 != 0) return TNQ_ESHAPE;
  if (k > 65536 || n > 0x7fffffff) return TNQ_EUNSUPPORTED;  // x is kept in shared memory as fp16
  if (!aligned16(x) || !aligned16(w)) return TNQ_EALIGN;
  if (scale_layout == TNQ_SCALES_SWIZZLED && !aligned16(w_sf)) return TNQ_EALIGN;
  return launch_gemv<false>(x, w, x_sf, w_sf, nullptr, nullptr, n, k, scale_layout, y_bf16, stream);
}

extern "C" int tnq_nvfp4_gemv(const void* x_packed, const void* w_packed, const void* x_sf, const void* w_sf,
                              const float* x_global, const float* w_global, int64_t n, int64_t k, int scale_layout,
                              void* y_bf16, tnq_stream_t stream) {
  if (n < 0 || k < 0) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (n == 0) return TNQ_OK;
  if (!x_packed || !w_packed || !x_sf || !w_sf || !y_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 32 != 0) return TNQ_ESHAPE;  // a lane takes whole 16-byte chunks of packed codes
  if (k > 65536 || n > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (!aligned16(x_packed) || !aligned16(w_packed)) return TNQ_EALIGN;
  if (scale_layout == TNQ_SCALES_SWIZZLED && !aligned16(w_sf)) return TNQ_EALIGN;
  return launch_gemv<true>(x_packed, w_packed, x_sf, w_sf, x_global, w_global, n, k, scale_layout, y_bf16, stream);
}
