// Block-scaled M = 1 GEMV on the quantizers' own output formats - the consumer that
// sits directly downstream of the casts:
//   MXFP8 : y[n] = sum_b 2^(sx[b]-127) * 2^(sw[n,b]-127) * sum_{k in b} x[k] * w[n,k]      (32-element blocks)
//   NVFP4 : y[n] = gx * gw * sum_b sx[b] * sw[n,b] * sum_{k in b} x[k] * w[n,k]            (16-element blocks)
// with e4m3 / packed e2m1 payloads, E8M0 / E4M3 block scales in raw row-major or
// swizzled 128x4 storage, fp32 accumulation, bf16 output.
//
// The weight matrix is read once from HBM; x is decoded once per CTA into shared memory as
// fp16 together with its block factors.  A warp owns four output rows at a time - rows i,
// i + 32, i + 64, i + 96 of a 128-row tile, whose swizzled scale bytes for four consecutive
// block columns are 16 contiguous bytes, so one 16-byte copy per lane and step brings every
// scale the lane needs - and walks K in 512-byte steps: lane j takes the j-th 16-byte chunk
// of each row.  The chunks travel through lane-private cp.async rings in shared memory (see
// the kernel), several steps ahead of their use.
//
// The inner loop is sized by instruction issue, not by arithmetic: payload bytes feed the
// hardware converters straight from the fetched words (cvt.rn.f16x2.e2m1x2 / e4m3x2 take a
// byte / half of a 32-bit register without an extract; the source must be a full 32-bit
// word, which is why x is decoded from 32-bit loads too), scale bytes go through cvt as
// well (ue8m0x2 -> bf16x2, e4m3x2 -> f16x2), MXFP8 accumulates exact products in fp32 with
// the mixed-precision FMA (fma.rn.f32.f16), NVFP4 sums the eight products of a half block
// exactly in fp16x2 (|sum| <= 288) before widening, and all per-row address arithmetic is
// one 32 x 32 -> 64-bit multiply-add per copy.  Lanes are folded with shuffles at the end
// of a row group; an output row is the sum of at most two warps' parts added in a fixed order, so a
// result is reproducible for a given shape and GPU (where the work is cut depends on the number of SMs).
#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace tnq {

constexpr int kGemvRows = 4;  // rows per warp and step
// Two shapes of CTA.  The fp16 copy of x (2 bytes per element of K) is per CTA, so a long K leaves room for few
// small CTAs: "narrow" = 128 threads and 4 ring slots per lane (3 steps of copies in flight; four CTAs per SM while
// x is short), "wide" = 512 threads and 3 slots sharing one copy of x (16 warps per SM whatever K is).
struct GemvNarrow {
  static constexpr int kThreads = 128, kStages = 4, kMinCtas = 4;
};
struct GemvWide {
  static constexpr int kThreads = 512, kStages = 3, kMinCtas = 1;
};

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

// ---------------------------------------------------------------- the kernel
// One warp owns one row group at a time.  Every lane keeps a private ring of C::kStages
// slots in shared memory; a slot holds the lane's 16-byte chunk of each of the four rows and
// (swizzled layout) the 16-byte piece with the rows' scale bytes.  Slots are filled with
// cp.async (one commit group per step) C::kStages - 1 steps ahead of consumption, so the
// bytes in flight are bounded by shared memory rather than by registers or by the order in
// which register loads retire, and no lane ever reads a slot another lane wrote: the
// pipeline needs neither a barrier nor a warp synchronisation for the weights.  The scale pieces of a step are copied
// once per warp and read across lanes, with a warp synchronisation on either side (one copy per lane, as the weights,
// moved every swizzled piece two (NVFP4) or eight (MXFP8) times: NVFP4 54.6 -> 50 us).
constexpr int kSlotBytes = (kGemvRows + 1) * 512;  // per warp: 4 rows x 512 B + 512 B of scale pieces

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <bool FP4, class C>
__global__ void __launch_bounds__(C::kThreads, C::kMinCtas)
    k_blockscaled_gemv(const uint8_t* __restrict__ w, const uint8_t* __restrict__ x, const uint8_t* __restrict__ x_sf,
                       const uint8_t* __restrict__ w_sf, const float* __restrict__ x_global,
                       const float* __restrict__ w_global, uint32_t n, uint32_t k, int layout,
                       uint16_t* __restrict__ y) {
  using F = GemvFmt<FP4>;
  constexpr int Q = FP4 ? 4 : 2;  // 16-byte pieces of fp16 x per 16-byte weight chunk
  constexpr int S = C::kStages, kGemvThreads = C::kThreads, kGemvWarps = C::kThreads / 32;
  extern __shared__ __align__(16) uint8_t tnq_gemv_smem[];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ring = smem_u32(tnq_gemv_smem) + warp * (S * kSlotBytes) + lane * 16;  // this lane's ring
  const uint32_t xs = smem_u32(tnq_gemv_smem) + kGemvWarps * S * kSlotBytes;             // x as f16x2 (whole warps)
  const uint32_t fx = xs + gemv_x_bytes<FP4>(k);                                         // x block factors (fp32)
  const uint32_t kb = k / F::kBlock;
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  float g = 1.0f;  // product of the global scales (NVFP4), read in the prologue

  // ---- this warp's work.  Group g owns rows (g / 32) * 128 + (g % 32) + 32 * r, r = 0..3; an item is one 512-byte
  // step of one group.  The CTAs split the groups evenly; inside a CTA the warps split its ITEMS evenly, so a
  // warp's range may begin and end inside a group.  Such a group belongs to two warps (a CTA with at least as many
  // groups as warps gives every warp at least `steps` items, so never to three): the later warp, which meets the
  // group's last steps at the very start of its range, leaves its four partial sums in shared memory; the earlier
  // warp, which reaches the group's first steps at the end of its range, adds them to its own (first part + second
  // part, a fixed order) and stores the rows.  CTAs with fewer groups than warps split whole groups.
  const uint32_t row_bytes = k / F::kElemsPerByte;
  const uint32_t chunks = row_bytes / 16;     // 16-byte chunks per row
  const uint32_t steps = (chunks + 31) / 32;  // 512-byte steps per row (the last may be ragged)
  const uint32_t groups = ((n + 127) / 128) * 32;
  const uint32_t cta_g0 = (uint32_t)((uint64_t)blockIdx.x * groups / gridDim.x);
  const uint32_t cta_ng = (uint32_t)((uint64_t)(blockIdx.x + 1) * groups / gridDim.x) - cta_g0;
  uint32_t item_a, item_b;  // this warp's items within the CTA: item = (group - cta_g0) * steps + step
  if (cta_ng >= (uint32_t)kGemvWarps) {
    item_a = (uint32_t)((uint64_t)warp * cta_ng * steps / kGemvWarps);
    item_b = (uint32_t)((uint64_t)(warp + 1) * cta_ng * steps / kGemvWarps);
  } else {
    item_a = (warp * cta_ng / kGemvWarps) * steps;
    item_b = ((warp + 1) * cta_ng / kGemvWarps) * steps;
  }
  const uint32_t items = item_b - item_a;
  const uint32_t g_begin = cta_g0 + item_a / steps, first_step = item_a % steps;
  const bool starts_inside = first_step != 0;           // the group's earlier steps belong to the previous warp
  __shared__ float s_part[32][kGemvRows];               // [warp]: partial sums of the group a warp starts inside
  __shared__ uint32_t s_part_ready[32];
  if (threadIdx.x < 32) s_part_ready[threadIdx.x] = 0;  // ordered before any use by the barrier behind the prologue
  // bit 2 of `layout` (set by the launcher): raw scales whose rows are 16-byte aligned and whole steps long, so
  // that a step's scale bytes of a row are whole 16-byte pieces and can travel through the rings as well
  const bool rawq = (layout & 4) != 0;
  layout &= 3;
  const bool swz = layout == TNQ_SCALES_SWIZZLED;
  const bool shared_sf = swz || rawq;             // scale pieces copied once per warp and read across lanes
  constexpr uint32_t kSfPieces = FP4 ? 16u : 4u;  // 16-byte scale pieces per step
  const uint32_t kb0 = FP4 ? 2 * lane : lane >> 1;  // first block column of this lane's chunk in step 0
  const uint32_t kb_step = FP4 ? 64 : 16;           // block columns a step advances
  const uint32_t sh = swz ? (kb0 & 3) * 8 : 0;      // where this lane's scale byte(s) sit in a scale word
  const uint32_t ktiles = (kb + 3) >> 2;

  // producer cursor: the group's (clamped) rows and scale base, the lane's chunk and block column
  uint32_t l_group = g_begin, l_step = first_step, l_c = lane + 32 * first_step, l_kb = kb0 + kb_step * first_step, l_item = 0,
           l_slot = 0;
  uint32_t l_row[kGemvRows];
  const uint8_t* l_sf = w_sf;
  auto enter_group = [&]() {
    const uint32_t row0 = (l_group >> 5) * 128 + (l_group & 31);
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) l_row[r] = min(row0 + 32 * r, n - 1);  // rows past the end re-read the last row
    if (swz) l_sf = w_sf + ((uint64_t)(row0 >> 7) * ktiles) * 512 + (row0 & 31) * 16;
  };
  enter_group();
  auto l_row_of = [&](uint32_t r) {
    uint32_t v = l_row[0];
#pragma unroll
    for (int i = 1; i < kGemvRows; ++i) v = r == (uint32_t)i ? l_row[i] : v;
    return v;
  };
  uint4 sv_next = make_uint4(0, 0, 0, 0);  // raw layout: the scale bytes of the step after the one being consumed
  auto load_raw_scales = [&](bool in_range, uint32_t group, uint32_t kbcol, uint32_t c) {
    uint32_t v[kGemvRows] = {0, 0, 0, 0};
    if (in_range && c < chunks) {
      const uint32_t row0 = (group >> 5) * 128 + (group & 31);
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        const uint8_t* sp = w_sf + (uint64_t)min(row0 + 32 * r, n - 1) * kb + kbcol;
        if constexpr (FP4) v[r] = *reinterpret_cast<const uint16_t*>(sp);
        else v[r] = *sp;
      }
    }
    return make_uint4(v[0], v[1], v[2], v[3]);
  };
  auto issue = [&]() {  // one commit group per item, empty when there is nothing to fetch
    if (l_item < items && l_c < chunks) {
      const uint32_t slot = ring + l_slot * kSlotBytes;
      const uint8_t* wp = w + (uint64_t)l_c * 16;
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) cp_async16(slot + r * 512, wp + (uint64_t)l_row[r] * row_bytes);
    }
    // The step's scale bytes: 4 rows x 16 (MXFP8) / 64 (NVFP4) block columns = 4 / 16 pieces of 16 bytes, copied once
    // by the first 4 / 16 lanes, each into its own piece of the slot's scale area, and read by the whole warp.
    if (shared_sf && l_item < items && lane < kSfPieces) {
      const uint32_t step_kb = l_kb - kb0;  // first block column of the step
      const uint32_t dst = ring + l_slot * kSlotBytes + kGemvRows * 512;
      if (swz) {  // piece p: the four rows' bytes for block columns 4 p .. 4 p + 3 of the step
        if ((step_kb >> 2) + lane < ktiles) cp_async16(dst, l_sf + (uint64_t)((step_kb >> 2) + lane) * 512);
      } else {  // raw: lane 4 r + q (NVFP4) / r (MXFP8) copies the q-th 16 bytes of row r
        const uint32_t r = FP4 ? lane >> 2 : lane, q = FP4 ? lane & 3u : 0u;
        cp_async16(dst, w_sf + (uint64_t)l_row_of(r) * kb + step_kb + 16u * q);
      }
    }
    cp_async_commit();
    ++l_item, l_c += 32, l_kb += kb_step;
    if (++l_slot == S) l_slot = 0;
    if (++l_step == steps) {
      l_step = 0, l_c = lane, l_kb = kb0, ++l_group;
      enter_group();
    }
  };

  float acc[kGemvRows];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r) acc[r] = 0.0f;
  uint32_t c_group = g_begin, c_step = first_step, c_c = lane + 32 * first_step, c_kb = kb0 + kb_step * first_step, c_slot = 0;
  uint32_t xi = lane + Q * 32 * first_step;  // uint4 index of this lane's first x piece of the step
  auto consume = [&](const uint4& sv_raw) {
    if (c_c >= chunks) return;
    const uint32_t slot = ring + c_slot * kSlotBytes;
    const uint32_t area = slot - lane * 16 + kGemvRows * 512;  // the warp's scale area of this slot
    // swizzled: the piece with this lane's block column(s): two lanes (NVFP4) / eight lanes (MXFP8) share one
    uint4 sv = swz ? lds128(area + (FP4 ? lane >> 1 : lane >> 3) * 16) : sv_raw;
    if (rawq) {  // row r's step bytes at 64 r (NVFP4, two bytes per lane) / 16 r (MXFP8)
      uint32_t v[kGemvRows];
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        if constexpr (FP4) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v[r]) : "r"(area + 64 * r + 2 * lane));
        else asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v[r]) : "r"(area + 16 * r + (lane >> 1)));
      }
      sv = make_uint4(v[0], v[1], v[2], v[3]);
    }
    const uint32_t sw[kGemvRows] = {sv.x >> sh, sv.y >> sh, sv.z >> sh, sv.w >> sh};
    if constexpr (FP4) {
      uint4 xv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) xv[q] = lds128(xs + (xi + q * 32) * 16);
      const float2 fxv = lds64f(fx + c_c * 8);
      const uint32_t fxh = half2_as_u32(__floats2half2_rn(fxv.x, fxv.y));  // e4m3 values: exact in fp16
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        const uint4 wv = lds128(slot + r * 512);
        const uint32_t wr[4] = {wv.x, wv.y, wv.z, wv.w};
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
        const uint4 wv = lds128(slot + r * 512);
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        cvt_e4m3x4_to_f16x2(wv.x, a0, a1);
        cvt_e4m3x4_to_f16x2(wv.y, a2, a3);
        cvt_e4m3x4_to_f16x2(wv.z, b0, b1);
        cvt_e4m3x4_to_f16x2(wv.w, b2, b3);
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
  auto step_done = [&](bool last_item) {
    c_c += 32, c_kb += kb_step, xi += Q * 32;
    if (++c_slot == S) c_slot = 0;
    const bool group_end = ++c_step == steps;
    if (group_end || last_item) {  // end of the group, or of this warp's part of it: fold the lanes, lane r takes row r
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) {
        float v = acc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[r] = v;
      }
      float v = acc[0];
#pragma unroll
      for (int r = 1; r < kGemvRows; ++r) v = lane == r ? acc[r] : v;
      if (starts_inside && c_group == g_begin) {
        // the group's later steps, met first: leave the partial sums for the previous warp
        if (lane < kGemvRows) s_part[warp][lane] = v;
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          *reinterpret_cast<volatile uint32_t*>(&s_part_ready[warp]) = 1u;
        }
      } else {
        if (!group_end) {  // this warp's range ends inside the group: the next warp left the rest long ago
          for (uint32_t spin = 0; spin < (1u << 26); ++spin)
            if (*reinterpret_cast<volatile uint32_t*>(&s_part_ready[warp + 1]) != 0u) break;
          __threadfence_block();
          if (lane < kGemvRows) v = __fadd_rn(v, *reinterpret_cast<volatile float*>(&s_part[warp + 1][lane]));
        }
        const uint32_t row = (c_group >> 5) * 128 + (c_group & 31) + 32 * lane;
        if (lane < kGemvRows && row < n) y[row] = __bfloat16_as_ushort(__float2bfloat16_rn(FP4 ? __fmul_rn(v, g) : v));
      }
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) acc[r] = 0.0f;
      c_step = 0, c_c = lane, c_kb = kb0, xi = lane, ++c_group;
    }
  };

  // ---- the pipeline: the first weight copies leave before x is decoded, so they fly during the prologue
#pragma unroll
  for (int d = 0; d < S - 1; ++d) issue();

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
  if constexpr (FP4) g = (x_global ? *x_global : 1.0f) * (w_global ? *w_global : 1.0f);

  uint4 sv_cur = make_uint4(0, 0, 0, 0);
  if (!shared_sf) sv_cur = load_raw_scales(items > 0, c_group, c_kb, c_c);
  for (uint32_t it = 0; it < items; ++it) {
    if (shared_sf) __syncwarp();  // every lane has read the scale pieces of the slot that is refilled next
    issue();  // refills the slot consumed in the previous iteration
    if (!shared_sf) {  // raw scale bytes that cannot go through 16-byte copies: one step ahead in registers
      uint32_t ng = c_group, nk = c_kb + kb_step, nc = c_c + 32;
      if (c_step + 1 == steps) ng = c_group + 1, nk = kb0, nc = lane;
      sv_next = load_raw_scales(it + 1 < items, ng, nk, nc);
    }
    cp_async_wait<S - 1>();  // everything but the S - 1 newest groups has landed: this item's slot is ready
    if (shared_sf) __syncwarp();   // ... for every lane: the scale pieces are read across lanes
    consume(sv_cur);
    step_done(it + 1 == items);
    sv_cur = sv_next;
  }
  cp_async_wait<0>();
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <bool FP4, class C>
static int launch_gemv_shape(const void* x, const void* w, const void* x_sf, const void* w_sf, const float* xg, const float* wg,
                             int64_t n, int64_t k, int layout, void* y, cudaStream_t stream) {
  using F = GemvFmt<FP4>;
  constexpr int kWarps = C::kThreads / 32;
  const int kb = (int)(k / F::kBlock);
  const int smem = kWarps * C::kStages * kSlotBytes + gemv_x_bytes<FP4>((int)k) + ((kb + 3) & ~3) * 4;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(k_blockscaled_gemv<FP4, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) !=
        cudaSuccess)
      return cuda_fail(cudaGetLastError());
    configured[dev] = 1;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_blockscaled_gemv<FP4, C>, C::kThreads, smem) !=
          cudaSuccess ||
      per_sm < 1)
    return TNQ_EUNSUPPORTED;
  const int64_t groups = ((n + 127) / 128) * 32;
  const int64_t want = (groups + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)per_sm * sm_count();
  const int grid = (int)(want < cap ? want : cap);
  // raw scales ride the copy rings when every row's scale bytes of a step are whole, aligned 16-byte pieces:
  // rows of whole 512-byte steps (K % 512 == 0 for MXFP8, % 1024 for NVFP4) and a 16-byte aligned buffer
  const int64_t chunks = k / F::kElemsPerByte / 16;
  const bool rawq = layout == TNQ_SCALES_RAW && chunks % 32 == 0 && kb % 16 == 0 && aligned16(w_sf);
  return launch_chained(k_blockscaled_gemv<FP4, C>, dim3(grid), dim3(C::kThreads), smem, stream, static_cast<const uint8_t*>(w),
                        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(x_sf), static_cast<const uint8_t*>(w_sf), xg,
                        wg, (uint32_t)n, (uint32_t)k, layout | (rawq ? 4 : 0), static_cast<uint16_t*>(y));
}

// shape: 0 = wide where it fits and the matrix has rows enough (default), 1 = narrow, 2 = wide (narrow if it does not fit)
static std::atomic<int> g_gemv_shape{0};
extern "C" int tnq_gemv_set_shape(int shape) {
  if (shape < 0 || shape > 2) return TNQ_EINVAL;
  g_gemv_shape.store(shape, std::memory_order_relaxed);
  return TNQ_OK;
}
// Measured on 256 MiB of weights, two matrices in turn (us, narrow / wide): MXFP8 K = 2048 45.9 / 45.0, 4096 47.4 /
// 44.7, 8192 46.6 / 44.6, 16384 48.5 / 45.3, 32768 57.1 / 49.3; NVFP4 K = 2048 58.8 / 55.0, 8192 57.4 / 54.3, 16384
// 65.6 / 56.1, 32768 67.5 / 57.1.  The wide shape keeps sixteen warps per SM whatever K is; it is the default and the
// narrow one takes over where sixteen rings and the copy of x no longer fit (K = 65536) and for matrices with too
// few rows to give most SMs a wide CTA of their own (MXFP8 4096 x 4096: 6.4 / 8.8 us, 1024 x 8192: 8.0 / 13.8).  Before the warps of a CTA
// split its items at step granularity the wide shape lost to the uneven split of whole row groups (3.5 groups per
// warp at N = 32768: MXFP8 K = 8192 48.7 / 48.1, NVFP4 K = 16384 59.6 / 63.5).
template <bool FP4>
static int launch_gemv(const void* x, const void* w, const void* x_sf, const void* w_sf, const float* xg, const float* wg,
                       int64_t n, int64_t k, int layout, void* y, cudaStream_t stream) {
  const int shape = g_gemv_shape.load(std::memory_order_relaxed);
  const int64_t groups = ((n + 127) / 128) * 32;  // wide CTAs wanted: one per sixteen row groups
  const bool wide = shape == 2 || (shape == 0 && groups * 20 >= (int64_t)sm_count() * 16 * 17);  // >= 0.85 per SM
  if (wide) {
    const int rc = launch_gemv_shape<FP4, GemvWide>(x, w, x_sf, w_sf, xg, wg, n, k, layout, y, stream);
    if (rc != TNQ_EUNSUPPORTED) return rc;  // x too long for sixteen rings beside it: the narrow shape
  }
  return launch_gemv_shape<FP4, GemvNarrow>(x, w, x_sf, w_sf, xg, wg, n, k, layout, y, stream);
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
