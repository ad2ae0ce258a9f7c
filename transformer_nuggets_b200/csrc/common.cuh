// Device helpers shared by the cast kernels (sm_100a only).
//
// Arithmetic contract: every product / quotient is a single IEEE fp32 operation
// (__fmul_rn / __fdiv_rn, never contracted into an FMA, no flush-to-zero), the
// fp8 / fp4 conversion is the hardware round-to-nearest-even `cvt`, and |x| maxima
// are taken on the integer view of the input (same order as the float order for
// every non-NaN value; any NaN compares above infinity and therefore wins).
#pragma once

#include <cstdint>
#include <type_traits>
#include <utility>

#include <cuda_runtime.h>

#include "../../include/tnq.h"

namespace tnq {

constexpr float kAmaxEps = 1e-12f;

// ------------------------------------------------------------------ loads / stores
struct alignas(32) Vec32B {
  uint32_t w[8];
};

__device__ __forceinline__ uint4 ldg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 256-bit global load (one instruction per 32 bytes; new with sm_100).
__device__ __forceinline__ Vec32B ldg256(const void* p) {
  Vec32B v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                 "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
// L2 eviction-priority policies and loads / stores that carry one
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ Vec32B ldg256_hint(const void* p, uint64_t policy) {
  Vec32B v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8], %9;"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                 "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ void stg128_hint(void* p, uint4 v, uint64_t policy) {
  asm volatile("st.global.L1::no_allocate.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void stg64_hint(void* p, uint2 v, uint64_t policy) {
  asm volatile("st.global.L1::no_allocate.L2::cache_hint.v2.u32 [%0], {%1,%2}, %3;" ::"l"(p), "r"(v.x), "r"(v.y),
               "l"(policy)
               : "memory");
}
__device__ __forceinline__ void stg128(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// 256-bit global store (sm_100)
__device__ __forceinline__ void stg256(void* p, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t w4,
                                       uint32_t w5, uint32_t w6, uint32_t w7) {
  asm volatile("st.global.L1::no_allocate.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w0), "r"(w1),
               "r"(w2), "r"(w3), "r"(w4), "r"(w5), "r"(w6), "r"(w7)
               : "memory");
}
// shared-memory accesses by 32-bit shared-space address (no generic-pointer arithmetic)
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
  return v;
}
// the same with a compile-time byte offset folded into the instruction
template <int OFF>
__device__ __forceinline__ uint4 lds128_at(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(saddr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32_at(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(saddr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ void sts8_at(uint32_t saddr, uint32_t v) {
  asm volatile("st.shared.u8 [%0+%1], %2;" ::"r"(saddr), "n"(OFF), "r"(v) : "memory");
}
// compile-time loop: f(std::integral_constant<int, 0>{}), ..., f(std::integral_constant<int, N-1>{})
template <class F, int... Is>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, Is...>) {
  (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(static_cast<F&&>(f), std::make_integer_sequence<int, N>{});
}
// named barrier ID (1..15) among COUNT threads (a multiple of 32); compile-time operands so
// that the kernel reserves only the barriers it names
template <int ID, int COUNT>
__device__ __forceinline__ void named_barrier() {
  asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory");
}
__device__ __forceinline__ void sts8(uint32_t saddr, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}
__device__ __forceinline__ void stg64(void* p, uint2 v) {
  asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void stg32(void* p, uint32_t v) {
  asm volatile("st.global.L1::no_allocate.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------------------ bf16 pairs
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// max of |.| over packed bf16 pairs, on the 15-bit magnitude
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t m, uint32_t w) {
  return __vmaxu2(m, w & 0x7fff7fffu);
}
// The same in ONE instruction per word: max of the magnitudes of two bf16 pairs; the sign bits of the
// result are meaningless (mask them off at the end) and any NaN makes the half the canonical NaN
// 0x7fff, which is above infinity in the integer order used to fold the result.
__device__ __forceinline__ uint32_t absmax_bf16x2_1op(uint32_t m, uint32_t w) {
  uint32_t r;
  asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(m), "r"(w));
  return r;
}
// ... and for one fp32 (bit pattern in and out)
__device__ __forceinline__ uint32_t absmax_f32_1op(uint32_t m, uint32_t w) {
  float r;
  asm("max.NaN.xorsign.abs.f32 %0, %1, %2;" : "=f"(r) : "f"(__uint_as_float(m)), "f"(__uint_as_float(w)));
  return __float_as_uint(r);
}
__device__ __forceinline__ uint32_t fold_u16x2(uint32_t m) { return max(m & 0xffffu, m >> 16); }
__device__ __forceinline__ float bf16bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// ------------------------------------------------------------------ fp8 conversion
template <int OUT>
struct Fp8Traits;
template <>
struct Fp8Traits<TNQ_FP8_E4M3> {
  static constexpr float kMax = 448.0f;
  static constexpr uint32_t kNanAdd = 0x01010101u;  // (b & 0x7f) == 0x7f  <=> NaN
  static constexpr uint32_t kOverflowByte = 0x7f;   // non-saturating overflow -> NaN
};
template <>
struct Fp8Traits<TNQ_FP8_E5M2> {
  static constexpr float kMax = 57344.0f;
  static constexpr uint32_t kNanAdd = 0x04040404u;  // (b & 0x7f) >= 0x7c  <=> inf / NaN
  static constexpr uint32_t kOverflowByte = 0x7c;   // non-saturating overflow -> inf
};

template <int OUT>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi) {
  uint16_t r;
  if constexpr (OUT == TNQ_FP8_E4M3) {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  }
  return r;
}
// four floats -> four fp8 bytes (a lowest); the two 16-bit halves are joined with a
// register-pair move so that the second conversion can merge into the first's register
template <int OUT>
__device__ __forceinline__ uint32_t cvt_fp8x4(float a, float b, float c, float d) {
  uint32_t r;
  if constexpr (OUT == TNQ_FP8_E4M3) {
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
  } else {
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e5m2x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e5m2x2.f32 hi, %4, %3;\n\tmov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
  }
  return r;
}

// Exact scalar cast with the corner cases of the CPU path the results are checked
// against: NaN keeps a sign (that of the scale if the scale is NaN, else that of a NaN x,
// else negative - the default NaN an x86 multiply produces for inf * 0); without
// saturation, overflow becomes NaN (e4m3fn, |y| rounds above 448, i.e. |y| > 464)
// or infinity (e5m2, |y| >= 61440).
template <int OUT, bool SAT>
__device__ __noinline__ uint32_t fp8_scalar_exact(float x, float scale) {
  const float y = __fmul_rn(x, scale);
  if (y != y) {
    uint32_t sign = 1u;
    if (scale != scale) sign = __float_as_uint(scale) >> 31;
    else if (x != x) sign = __float_as_uint(x) >> 31;
    return 0x7fu | (sign << 7);
  }
  uint32_t b = cvt_fp8x2<OUT>(y, 0.0f) & 0xffu;
  if constexpr (!SAT) {
    const float a = fabsf(y);
    const bool over = (OUT == TNQ_FP8_E4M3) ? (a > 464.0f) : (a >= 61440.0f);
    if (over) b = (b & 0x80u) | Fp8Traits<OUT>::kOverflowByte;
  }
  return b;
}

// Four scaled values -> four fp8 bytes.  The fast path is two hardware cvt; a word
// that contains a NaN byte (or, without saturation, an overflowing value) is redone
// element by element.  x0..x3 are the unscaled inputs.
template <int OUT, bool SAT>
__device__ __forceinline__ uint32_t quant4(float x0, float x1, float x2, float x3, float s) {
  const float y0 = __fmul_rn(x0, s), y1 = __fmul_rn(x1, s), y2 = __fmul_rn(x2, s), y3 = __fmul_rn(x3, s);
  uint32_t w = cvt_fp8x4<OUT>(y0, y1, y2, y3);
  bool redo = (((w & 0x7f7f7f7fu) + Fp8Traits<OUT>::kNanAdd) & 0x80808080u) != 0u;
  if constexpr (!SAT) {
    const float m = fmaxf(fmaxf(fabsf(y0), fabsf(y1)), fmaxf(fabsf(y2), fabsf(y3)));
    redo = redo || ((OUT == TNQ_FP8_E4M3) ? (m > 464.0f) : (m >= 61440.0f));
  }
  if (__builtin_expect(redo, 0)) {
    w = fp8_scalar_exact<OUT, SAT>(x0, s) | (fp8_scalar_exact<OUT, SAT>(x1, s) << 8) |
        (fp8_scalar_exact<OUT, SAT>(x2, s) << 16) | (fp8_scalar_exact<OUT, SAT>(x3, s) << 24);
  }
  return w;
}

// 8 bf16 (one 16-byte vector) -> 8 fp8 bytes
template <int OUT, bool SAT>
__device__ __forceinline__ uint2 quant8_bf16(uint4 v, float s) {
  uint2 o;
  o.x = quant4<OUT, SAT>(bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y), s);
  o.y = quant4<OUT, SAT>(bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w), s);
  return o;
}
// 4 fp32 (one 16-byte vector) -> 4 fp8 bytes
template <int OUT, bool SAT>
__device__ __forceinline__ uint32_t quant4_f32(uint4 v, float s) {
  return quant4<OUT, SAT>(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z),
                          __uint_as_float(v.w), s);
}

// Unchecked variants for callers that have established that every input and the scale
// are finite (then no product can be NaN and saturation covers the rest).
template <int OUT>
__device__ __forceinline__ uint2 quant8_bf16_finite(uint4 v, float s) {
  uint2 o;
  o.x = cvt_fp8x4<OUT>(__fmul_rn(bf16lo(v.x), s), __fmul_rn(bf16hi(v.x), s), __fmul_rn(bf16lo(v.y), s),
                       __fmul_rn(bf16hi(v.y), s));
  o.y = cvt_fp8x4<OUT>(__fmul_rn(bf16lo(v.z), s), __fmul_rn(bf16hi(v.z), s), __fmul_rn(bf16lo(v.w), s),
                       __fmul_rn(bf16hi(v.w), s));
  return o;
}
template <int OUT>
__device__ __forceinline__ uint32_t quant4_f32_finite(uint4 v, float s) {
  return cvt_fp8x4<OUT>(__fmul_rn(__uint_as_float(v.x), s), __fmul_rn(__uint_as_float(v.y), s),
                        __fmul_rn(__uint_as_float(v.z), s), __fmul_rn(__uint_as_float(v.w), s));
}

// bf16x2 helpers on raw 32-bit words
__device__ __forceinline__ uint32_t max_pk_bf16(uint32_t a, uint32_t b) {  // per-half max
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// per-half max(|a|, |b|) of two bf16 pairs in one instruction; the result's sign bits are the XOR of the
// operands' and carry no meaning (mask with 0x7fff7fff before use).  Like max.bf16x2 it returns the other
// operand when one is NaN (blocks that contain NaN are outside the block-scaled quantizers' contract).
__device__ __forceinline__ uint32_t absmax_pk_bf16(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// magnitude bits of a bf16 pair; the result orders like an unsigned integer per half
__device__ __forceinline__ uint32_t mag_pk_bf16(uint32_t a) { return a & 0x7fff7fffu; }
__device__ __forceinline__ uint32_t mul_pk_bf16(uint32_t a, uint32_t s) {  // per-half product, RNE
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(s));
  return r;
}

// amax as fp32 -> scale = fp8_max / max(amax, 1e-12); a NaN amax stays NaN.
__device__ __forceinline__ float scale_from_amax(float amax, float fp8_max) {
  const float a = (amax != amax) ? amax : fmaxf(amax, kAmaxEps);
  return __fdiv_rn(fp8_max, a);
}

// ------------------------------------------------------------------ reductions
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) { return __reduce_max_sync(0xffffffffu, v); }

// max over a CTA of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ uint32_t block_max_u32(uint32_t v, uint32_t* smem32 /* >= 33 words */) {
  v = warp_max_u32(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();  // smem32 may still be read by a previous call
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  uint32_t r = (lane < nwarp) ? smem32[lane] : 0u;
  return warp_max_u32(r);
}

// ------------------------------------------------------------------ scale swizzle
// Byte offset of scale element (r, c) of an [H, W] scale matrix in the 128x4
// ("SWIZZLE_32_4_4") layout; ncb = ceil(W / 4).
__device__ __host__ __forceinline__ int64_t swizzled_offset(int64_t r, int64_t c, int64_t ncb) {
  return ((r >> 7) * ncb + (c >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (c & 3);
}

// ------------------------------------------------------------------ mbarrier + bulk copy (TMA)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait for a phase.  Returns false if the phase did not complete within
// about one second; the caller must then flag the failure and leave.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) return false;
    }
  }
}
// 1-D bulk copy global -> this CTA's shared memory; completion on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.  Single destination CTA.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 2-D tiled TMA load global -> this CTA's shared memory (x = innermost coordinate,
// x * element size must be a multiple of 16 bytes).  Single destination CTA (the
// kernels run with cluster size 1, so shared::cluster names this CTA's memory).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int32_t x, int32_t y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// 2-D tiled TMA store this CTA's shared memory -> global, tracked by the issuing thread's bulk
// async-group.  The part of the box that lies outside the tensor is not written.  x * element
// size must be a multiple of 16 bytes and neither coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t smem_src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}
// the same two copies carrying an L2 eviction-priority policy (createpolicy)
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const void* tmap, int32_t x, int32_t y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], "
      "[%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const void* tmap, uint32_t smem_src, int32_t x, int32_t y, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(tmap),
               "r"(smem_src), "r"(x), "r"(y), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_group_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's committed bulk groups have finished READING shared memory (it may be reused)
__device__ __forceinline__ void bulk_group_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... have completed altogether
__device__ __forceinline__ void bulk_group_wait() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// Programmatic dependent launch: wait for the grid this one depends on / let the
// dependent grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_if(bool wait) {  // the wait as one predicated instruction
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %0, 0;\n\t@p griddepcontrol.wait;\n\t}" ::"r"((uint32_t)wait) : "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace tnq

// ------------------------------------------------------------------ host helpers
namespace tnq_host {
extern thread_local int g_last_cuda_error;
bool tile_loads_evict_first();  // tuning switch TNQ_OPT_TILE_EVICT_FIRST (fp8_tensor.cu)
// Tensor-wide amax pass of the per-tensor cast (fp8_tensor.cu) into the workspace (amax bits in word 1, fp8_max / amax
// in word 2; the latter also to *scale_out when given).  tail_stays: a pass that walks the same tensor from its end
// follows; tensors that exceed L2 are then read with the policy that keeps their last TNQ_OPT_L2_KEEP_MB in L2.
int amax_pass(const void* x, int64_t n, int in_dtype, void* workspace, float* scale_out, float fp8_max, cudaStream_t stream,
              bool tail_stays);
int sm_count();  // SMs of the current device (cached per device)
// single-launch path for tensors that fit in the GPU's shared memory (fp8_fused.cu)
bool fused_plan(int64_t total_bytes, int* grid, uint32_t* slab_bytes);
int fused_dynamic_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype, void* workspace,
                       float* scale_out, cudaStream_t stream, int grid, uint32_t slab_bytes);
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return TNQ_ECUDA;
}
inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}
// Chained launch (TNQ_OPT_PDL_CHAIN, fp8_tensor.cu): the kernel is launched with programmatic stream
// serialization, so its CTAs are placed and run their prologue (barrier setup, descriptor prefetch)
// while the stream's previous kernel drains; every kernel launched this way executes
// griddepcontrol.wait before it touches global memory and releases its own successor right after.
bool pdl_chain();
template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_chain() ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}
}  // namespace tnq_host
