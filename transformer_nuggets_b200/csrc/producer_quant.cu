// Producer epilogues: the op that makes a bf16 activation (RMSNorm, SwiGLU) fused with the
// quantizer that consumes it (row-wise dynamic FP8, MXFP8 row-wise); the bf16 tensor the
// producer would write and the quantizer would read back never touches HBM.
//
// RMSNorm:
//     var  = mean(f32(x)^2) over the row            fp32, fixed summation order (below)
//     rstd = 1 / sqrt(var + eps)                    two IEEE fp32 operations
//     y    = bf16( (f32(x) * rstd) * f32(w) )        two fp32 products, one RNE rounding
//     q    = e4m3_sat( f32(y) * s ),  s = 448 / max(max|y|, 1e-12)      per row          (row-wise FP8)
//  or q    = e4m3( y * 2^-e ),  E8M0 byte = e + 127 per 32 elements                       (MXFP8, mxfp8.cu's rule)
//
// which is the eager RMSNorm the reference profiles for fusion
// (examples/rms_norm_fusion_profile.py:26-31: square, mean, rsqrt, two products, one cast to
// the input dtype) followed by the row-wise cast of fp8_rowwise.cu on its bf16 result.  Every
// step after the sum of squares is a single correctly rounded operation and so is identical on
// any IEEE machine; the sum itself depends on the order of the additions, which here is: each
// thread keeps four partial sums over its elements (element j goes to sum j mod 4) and adds
// them as (p0 + p1) + (p2 + p3), lanes are combined by a butterfly (xor 16, 8, 4, 2, 1), warps
// in warp order.  A CPU run of the eager formula adds in another
// order, so its variance can differ in the last bits and y in an occasional last-place bf16
// rounding; the cast of y is exact.  `y_out` (optional) returns y for callers that also need
// the normalised activation, and lets a test check the cast against the y actually used.
//
// SwiGLU: y = bf16( f32(bf16(silu(f32(a)))) * f32(b) ), silu(a) = a / (1 + exp(-a)) - the eager
// bf16 evaluation of `F.silu(w1(x)) * w3(x)` (llama/model.py:228), whose result is the operand
// of the next GEMM.  exp and the division use the hardware approximations (ex2.approx, rcp:
// relative error near 2^-21), so here too y can differ from a CPU run in an occasional
// last-place bf16 rounding while the quantization of y is exact.
//
// A row is owned by G threads holding their share (VPT 32-byte vectors each) in registers; where
// the registers allow (VPT <= 2) the next row's loads are issued before this row's arithmetic.
// (A lane-private cp.async ring, four rows deep, measured slower here: the kernel is bound by the
// two dependent row reductions, not by bytes in flight.)  bf16 halves are squared and widened
// by the mixed-precision FMA (fma.rn.f32.bf16) straight from the packed registers.  The weight
// vectors of a thread's fixed columns are loaded once and reused for every row.  The
// kernel reads 2 bytes and writes 1 byte per element (plus 4 bytes per row).
#include "mx_scale.cuh"

namespace tnq {

constexpr int kNormThreads = 256;

// acc + a.lo^2 + a.hi^2 for a packed bf16 pair (each square is exact in fp32, each addition rounds)
__device__ __forceinline__ void sumsq_pk(uint32_t pk, float& acc_lo, float& acc_hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tfma.rn.f32.bf16 %0, l, l, %0;\n\tfma.rn.f32.bf16 %1, h, h, %1;\n\t}"
      : "+f"(acc_lo), "+f"(acc_hi)
      : "r"(pk));
}
// the two halves of a packed bf16 pair as fp32 (x * 1 - 0 on the FMA pipe)
__device__ __forceinline__ void widen_pk(uint32_t pk, float& lo, float& hi) {
  asm("{\n\t.reg .b16 l, h, one;\n\tmov.b32 {l, h}, %2;\n\tmov.b16 one, 0x3f80;\n\t"
      "fma.rn.f32.bf16 %0, l, one, 0f80000000;\n\tfma.rn.f32.bf16 %1, h, one, 0f80000000;\n\t}"
      : "=&f"(lo), "=&f"(hi)
      : "r"(pk));
}

// Outputs of the fused kernel: row-wise FP8 (q + one fp32 scale per row) or MXFP8 (q + one E8M0
// byte per 32 elements, raw [rows, cols / 32] or swizzled 128x4), optionally the normalised rows.
struct NormOut {
  uint8_t* q;
  float* scale;    // row-wise
  uint8_t* sf;     // MXFP8
  int e8m0_bias;   // (m + bias) >> 7 is the stored byte before its floor of 1: ceil or floor rule
  int sf_layout;
  int64_t sf_w;    // scale columns per row (cols / 32)
  uint8_t* y;
};
constexpr int kNormRowwise = 0, kNormMx = 1;

constexpr int kProdRmsNorm = 0, kProdSwiGlu = 1;

// silu(a) * b the way eager bf16 PyTorch evaluates it (llama/model.py:228 of the reference):
// silu in fp32 (a / (1 + exp(-a))) rounded to bf16, the product in fp32 rounded to bf16.
__device__ __forceinline__ uint32_t swiglu_pk(uint32_t a_pk, uint32_t b_pk) {
  float a0, a1, b0, b1;
  widen_pk(a_pk, a0, a1);
  widen_pk(b_pk, b0, b1);
  // exp and the reciprocal are the hardware approximations (relative error near 2^-22, far below half a
  // bf16 step), spelled out rather than taken from __expf / __fdividef so that both run in their
  // flush-to-zero forms (no extra range handling; neither flushes anything that matters here: a
  // subnormal exp(-a) leaves 1 + exp(-a) = 1 either way, and the divisor below is never subnormal).
  // An approximate division returns 0 for a divisor in (2^126, 2^128), which 1 + exp(-a) reaches for a in
  // about (-88.7, -87.3) although the quotient there (about -5e-37) is still a normal bf16 value: both
  // operands are therefore scaled by 2^-4 (exact; (1 + e) / 16 comes out of one FMA bit-identical to the
  // sum rounded and then scaled), which keeps the divisor below 2^124.
  auto silu = [](float a) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(a, -1.4426950408889634f)));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(e, 0.0625f, 0.0625f)));
    return __fmul_rn(__fmul_rn(a, 0.0625f), r);
  };
  const float s0 = silu(a0), s1 = silu(a1);
  uint32_t s_pk;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(s_pk) : "f"(s1), "f"(s0));
  float t0, t1;
  widen_pk(s_pk, t0, t1);
  uint32_t p;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(__fmul_rn(t1, b1)), "f"(__fmul_rn(t0, b0)));
  return p;
}

// PROD = kProdRmsNorm: `second` is the bf16 weight vector [cols].
// PROD = kProdSwiGlu : `second` is the bf16 matrix b [rows, cols]; y = silu(x) * b, eps unused.
// The RMSNorm -> row-wise kernel is held to 80 registers so that three CTAs fit on an SM (75.9 -> 71.2 us at
// 16384 x 8192; it would take 110 and two CTAs otherwise).  The other forms leave the register count to the
// compiler (a minimum of 0 means "not specified"; asking for 1 lets it take 128 and costs SwiGLU 12 %).
template <int G, int VPT, int KIND, int PROD, bool WRITE_Y>
__global__ void __launch_bounds__(kNormThreads, (PROD == kProdRmsNorm && KIND == kNormRowwise && VPT <= 2) ? 3 : 0)
    k_producer_quant(const uint8_t* __restrict__ x, const uint8_t* __restrict__ second, float eps, int64_t rows, int64_t cols,
                    int nvec_row, NormOut out) {
  const uint8_t* const weight = second;
  uint8_t* const q = out.q;
  float* const scale = out.scale;
  uint8_t* const y_out = out.y;
  constexpr int kGroups = kNormThreads / G;
  constexpr int kWarpsPerGroup = G / 32;
  // a second register copy of the row(s) fits
  constexpr bool kPrefetch = PROD == kProdRmsNorm ? VPT <= 2 : VPT <= 1;
  constexpr int kB = PROD == kProdSwiGlu ? VPT : 1;
  __shared__ float s_sum[kNormThreads / 32];
  __shared__ uint32_t s_max[kNormThreads / 32];
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int64_t row_bytes = (int64_t)nvec_row * 32;
  const int64_t n_steps = (rows + kGroups - 1) / kGroups;  // identical trip count for every thread of a CTA
  const float n = (float)cols;

  Vec32B wv[PROD == kProdRmsNorm ? VPT : 1];  // the weights of this thread's columns, reused for every row
  if constexpr (PROD == kProdRmsNorm) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = t + k * G;
      if (vi < nvec_row) {
        wv[k] = ldg256(weight + (int64_t)vi * 32);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[k].w[i] = 0u;
      }
    }
  }
  auto load_row = [&](Vec32B (&dst)[VPT], Vec32B (&dst_b)[kB], int64_t step) {
    const int64_t r = step * kGroups + g;
    const bool ok = step < n_steps && r < rows;
    const uint8_t* xr = x + r * row_bytes;
    const uint8_t* br = second + r * row_bytes;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = t + k * G;
      if (ok && vi < nvec_row) {
        dst[k] = ldg256(xr + (int64_t)vi * 32);
        if constexpr (PROD == kProdSwiGlu) dst_b[k] = ldg256(br + (int64_t)vi * 32);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[k].w[i] = 0u;
        if constexpr (PROD == kProdSwiGlu) {
#pragma unroll
          for (int i = 0; i < 8; ++i) dst_b[k].w[i] = 0u;
        }
      }
    }
  };
  Vec32B v[VPT], vn[kPrefetch ? VPT : 1];
  Vec32B bv[kB], bn[(kPrefetch && PROD == kProdSwiGlu) ? VPT : 1];
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  load_row(v, bv, blockIdx.x);
  for (int64_t step = blockIdx.x; step < n_steps; step += gridDim.x) {
    const int64_t r = step * kGroups + g;
    const bool live = r < rows;
    if constexpr (kPrefetch) {  // the next row's loads fly during this row's math
      if constexpr (PROD == kProdSwiGlu) load_row(vn, bn, step + gridDim.x);
      else load_row(vn, bv, step + gridDim.x);  // bv is a dummy here
    }
    uint32_t m = 0;
    if constexpr (PROD == kProdSwiGlu) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t p = swiglu_pk(v[k].w[i], bv[k].w[i]);
          v[k].w[i] = p;
          m = absmax_bf16x2_1op(m, p);  // one instruction; NaN -> 0x7fff; sign bits meaningless until masked
        }
      }
    } else {
    // ---- sum of squares: four interleaved partial sums per thread, then the butterfly
    float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        sumsq_pk(v[k].w[i], p0, p1);
        sumsq_pk(v[k].w[i + 1], p2, p3);
      }
    }
    float ss = __fadd_rn(__fadd_rn(p0, p1), __fadd_rn(p2, p3));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if constexpr (G > 32) {
      __syncthreads();  // the previous row's readers are done with s_sum / s_max
      if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = s_sum[g * kWarpsPerGroup];
#pragma unroll
      for (int w = 1; w < kWarpsPerGroup; ++w) tot = __fadd_rn(tot, s_sum[g * kWarpsPerGroup + w]);
      ss = tot;
    }
    const float var = __fdiv_rn(ss, n);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    // ---- y in place of x (bf16 pairs), and its magnitude maximum
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float xa, xb, wa, wb;
        widen_pk(v[k].w[i], xa, xb);
        widen_pk(wv[k].w[i], wa, wb);
        const float a = __fmul_rn(__fmul_rn(xa, rstd), wa), b = __fmul_rn(__fmul_rn(xb, rstd), wb);
        uint32_t p;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(b), "f"(a));  // a in the low half, RNE
        v[k].w[i] = p;
        m = absmax_bf16x2_1op(m, p);  // one instruction; NaN -> 0x7fff; sign bits meaningless until masked
      }
    }
    }  // RMSNorm
    if constexpr (KIND == kNormMx) {
      // a 32-element block = the vectors of two adjacent lanes: one shuffle gives the block amax
      if (live) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int vi = t + k * G;
          uint32_t bm = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) bm = absmax_bf16x2(bm, v[k].w[i]);
          bm = fold_u16x2(bm);
          bm = max(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
          const uint32_t byte = (uint32_t)max(((int)bm + out.e8m0_bias) >> 7, 1);
          const uint16_t inv = (uint16_t)((254u - byte) << 7);  // bf16 bits of 2^-e
          if (vi < nvec_row) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = e4m3x4_scaled(v[k].w[2 * j], v[k].w[2 * j + 1], inv);
            stg128(q + r * cols + (int64_t)vi * 16, make_uint4(o[0], o[1], o[2], o[3]));
            if ((t & 1) == 0) {
              const int64_t b = vi >> 1;
              const int64_t at = out.sf_layout == TNQ_SCALES_SWIZZLED ? swizzled_offset(r, b, (out.sf_w + 3) >> 2)
                                                                      : r * out.sf_w + b;
              out.sf[at] = (uint8_t)byte;
            }
            if constexpr (WRITE_Y)
              stg256(y_out + r * row_bytes + (int64_t)vi * 32, v[k].w[0], v[k].w[1], v[k].w[2], v[k].w[3], v[k].w[4],
                     v[k].w[5], v[k].w[6], v[k].w[7]);
          }
        }
      }
    } else {
    m = warp_max_u32(fold_u16x2(m & 0x7fff7fffu) << 16);
    if constexpr (G > 32) {
      if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
      __syncthreads();
      uint32_t mm = 0;
#pragma unroll
      for (int w = 0; w < kWarpsPerGroup; ++w) mm = max(mm, s_max[g * kWarpsPerGroup + w]);
      m = mm;
    }
    if (live) {
      const float s = scale_from_amax(__uint_as_float(m), 448.0f);
      const bool finite = m < 0x7f800000u;  // uniform over the row's threads
      if (t == 0) scale[r] = s;
      uint8_t* qr = q + r * cols;
      if (!finite) {  // a NaN as the CPU cast to bf16 writes it (0x7fc0), only where one can occur
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t p = v[k].w[i];
            if ((p & 0x7fffu) > 0x7f80u) p = (p & 0xffff0000u) | 0x7fc0u;
            if ((p & 0x7fff0000u) > 0x7f800000u) p = (p & 0xffffu) | 0x7fc00000u;
            v[k].w[i] = p;
          }
        }
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int vi = t + k * G;
        if (vi >= nvec_row) continue;
        uint32_t o[4];
        if (finite) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float y0, y1, y2, y3;
            widen_pk(v[k].w[2 * j], y0, y1);
            widen_pk(v[k].w[2 * j + 1], y2, y3);
            o[j] = cvt_fp8x4<TNQ_FP8_E4M3>(__fmul_rn(y0, s), __fmul_rn(y1, s), __fmul_rn(y2, s), __fmul_rn(y3, s));
          }
        } else {
          const uint2 a = quant8_bf16<TNQ_FP8_E4M3, true>(make_uint4(v[k].w[0], v[k].w[1], v[k].w[2], v[k].w[3]), s);
          const uint2 b = quant8_bf16<TNQ_FP8_E4M3, true>(make_uint4(v[k].w[4], v[k].w[5], v[k].w[6], v[k].w[7]), s);
          o[0] = a.x, o[1] = a.y, o[2] = b.x, o[3] = b.y;
        }
        stg128(qr + (int64_t)vi * 16, make_uint4(o[0], o[1], o[2], o[3]));
        if constexpr (WRITE_Y)
          stg256(y_out + r * row_bytes + (int64_t)vi * 32, v[k].w[0], v[k].w[1], v[k].w[2], v[k].w[3], v[k].w[4],
                 v[k].w[5], v[k].w[6], v[k].w[7]);
      }
    }
    }  // row-wise FP8
    if constexpr (kPrefetch) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) v[k] = vn[k];
      if constexpr (PROD == kProdSwiGlu) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) bv[k] = bn[k];
      }
    } else {
      load_row(v, bv, step + gridDim.x);
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <int G, int VPT, int KIND, int PROD, bool WRITE_Y>
static int launch_norm(const uint8_t* x, const uint8_t* w, float eps, int64_t rows, int64_t cols, int nvec_row,
                       const NormOut& out, cudaStream_t stream) {
  constexpr int kGroups = kNormThreads / G;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_producer_quant<G, VPT, KIND, PROD, WRITE_Y>, kNormThreads, 0) !=
            cudaSuccess ||
        per_sm < 1)
      per_sm = 1;
    cached[dev] = per_sm * sm_count();
  }
  const int64_t steps = (rows + kGroups - 1) / kGroups;
  const int grid = (int)(steps < cached[dev] ? steps : cached[dev]);
  return launch_chained(k_producer_quant<G, VPT, KIND, PROD, WRITE_Y>, dim3(grid), dim3(kNormThreads), 0, stream, x, w, eps, rows,
                        cols, nvec_row, out);
}

template <int G, int VPT, int KIND, int PROD>
static int launch_norm_y(const uint8_t* x, const uint8_t* w, float eps, int64_t rows, int64_t cols, int nvec_row,
                         const NormOut& out, cudaStream_t stream) {
  return out.y ? launch_norm<G, VPT, KIND, PROD, true>(x, w, eps, rows, cols, nvec_row, out, stream)
               : launch_norm<G, VPT, KIND, PROD, false>(x, w, eps, rows, cols, nvec_row, out, stream);
}

// the largest group that still gives every thread a vector (as in the plain row-wise cast)
template <int KIND, int PROD>
static int launch_norm_shape(const uint8_t* xp, const uint8_t* wp, float eps, int64_t rows, int64_t cols, int nv,
                             const NormOut& out, cudaStream_t stream) {
  if (nv > 4 * 128 || nv >= 256) {
    if (nv <= 256) return launch_norm_y<256, 1, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
    if (nv <= 512) return launch_norm_y<256, 2, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
    return launch_norm_y<256, 4, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
  }
  if (nv >= 128) {
    if (nv <= 128) return launch_norm_y<128, 1, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
    return launch_norm_y<128, 2, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
  }
  if (nv >= 64) {
    if (nv <= 64) return launch_norm_y<64, 1, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
    return launch_norm_y<64, 2, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
  }
  if (nv <= 32) return launch_norm_y<32, 1, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
  return launch_norm_y<32, 2, KIND, PROD>(xp, wp, eps, rows, cols, nv, out, stream);
}

static int norm_common_checks(const void* x, const void* weight, int64_t rows, int64_t cols, const void* q, const void* y,
                              int64_t multiple) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (!x || !weight || !q) return TNQ_EINVAL;
  if (cols % multiple != 0) return TNQ_ESHAPE;
  if (cols / 16 > 4 * 256) return TNQ_EUNSUPPORTED;  // rows of up to 16384 elements stay in registers
  if ((reinterpret_cast<uintptr_t>(x) & 31u) || (reinterpret_cast<uintptr_t>(weight) & 31u) || !aligned16(q) ||
      (y && (reinterpret_cast<uintptr_t>(y) & 31u)))
    return TNQ_EALIGN;
  return -1;  // go on
}

extern "C" int tnq_rmsnorm_fp8_rowwise(const void* x, const void* weight, float eps, int64_t rows, int64_t cols,
                                       void* q_e4m3, float* scale, void* y_bf16, tnq_stream_t stream) {
  const int rc = norm_common_checks(x, weight, rows, cols, q_e4m3, y_bf16, 16);  // whole 32-byte vectors of bf16
  if (rc >= 0) return rc;
  if (!scale) return TNQ_EINVAL;
  NormOut out{};
  out.q = static_cast<uint8_t*>(q_e4m3), out.scale = scale, out.y = static_cast<uint8_t*>(y_bf16);
  return launch_norm_shape<kNormRowwise, kProdRmsNorm>(static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), eps, rows,
                                         cols, (int)(cols / 16), out, stream);
}

extern "C" int tnq_rmsnorm_mxfp8(const void* x, const void* weight, float eps, int64_t rows, int64_t cols, void* q_e4m3,
                                 void* sf, int scale_mode, int scale_layout, void* y_bf16, tnq_stream_t stream) {
  if (scale_mode != TNQ_E8M0_CEIL && scale_mode != TNQ_E8M0_FLOOR) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  const int rc = norm_common_checks(x, weight, rows, cols, q_e4m3, y_bf16, 32);  // whole 32-element blocks
  if (rc >= 0) return rc;
  if (!sf) return TNQ_EINVAL;
  NormOut out{};
  out.q = static_cast<uint8_t*>(q_e4m3), out.sf = static_cast<uint8_t*>(sf), out.y = static_cast<uint8_t*>(y_bf16);
  out.e8m0_bias = scale_mode == TNQ_E8M0_CEIL ? (0x1f - 1024) : -1024;
  out.sf_layout = scale_layout, out.sf_w = cols / 32;
  return launch_norm_shape<kNormMx, kProdRmsNorm>(static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), eps, rows, cols,
                                    (int)(cols / 16), out, stream);
}

extern "C" int tnq_swiglu_fp8_rowwise(const void* a, const void* b, int64_t rows, int64_t cols, void* q_e4m3, float* scale,
                                      void* y_bf16, tnq_stream_t stream) {
  const int rc = norm_common_checks(a, b, rows, cols, q_e4m3, y_bf16, 16);
  if (rc >= 0) return rc;
  if (!scale) return TNQ_EINVAL;
  NormOut out{};
  out.q = static_cast<uint8_t*>(q_e4m3), out.scale = scale, out.y = static_cast<uint8_t*>(y_bf16);
  return launch_norm_shape<kNormRowwise, kProdSwiGlu>(static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), 0.0f,
                                                      rows, cols, (int)(cols / 16), out, stream);
}

extern "C" int tnq_swiglu_mxfp8(const void* a, const void* b, int64_t rows, int64_t cols, void* q_e4m3, void* sf,
                                int scale_mode, int scale_layout, void* y_bf16, tnq_stream_t stream) {
  if (scale_mode != TNQ_E8M0_CEIL && scale_mode != TNQ_E8M0_FLOOR) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  const int rc = norm_common_checks(a, b, rows, cols, q_e4m3, y_bf16, 32);
  if (rc >= 0) return rc;
  if (!sf) return TNQ_EINVAL;
  NormOut out{};
  out.q = static_cast<uint8_t*>(q_e4m3), out.sf = static_cast<uint8_t*>(sf), out.y = static_cast<uint8_t*>(y_bf16);
  out.e8m0_bias = scale_mode == TNQ_E8M0_CEIL ? (0x1f - 1024) : -1024;
  out.sf_layout = scale_layout, out.sf_w = cols / 32;
  return launch_norm_shape<kNormMx, kProdSwiGlu>(static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), 0.0f, rows,
                                                 cols, (int)(cols / 16), out, stream);
}
