// NVFP4 quantizer: 16-element blocks along the row, e4m3 block scale, fp32 global
// scale, e2m1 codes packed two per byte (low nibble first).
//
// Arithmetic (every step one correctly rounded fp32 operation):
//   A     = max(amax_tensor, 1e-12)     g_dec = A / 2688      g_enc = 2688 / A
//   block: s   = (amax_b / 6) * g_enc    s_q = e4m3(s)  (RNE, saturating at 448)
//          d   = f32(s_q) * g_dec        r   = d == 0 ? 0 : 1 / d
//          code_i = e2m1(x_i * r)        (RNE, ties to the even code, saturating at 6)
// The tile pipeline stages 128x128 bf16 tiles by TMA; a lane owns one block (two
// 16-byte shared loads, block amax on packed bf16 pairs, the block-scale arithmetic
// once per 16 elements), emits 8 packed bytes, and the 128x8 block scales of a tile
// form two 512-byte atoms of the swizzled layout.  NaN inputs are outside the contract.
#include <cuda_fp16.h>

#include "tile_pipeline.cuh"

namespace tnq {

__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
      : "=h"(r)
      : "f"(hi), "f"(lo));
  return r;
}
// eight floats -> eight e2m1 codes in one 32-bit word (f0 in the lowest nibble)
__device__ __forceinline__ uint32_t cvt_e2m1x8(float f0, float f1, float f2, float f3, float f4, float f5, float f6,
                                               float f7) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return r;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)byte));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}

struct Fp4Params {
  int64_t rows, cols;
  const float* global_amax;
  uint8_t* packed;
  uint8_t* sf;
  int layout;
  int64_t sf_w;  // cols / 16
  float* global_scale_out;
};

// x / 6 for a bf16-valued x, correctly rounded, without the division sequence:
// q = x * (1/6), then one residual correction with two FMAs.  Equal to the IEEE
// quotient for every one of the 32 640 finite non-negative bf16 values (checked
// exhaustively on the host and by the parity tests).
__device__ __forceinline__ float div6_bf16_valued(float x) {
  const float c = 1.0f / 6.0f;
  const float q = __fmul_rn(x, c);
  const float r = __fmaf_rn(-q, 6.0f, x);
  return __fmaf_rn(r, c, q);
}

struct Fp4Op {
  using Params = Fp4Params;
  static constexpr int kThreads = 512;
  struct State {
    float g_dec, g_enc;
  };

  __device__ static __forceinline__ State init(const Params& p) {
    const float a_raw = *p.global_amax;
    const float A = (a_raw != a_raw) ? a_raw : fmaxf(a_raw, kAmaxEps);
    State st;
    st.g_dec = __fdiv_rn(A, 2688.0f);
    st.g_enc = __fdiv_rn(2688.0f, A);
    if (p.global_scale_out && blockIdx.x == 0 && threadIdx.x == 0) *p.global_scale_out = st.g_dec;
    return st;
  }

  // A lane owns one 16-element block: block b = lane & 7 of row (lane >> 3) of a four-row
  // group; a warp covers four rows per step and two steps per tile (16 warps).  The two
  // 16-byte halves of the block are fetched in an order that keeps each quarter-warp on
  // distinct shared-memory banks.
  template <bool FULL>
  __device__ static __forceinline__ void process(const Params& p, const State& st, uint32_t tile, uint32_t sf,
                                                 uint32_t tr, uint32_t tc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = lane & 7, sub = lane >> 3;
    const int swap = b >> 2;  // lanes 4-7 of a row fetch the upper half first
    const uint32_t off_first = (uint32_t)(2 * b + swap) * 16u, off_second = (uint32_t)(2 * b + 1 - swap) * 16u;
    const int64_t gcol = (int64_t)tc * kTileCols + b * 16;
    const bool col_ok = FULL || gcol < p.cols;
    const float g_dec = st.g_dec, g_enc = st.g_enc;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int r = (it * 16 + warp) * 4 + sub;
      const uint32_t src = tile + r * 256;
      const uint4 va = lds128(src + off_first);
      const uint4 vb = lds128(src + off_second);
      // max of the sixteen magnitudes, one instruction per word (sign bits of m are meaningless until masked)
      const uint32_t m = absmax_pk_bf16(absmax_pk_bf16(absmax_pk_bf16(va.x, va.y), absmax_pk_bf16(va.z, va.w)),
                                        absmax_pk_bf16(absmax_pk_bf16(vb.x, vb.y), absmax_pk_bf16(vb.z, vb.w)));
      const float amax_b = bf16bits_to_f32(fold_u16x2(m & 0x7fff7fffu));
      const float s = __fmul_rn(div6_bf16_valued(amax_b), g_enc);
      const uint32_t s_q = cvt_fp8x2<TNQ_FP8_E4M3>(s, 0.0f) & 0xffu;
      const float d = __fmul_rn(e4m3_to_f32(s_q), g_dec);
      const float rcp = (d == 0.0f) ? 0.0f : __frcp_rn(d);
      auto quant8 = [rcp](const uint4& v) -> uint32_t {
        return cvt_e2m1x8(__fmul_rn(bf16lo(v.x), rcp), __fmul_rn(bf16hi(v.x), rcp), __fmul_rn(bf16lo(v.y), rcp),
                          __fmul_rn(bf16hi(v.y), rcp), __fmul_rn(bf16lo(v.z), rcp), __fmul_rn(bf16hi(v.z), rcp),
                          __fmul_rn(bf16lo(v.w), rcp), __fmul_rn(bf16hi(v.w), rcp));
      };
      const uint32_t oa = quant8(va), ob = quant8(vb);
      const int64_t row = (int64_t)tr * kTileRows + r;
      const bool ok = FULL || (col_ok && row < p.rows);
      if (ok) stg64(p.packed + (row * p.cols + gcol) / 2, swap ? make_uint2(ob, oa) : make_uint2(oa, ob));
      sts8(sf + (b >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b & 3), ok ? s_q : 0u);
    }
  }

  __device__ static __forceinline__ void finish(const Params&, const State&) {}

  __device__ static __forceinline__ void flush(const Params& p, uint32_t sf, uint32_t tr, uint32_t tc) {
    const int64_t ncb = (p.sf_w + 3) / 4;
    if (p.layout == TNQ_SCALES_SWIZZLED) {
      if (threadIdx.x < 64) {
        const int a = threadIdx.x >> 5, t = threadIdx.x & 31;
        const int64_t ac = (int64_t)tc * 2 + a;
        if (ac < ncb) stg128(p.sf + (tr * ncb + ac) * 512 + t * 16, lds128(sf + a * 512 + t * 16));
      }
    } else {
      for (int idx = threadIdx.x; idx < 256; idx += kThreads) {  // 4 scale bytes (one atom row) per thread
        const int r = idx >> 1, a = idx & 1;
        const int64_t gr = (int64_t)tr * 128 + r;
        if (gr >= p.rows) continue;
        const uint32_t four = lds32(sf + a * 512 + (r & 31) * 16 + (r >> 5) * 4);
        for (int c = 0; c < 4; ++c) {
          const int64_t gc = (int64_t)tc * 8 + a * 4 + c;
          if (gc < p.sf_w) p.sf[gr * p.sf_w + gc] = (uint8_t)(four >> (8 * c));
        }
      }
    }
  }
};

__global__ void __launch_bounds__(Fp4Op::kThreads, 2)
    k_nvfp4(const __grid_constant__ CUtensorMap tmap, Fp4Params p, uint32_t tiles_r, uint32_t tiles_c, uint32_t* status,
            int evict_first) {
  run_tile_pipeline<Fp4Op>(&tmap, p, tiles_r, tiles_c, status, evict_first != 0);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

static int nvfp4_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype, const float* global_amax, void* packed,
                          void* sf, int scale_layout, float* global_scale_out, uint32_t* status, cudaStream_t stream,
                          void* amax_workspace) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16) return TNQ_EUNSUPPORTED;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (global_amax == nullptr) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (x == nullptr || packed == nullptr || sf == nullptr) return TNQ_EINVAL;
  if (cols % 16 != 0) return TNQ_ESHAPE;
  if (rows > 0x7fffffff || cols > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (((rows + 127) / 128) * ((cols + 127) / 128) > 0x7fffffff) return TNQ_EUNSUPPORTED;  // 32-bit tile cursor
  if (!aligned16(x) || !aligned16(packed) || !aligned16(sf)) return TNQ_EALIGN;
  CUtensorMap map;
  int rc = make_tile_map(&map, x, rows, cols);
  if (rc != TNQ_OK) return rc;
  Fp4Params p;
  p.rows = rows, p.cols = cols;
  p.global_amax = global_amax;
  p.packed = static_cast<uint8_t*>(packed), p.sf = static_cast<uint8_t*>(sf);
  p.layout = scale_layout;
  p.sf_w = cols / 16;
  p.global_scale_out = global_scale_out;
  const int cap = tile_resident_ctas<k_nvfp4, Fp4Op::kThreads>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (rows + kTileRows - 1) / kTileRows, tiles_c = (cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  // Dynamic global scale: the amax pass first.  Keeping the end of the matrix in L2 for the quantizer and walking
  // the tiles from that end (what the per-tensor cast does) was measured here and gives nothing: the quantizer then
  // reads 477 MB instead of 537 MB from HBM and takes the same time, it is not bound by its reads.
  if (amax_workspace != nullptr) {
    rc = amax_pass(x, rows * cols, in_dtype, amax_workspace, nullptr, 448.0f, stream, false);
    if (rc != TNQ_OK) return rc;
  }
  return launch_chained(k_nvfp4, dim3(grid), dim3(Fp4Op::kThreads), kTileSmemBytes, stream, map, p, (uint32_t)tiles_r,
                        (uint32_t)tiles_c, status, tile_loads_evict_first() ? 1 : 0);
}

extern "C" int tnq_nvfp4_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype,
                                  const float* global_amax, void* packed, void* sf, int scale_layout,
                                  float* global_scale_out, uint32_t* status, tnq_stream_t stream) {
  return nvfp4_quantize(x, rows, cols, in_dtype, global_amax, packed, sf, scale_layout, global_scale_out, status, stream,
                        nullptr);
}

extern "C" int tnq_nvfp4_quantize_dynamic(const void* x, int64_t rows, int64_t cols, int in_dtype, void* workspace,
                                          void* packed, void* sf, int scale_layout, float* global_scale_out,
                                          tnq_stream_t stream) {
  if (workspace == nullptr) return TNQ_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 31u) != 0) return TNQ_EALIGN;  // the amax pass reads 256-bit vectors
  uint32_t* words = static_cast<uint32_t*>(workspace);
  return nvfp4_quantize(x, rows, cols, in_dtype, reinterpret_cast<const float*>(words + 1), packed, sf, scale_layout,
                        global_scale_out, words + 3, stream, workspace);
}

// ---------------------------------------------------------------- code packing
namespace tnq {
// codes[rows, cols] (one e2m1 code per byte, 0..15) -> packed[rows, cols/2],
// byte = code[2i] | code[2i+1] << 4.  Each thread packs 16 codes into 8 bytes.
__global__ void __launch_bounds__(256) k_pack_fp4(const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n16) {
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = ldg128(codes + i * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[2] = {0u, 0u};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      // bytes c0 c1 c2 c3 -> (c0 | c1 << 4), (c2 | c3 << 4)
      const uint32_t lo = (w[k] & 0xfu) | ((w[k] >> 4) & 0xf0u);
      const uint32_t hi = ((w[k] >> 16) & 0xfu) | ((w[k] >> 20) & 0xf0u);
      o[k >> 1] |= (lo | (hi << 8)) << ((k & 1) * 16);
    }
    stg64(packed + i * 8, make_uint2(o[0], o[1]));
  }
}
}  // namespace tnq

extern "C" int tnq_pack_fp4_codes(const void* codes, int64_t rows, int64_t cols, void* packed, tnq_stream_t stream) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (codes == nullptr || packed == nullptr) return TNQ_EINVAL;
  if (cols % 16 != 0) return TNQ_ESHAPE;
  if (!aligned16(codes) || !aligned16(packed)) return TNQ_EALIGN;
  const int64_t n16 = rows * cols / 16;
  int64_t blocks = (n16 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return launch_chained(tnq::k_pack_fp4, dim3((unsigned)blocks), dim3(256), 0, stream, static_cast<const uint8_t*>(codes),
                        static_cast<uint8_t*>(packed), n16);
}
