// NVFP4 quantizer: 16-element blocks along the row, e4m3 block scale, fp32 global
// scale, e2m1 codes packed two per byte (low nibble first).
//
// Arithmetic (every step one correctly rounded fp32 operation):
//   A     = max(amax_tensor, 1e-12)     g_dec = A / 2688      g_enc = 2688 / A
//   block: s   = (amax_b / 6) * g_enc    s_q = e4m3(s)  (RNE, saturating at 448)
//          d   = f32(s_q) * g_dec        r   = d == 0 ? 0 : 1 / d
//          code_i = e2m1(x_i * r)        (RNE, ties to the even code, saturating at 6)
// The tile pipeline stages 128x128 bf16 tiles by TMA; two adjacent lanes own one
// block (16-byte shared loads, one shuffle), each lane emits 4 packed bytes, and
// the 128x8 block scales of a tile form two 512-byte atoms of the swizzled layout.
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

struct Fp4Op {
  using Params = Fp4Params;

  __device__ static __forceinline__ void process(const Params& p, const uint8_t* tile, uint8_t* sf, int64_t tr,
                                                 int64_t tc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float a_raw = *p.global_amax;
    const float A = (a_raw != a_raw) ? a_raw : fmaxf(a_raw, kAmaxEps);
    const float g_dec = __fdiv_rn(A, 2688.0f), g_enc = __fdiv_rn(2688.0f, A);
    if (p.global_scale_out && blockIdx.x == 0 && threadIdx.x == 0) *p.global_scale_out = g_dec;
    const int chunk = lane & 15;
    const int64_t col0 = tc * kTileCols + chunk * 8;
    const bool col_ok = col0 < p.cols;
#pragma unroll 4
    for (int it = 0; it < 8; ++it) {
      const int r = warp * 16 + it * 2 + (lane >> 4);
      const uint4 v = *reinterpret_cast<const uint4*>(tile + r * 256 + chunk * 16);
      uint32_t m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(0u, v.x), v.y), v.z), v.w);
      m = fold_u16x2(m);
      m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
      const float amax_b = bf16bits_to_f32(m);
      const float s = __fmul_rn(__fdiv_rn(amax_b, 6.0f), g_enc);
      const uint32_t s_q = cvt_fp8x2<TNQ_FP8_E4M3>(s, 0.0f) & 0xffu;
      const float d = __fmul_rn(e4m3_to_f32(s_q), g_dec);
      const float rcp = (d == 0.0f) ? 0.0f : __fdiv_rn(1.0f, d);
      const uint32_t b0 = cvt_e2m1x2(__fmul_rn(bf16lo(v.x), rcp), __fmul_rn(bf16hi(v.x), rcp));
      const uint32_t b1 = cvt_e2m1x2(__fmul_rn(bf16lo(v.y), rcp), __fmul_rn(bf16hi(v.y), rcp));
      const uint32_t b2 = cvt_e2m1x2(__fmul_rn(bf16lo(v.z), rcp), __fmul_rn(bf16hi(v.z), rcp));
      const uint32_t b3 = cvt_e2m1x2(__fmul_rn(bf16lo(v.w), rcp), __fmul_rn(bf16hi(v.w), rcp));
      const int64_t row = tr * kTileRows + r;
      const bool ok = col_ok && row < p.rows;
      if (ok) stg32(p.packed + (row * p.cols + col0) / 2, b0 | (b1 << 8) | (b2 << 16) | (b3 << 24));
      if ((lane & 1) == 0) {
        const int cb = chunk >> 1;  // 0..7: block within the tile row
        sf[(cb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (cb & 3)] = ok ? (uint8_t)s_q : (uint8_t)0;
      }
    }
  }

  __device__ static __forceinline__ void flush(const Params& p, const uint8_t* sf, int64_t tr, int64_t tc) {
    const int64_t ncb = (p.sf_w + 3) / 4;
    if (p.layout == TNQ_SCALES_SWIZZLED) {
      if (threadIdx.x < 64) {
        const int a = threadIdx.x >> 5, t = threadIdx.x & 31;
        const int64_t ac = tc * 2 + a;
        if (ac < ncb) stg128(p.sf + (tr * ncb + ac) * 512 + t * 16, *reinterpret_cast<const uint4*>(sf + a * 512 + t * 16));
      }
    } else {
      for (int idx = threadIdx.x; idx < 1024; idx += kTileThreads) {
        const int r = idx >> 3, c = idx & 7;
        const int64_t gr = tr * 128 + r, gc = tc * 8 + c;
        if (gr < p.rows && gc < p.sf_w) p.sf[gr * p.sf_w + gc] = sf[(c >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (c & 3)];
      }
    }
  }
};

__global__ void __launch_bounds__(kTileThreads)
    k_nvfp4(const __grid_constant__ CUtensorMap tmap, Fp4Params p, int64_t tiles_r, int64_t tiles_c, uint32_t* status) {
  run_tile_pipeline<Fp4Op>(&tmap, p, tiles_r, tiles_c, status);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

extern "C" int tnq_nvfp4_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype,
                                  const float* global_amax, void* packed, void* sf, int scale_layout,
                                  float* global_scale_out, uint32_t* status, tnq_stream_t stream) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16) return TNQ_EUNSUPPORTED;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  if (global_amax == nullptr) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (x == nullptr || packed == nullptr || sf == nullptr) return TNQ_EINVAL;
  if (cols % 16 != 0) return TNQ_ESHAPE;
  if (rows > 0x7fffffff || cols > 0x7fffffff) return TNQ_EUNSUPPORTED;
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
  const int cap = tile_resident_ctas<k_nvfp4>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (rows + kTileRows - 1) / kTileRows, tiles_c = (cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  k_nvfp4<<<grid, kTileThreads, kTileSmemBytes, stream>>>(map, p, tiles_r, tiles_c, status);
  return check_launch();
}

// ---------------------------------------------------------------- code packing
namespace tnq {
// codes[rows, cols] (one e2m1 code per byte, 0..15) -> packed[rows, cols/2],
// byte = code[2i] | code[2i+1] << 4.  Each thread packs 16 codes into 8 bytes.
__global__ void __launch_bounds__(256) k_pack_fp4(const uint8_t* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n16) {
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
  tnq::k_pack_fp4<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(codes), static_cast<uint8_t*>(packed), n16);
  return check_launch();
}
