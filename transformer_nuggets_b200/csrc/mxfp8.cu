// MXFP8 quantizer: 32-element blocks, E8M0 scale byte, e4m3 payload; row-wise
// (blocks along the row) and column-wise (blocks along the column, stored
// transposed) outputs from ONE read of the input.
//
// A 128x128 tile staged in shared memory by TMA is consumed twice: a row pass in
// which four adjacent lanes own one 32-element block (conflict-free 16-byte shared
// loads, two shuffles for the block amax, 8-byte coalesced stores), and a column
// pass in which a thread owns two adjacent columns over 32 rows (conflict-free
// 4-byte shared loads, 32 contiguous output bytes per column).  One tile yields
// exactly one 512-byte atom of the swizzled 128x4 scale layout in each direction;
// the atom is assembled in shared memory and written with 16-byte stores.
//
// Exponent rule on the bf16 amax bits (E = biased exponent, m = 7-bit mantissa):
//   ceil : e = E - 127 - 8 + (m > 0x60)      == ceil(log2(amax / 448))
//   floor: e = E - 127 - 8                   == floor(log2(amax)) - 8
// clamped to [-126, 127]; zero / subnormal amax gives -126.  x * 2^-e is exact.
#include "tile_pipeline.cuh"

namespace tnq {

template <int MODE>
__device__ __forceinline__ int e8m0_exponent(uint32_t amax_bf16_bits) {
  const int E = (int)((amax_bf16_bits >> 7) & 0xffu);
  const int m = (int)(amax_bf16_bits & 0x7fu);
  if (E == 0) return -126;
  int e = E - 135;
  if (MODE == TNQ_E8M0_CEIL) e += (m > 0x60) ? 1 : 0;
  return max(-126, min(127, e));
}
__device__ __forceinline__ float exp2_neg(int e) {  // 2^-e, e in [-126, 126]
  return __uint_as_float((uint32_t)(127 - e) << 23);
}

struct MxParams {
  int64_t rows, cols;
  uint8_t* q_row;
  uint8_t* sf_row;
  uint8_t* q_col;
  uint8_t* sf_col;
  int layout;
  int64_t sf_row_w;  // cols / 32
  int64_t sf_col_w;  // rows / 32
};

template <bool ROW, bool COL, int MODE>
struct MxOp {
  using Params = MxParams;

  __device__ static __forceinline__ void process(const Params& p, const uint8_t* tile, uint8_t* sf, int64_t tr,
                                                 int64_t tc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if constexpr (ROW) {
      uint8_t* sf_row = sf;  // 512 bytes
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
        m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
        const int e = e8m0_exponent<MODE>(m);
        const uint2 o = quant8_bf16<TNQ_FP8_E4M3, true>(v, exp2_neg(e));
        const int64_t row = tr * kTileRows + r;
        const bool ok = col_ok && row < p.rows;
        if (ok) stg64(p.q_row + row * p.cols + col0, o);
        if ((lane & 3) == 0) sf_row[(r & 31) * 16 + (r >> 5) * 4 + (chunk >> 2)] = ok ? (uint8_t)(e + 127) : (uint8_t)0;
      }
    }
    if constexpr (COL) {
      uint8_t* sf_col = sf + 512;
      const int w = threadIdx.x & 63, rb = threadIdx.x >> 6;
      uint32_t vals[32];
      uint32_t m = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        vals[i] = *reinterpret_cast<const uint32_t*>(tile + (rb * 32 + i) * 256 + w * 4);
        m = absmax_bf16x2(m, vals[i]);
      }
      const int e_lo = e8m0_exponent<MODE>(m & 0xffffu), e_hi = e8m0_exponent<MODE>(m >> 16);
      const float s_lo = exp2_neg(e_lo), s_hi = exp2_neg(e_hi);
      uint32_t lo[8], hi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        lo[j] = quant4<TNQ_FP8_E4M3, true>(bf16lo(vals[4 * j]), bf16lo(vals[4 * j + 1]), bf16lo(vals[4 * j + 2]),
                                           bf16lo(vals[4 * j + 3]), s_lo);
        hi[j] = quant4<TNQ_FP8_E4M3, true>(bf16hi(vals[4 * j]), bf16hi(vals[4 * j + 1]), bf16hi(vals[4 * j + 2]),
                                           bf16hi(vals[4 * j + 3]), s_hi);
      }
      const int64_t c = tc * kTileCols + 2 * w;
      const int64_t r0 = tr * kTileRows + rb * 32;
      const bool ok = c < p.cols && r0 < p.rows;
      if (ok) {
        uint8_t* d0 = p.q_col + c * p.rows + r0;
        stg128(d0, make_uint4(lo[0], lo[1], lo[2], lo[3]));
        stg128(d0 + 16, make_uint4(lo[4], lo[5], lo[6], lo[7]));
        uint8_t* d1 = d0 + p.rows;
        stg128(d1, make_uint4(hi[0], hi[1], hi[2], hi[3]));
        stg128(d1 + 16, make_uint4(hi[4], hi[5], hi[6], hi[7]));
      }
      const int c0 = 2 * w, c1 = 2 * w + 1;
      sf_col[(c0 & 31) * 16 + (c0 >> 5) * 4 + rb] = ok ? (uint8_t)(e_lo + 127) : (uint8_t)0;
      sf_col[(c1 & 31) * 16 + (c1 >> 5) * 4 + rb] = ok ? (uint8_t)(e_hi + 127) : (uint8_t)0;
    }
  }

  // sf holds one swizzled atom per direction; write it out swizzled (whole atom) or raw.
  __device__ static __forceinline__ void flush_one(const uint8_t* atom, uint8_t* dst, int layout, int64_t R,
                                                   int64_t W, int64_t ar, int64_t ac) {
    // atom covers scale rows ar*128..+127 and scale columns ac*4..+3 of an [R, W] scale matrix
    if (layout == TNQ_SCALES_SWIZZLED) {
      const int64_t ncb = (W + 3) / 4;
      if (threadIdx.x < 32)
        stg128(dst + (ar * ncb + ac) * 512 + threadIdx.x * 16, *reinterpret_cast<const uint4*>(atom + threadIdx.x * 16));
    } else {
      for (int idx = threadIdx.x; idx < 512; idx += kTileThreads) {
        const int r = idx >> 2, c = idx & 3;
        const int64_t gr = ar * 128 + r, gc = ac * 4 + c;
        if (gr < R && gc < W) dst[gr * W + gc] = atom[(r & 31) * 16 + (r >> 5) * 4 + c];
      }
    }
  }

  __device__ static __forceinline__ void flush(const Params& p, const uint8_t* sf, int64_t tr, int64_t tc) {
    if constexpr (ROW) flush_one(sf, p.sf_row, p.layout, p.rows, p.sf_row_w, tr, tc);
    if constexpr (COL) flush_one(sf + 512, p.sf_col, p.layout, p.cols, p.sf_col_w, tc, tr);
  }
};

template <bool ROW, bool COL, int MODE>
__global__ void __launch_bounds__(kTileThreads)
    k_mxfp8(const __grid_constant__ CUtensorMap tmap, MxParams p, int64_t tiles_r, int64_t tiles_c, uint32_t* status) {
  run_tile_pipeline<MxOp<ROW, COL, MODE>>(&tmap, p, tiles_r, tiles_c, status);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <bool ROW, bool COL, int MODE>
static int launch_mx(const CUtensorMap& map, const MxParams& p, uint32_t* status, cudaStream_t stream) {
  const int cap = tile_resident_ctas<k_mxfp8<ROW, COL, MODE>>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  k_mxfp8<ROW, COL, MODE><<<grid, kTileThreads, kTileSmemBytes, stream>>>(map, p, tiles_r, tiles_c, status);
  return check_launch();
}

template <int MODE>
static int launch_mx_mode(bool row, bool col, const CUtensorMap& map, const MxParams& p, uint32_t* status,
                          cudaStream_t stream) {
  if (row && col) return launch_mx<true, true, MODE>(map, p, status, stream);
  if (row) return launch_mx<true, false, MODE>(map, p, status, stream);
  return launch_mx<false, true, MODE>(map, p, status, stream);
}

extern "C" int tnq_mxfp8_quantize(const void* x, int64_t rows, int64_t cols, int in_dtype, void* q_row,
                                  void* sf_row, void* q_col, void* sf_col, int e8m0_mode, int scale_layout,
                                  uint32_t* status, tnq_stream_t stream) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16) return TNQ_EUNSUPPORTED;
  if (e8m0_mode != TNQ_E8M0_CEIL && e8m0_mode != TNQ_E8M0_FLOOR) return TNQ_EINVAL;
  if (scale_layout != TNQ_SCALES_RAW && scale_layout != TNQ_SCALES_SWIZZLED) return TNQ_EINVAL;
  const bool row = q_row != nullptr, col = q_col != nullptr;
  if (!row && !col) return TNQ_EINVAL;
  if ((row && !sf_row) || (col && !sf_col)) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (x == nullptr) return TNQ_EINVAL;
  if (cols % 8 != 0) return TNQ_ESHAPE;  // TMA row pitch must be a multiple of 16 bytes
  if (row && cols % 32 != 0) return TNQ_ESHAPE;
  if (col && rows % 32 != 0) return TNQ_ESHAPE;
  if (rows > 0x7fffffff || cols > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (!aligned16(x) || (row && (!aligned16(q_row) || !aligned16(sf_row))) ||
      (col && (!aligned16(q_col) || !aligned16(sf_col))))
    return TNQ_EALIGN;
  CUtensorMap map;
  int rc = make_tile_map(&map, x, rows, cols);
  if (rc != TNQ_OK) return rc;
  MxParams p;
  p.rows = rows, p.cols = cols;
  p.q_row = static_cast<uint8_t*>(q_row), p.sf_row = static_cast<uint8_t*>(sf_row);
  p.q_col = static_cast<uint8_t*>(q_col), p.sf_col = static_cast<uint8_t*>(sf_col);
  p.layout = scale_layout;
  p.sf_row_w = cols / 32, p.sf_col_w = rows / 32;
  if (e8m0_mode == TNQ_E8M0_CEIL) return launch_mx_mode<TNQ_E8M0_CEIL>(row, col, map, p, status, stream);
  return launch_mx_mode<TNQ_E8M0_FLOOR>(row, col, map, p, status, stream);
}
