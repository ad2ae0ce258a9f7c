// Per-tensor scaled FP8 cast that also emits the transposed copy:
//     out[r, c] = fp8(x[r, c] * s)        row-major [rows, cols]
//     out_t[c, r] = out[r, c]             row-major [cols, rows]
// from ONE read of x.  An FP8 training step needs both layouts of the same tensor (the
// forward GEMM contracts over one dimension, the weight-gradient GEMM over the other); done
// separately that is a cast (2 + 1 B/elem) plus a transpose (1 + 1 B/elem), here it is
// 2 + 1 + 1.  Same arithmetic as the plain cast (fp8_tensor.cu): y = f32(x) * s as one fp32
// product, optional saturation, RNE cvt, the CPU cast's NaN / overflow corner cases; the two
// outputs hold identical bytes.  Optional side output: abs_max = max(abs_max, max|x|) for
// delayed scaling.
//
// 128 x 128 bf16 tiles arrive by 2-D TMA into an mbarrier ring.  Two kernels: k_cast_transpose_bt
// (default) converts every element once and transposes the fp8 bytes in shared memory;
// k_cast_transpose (threads 0-255 make the row-major output, threads 256-511 the transposed one, every
// element converted twice, plain global stores) serves the shapes the first cannot take.
#include <atomic>

#include "tile_pipeline.cuh"

namespace tnq {

struct CastTParams {
  int64_t rows, cols;
  const float* scale;
  int scale_kind;
  float* abs_max;  // nullable
  uint8_t* out;
  uint8_t* out_t;
  int t_aligned;  // rows % 32 == 0: every 32-row run of out_t starts on a 32-byte boundary
};

// 16 bytes of bf16 -> 8 bytes of fp8 per thread and row; a warp writes two 128-byte row
// segments.  `m` collects the magnitude bits of everything the thread saw.
template <int OUT, bool SAT, bool FULL>
__device__ __forceinline__ void ct_row_pass(const CastTParams& p, float s, uint32_t& m, uint32_t tile, uint32_t tr,
                                            uint32_t tc, int t) {
  const int piece = t & 15, r_in = t >> 4;
  const int64_t c = (int64_t)tc * kTileCols + piece * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = i * 16 + r_in;
    const int64_t r = (int64_t)tr * kTileRows + row;
    const uint4 v = lds128(tile + row * 256 + piece * 16);  // zeros outside the matrix
    m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m, v.x), v.y), v.z), v.w);
    if (FULL || (r < p.rows && c < p.cols)) stg64(p.out + r * p.cols + c, quant8_bf16<OUT, SAT>(v, s));
  }
}

// A thread owns two adjacent columns over 32 rows: 32 conflict-free 4-byte shared loads -> the 32
// output bytes of each column.
template <int OUT, bool SAT>
__device__ __forceinline__ void ct_col_compute(float s, uint32_t tile, int u, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
  const int w = u & 63, rb = u >> 6;
  const uint32_t src = tile + rb * 32 * 256 + w * 4;
  uint32_t v[32];
  static_for<32>([&](auto I) {
    constexpr int i = decltype(I)::value;
    v[i] = lds32_at<i * 256>(src);
  });
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    lo[j] = quant4<OUT, SAT>(bf16lo(v[4 * j]), bf16lo(v[4 * j + 1]), bf16lo(v[4 * j + 2]), bf16lo(v[4 * j + 3]), s);
    hi[j] = quant4<OUT, SAT>(bf16hi(v[4 * j]), bf16hi(v[4 * j + 1]), bf16hi(v[4 * j + 2]), bf16hi(v[4 * j + 3]), s);
  }
}

// ... and one 32-byte store per column of the transposed output.
template <int OUT, bool SAT, bool FULL>
__device__ __forceinline__ void ct_col_pass(const CastTParams& p, float s, uint32_t tile, uint32_t tr, uint32_t tc,
                                            int u) {
  const int w = u & 63, rb = u >> 6;
  uint32_t lo[8], hi[8];
  ct_col_compute<OUT, SAT>(s, tile, u, lo, hi);
  const int64_t c = (int64_t)tc * kTileCols + 2 * w;
  const int64_t r0 = (int64_t)tr * kTileRows + rb * 32;
  if (FULL || (c < p.cols && r0 < p.rows)) {  // cols is even, so column c + 1 exists with column c
    uint8_t* d0 = p.out_t + c * p.rows + r0;
    if (p.t_aligned && (FULL || r0 + 32 <= p.rows)) {
      stg256(d0, lo[0], lo[1], lo[2], lo[3], lo[4], lo[5], lo[6], lo[7]);
      stg256(d0 + p.rows, hi[0], hi[1], hi[2], hi[3], hi[4], hi[5], hi[6], hi[7]);
    } else {  // ragged or unaligned rows: byte stores
      const int nr = (int)min((int64_t)32, p.rows - r0);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < nr) {
          d0[i] = (uint8_t)(lo[i >> 2] >> (8 * (i & 3)));
          d0[p.rows + i] = (uint8_t)(hi[i >> 2] >> (8 * (i & 3)));
        }
      }
    }
  }
}

// The two groups walk the tile sequence at their own pace (as in the MXFP8 row + column
// kernel): a group waits only for the tile's mbarrier and for its own members (named
// barrier); whichever group releases a stage second re-arms it and issues the next load.
template <int OUT, bool SAT>
__global__ void __launch_bounds__(512, 2)
    k_cast_transpose(const __grid_constant__ CUtensorMap tmap, CastTParams p, uint32_t tiles_r, uint32_t tiles_c,
                     uint32_t* status) {
  extern __shared__ uint8_t tnq_dyn_smem[];
  uint8_t* const base = tile_smem_base(tnq_dyn_smem);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base + kStages * kTileBytes);       // kStages x 8 bytes
  uint32_t* const done = reinterpret_cast<uint32_t*>(base + kStages * kTileBytes + 32);  // kStages x 4 bytes
  uint32_t* const cta_max = done + kStages;                                              // one word
  const uint32_t tile0 = smem_u32(base);
  const uint32_t ntiles = tiles_r * tiles_c;
  const uint32_t first = blockIdx.x;
  const uint32_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;
  const int group = threadIdx.x >> 8, gtid = threadIdx.x & 255;

  TileCursor cur, ahead;
  cur.init(first, gridDim.x, tiles_c);
  ahead = cur;
  auto issue = [&](uint32_t s) {  // one thread: arm stage s and load the tile at `ahead` into it
    mbar_expect_tx(&bars[s], kTileBytes);
    tma_load_2d(base + s * kTileBytes, &tmap, (int32_t)(ahead.tc * kTileCols), (int32_t)(ahead.tr * kTileRows), &bars[s]);
  };
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars[s], 1);
      done[s] = 0;
    }
    *cta_max = 0;
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {  // every thread keeps `ahead` kStages tiles in front of `cur`
    if (threadIdx.x == 0 && s < count) issue(s);
    ahead.advance();
  }
  const float v = *p.scale;
  const float scale = p.scale_kind == TNQ_SCALE_IS_AMAX ? scale_from_amax(v, Fp8Traits<OUT>::kMax) : v;
  uint32_t m = 0;

  uint32_t s = 0, phase = 0;
  for (uint32_t k = 0; k < count; ++k) {
    if (!mbar_wait(&bars[s], phase)) {
      if (gtid == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      return;
    }
    const uint32_t tile = tile0 + s * kTileBytes;
    const bool full = (int64_t)(cur.tr + 1) * kTileRows <= p.rows && (int64_t)(cur.tc + 1) * kTileCols <= p.cols;
    if (group == 0) {
      if (full) ct_row_pass<OUT, SAT, true>(p, scale, m, tile, cur.tr, cur.tc, gtid);
      else ct_row_pass<OUT, SAT, false>(p, scale, m, tile, cur.tr, cur.tc, gtid);
      named_barrier<1, 256>();
    } else {
      if (full) ct_col_pass<OUT, SAT, true>(p, scale, tile, cur.tr, cur.tc, gtid);
      else ct_col_pass<OUT, SAT, false>(p, scale, tile, cur.tr, cur.tc, gtid);
      named_barrier<2, 256>();
    }
    if (gtid == 0) {
      __threadfence_block();
      if (atomicAdd(&done[s], 1u) == 1u) {  // the other group released the stage earlier: reuse it
        atomicExch(&done[s], 0u);
        if (k + kStages < count) issue(s);  // `ahead` is the tile kStages after `cur`
      }
    }
    cur.advance();
    ahead.advance();
    if (++s == (uint32_t)kStages) s = 0, phase ^= 1u;
  }
  // max|x| of everything the row group saw -> abs_max.  Signed compare of the bit patterns:
  // non-negative floats order like their bits with NaN on top, and a negative old value
  // (callers start from -1.0) loses to any magnitude
  if (p.abs_max != nullptr && group == 0) {
    const uint32_t wm = warp_max_u32(fold_u16x2(m));
    if ((gtid & 31) == 0 && wm != 0u) atomicMax(cta_max, wm);
    named_barrier<1, 256>();
    if (gtid == 0) atomicMax(reinterpret_cast<int*>(p.abs_max), (int)(*cta_max << 16));
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <int OUT, bool SAT>
static int launch_cast_transpose(const CUtensorMap& map, const CastTParams& p, uint32_t* status, cudaStream_t stream) {
  const int cap = tile_resident_ctas<k_cast_transpose<OUT, SAT>, 512>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  return launch_chained(k_cast_transpose<OUT, SAT>, dim3(grid), dim3(512), kTileSmemBytes, stream, map, p, (uint32_t)tiles_r,
                        (uint32_t)tiles_c, status);
}

namespace tnq {

// The same result with every element converted ONCE: all 512 threads convert the tile row-major
// (8 fp8 bytes per thread and row: stored to `out` and, XOR-swizzled, into a 128 x 128-byte fp8 tile in
// shared memory), then all 512 threads transpose that tile in 4 x 4-byte squares - four conflict-free
// 4-byte shared loads, eight byte permutes, four conflict-free 4-byte stores into the staging tile that
// one TMA store (128-byte swizzle) sends to out_t, so that every out_t row receives a full 128-byte
// line.  Input tiles are loaded with an L2 evict-first policy.  16384 x 8192: 101.7 us against 112.9 -
// 115.6 us for the kernel above (converting twice with a staged TMA store for out_t: 104.0 - 105.3 us).
// Needs a 16-byte row pitch of out_t (rows % 16 == 0).  The dynamic shared memory is declared 1 KiB
// aligned (the swizzle needs that); the kernel checks it and refuses to run otherwise.
// Shared memory: [transposed staging 16 KiB][fp8 tile 16 KiB][2 input stages][barriers].
constexpr int kBtStages = 2;
constexpr int kBtSmemBytes = 2 * kStageOutBytes + kBtStages * kTileBytes + 64;

template <int OUT, bool SAT>
__global__ void __launch_bounds__(512, 2)
    k_cast_transpose_bt(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap map_col, CastTParams p,
                        uint32_t tiles_r, uint32_t tiles_c, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t tnq_dyn_smem_1k[];
  uint8_t* const base = tnq_dyn_smem_1k;
  const uint32_t stg_t = smem_u32(base);  // transposed staging, read by the TMA store
  if ((stg_t & 1023u) != 0u) {            // never seen; a misplaced staging tile would scramble out_t silently
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_EALIGN);
    return;
  }
  const uint32_t stg_q = stg_t + kStageOutBytes;  // row-major fp8 tile, word w of row r at word w ^ (r >> 2)
  uint8_t* const tiles = base + 2 * kStageOutBytes;
  const uint32_t tile0 = smem_u32(tiles);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(tiles + kBtStages * kTileBytes);
  uint32_t* const cta_max = reinterpret_cast<uint32_t*>(tiles + kBtStages * kTileBytes + 32);
  const uint32_t ntiles = tiles_r * tiles_c;
  const uint32_t first = blockIdx.x;
  const uint32_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint64_t pol = l2_policy_evict_first();

  TileCursor cur, ahead;
  cur.init(first, gridDim.x, tiles_c);
  ahead = cur;
  auto issue = [&](uint32_t s) {
    mbar_expect_tx(&bars[s], kTileBytes);
    tma_load_2d_hint(tiles + s * kTileBytes, &tmap, (int32_t)(ahead.tc * kTileCols), (int32_t)(ahead.tr * kTileRows), &bars[s], pol);
  };
  if (t == 0) {
    prefetch_tmap(&tmap);
    prefetch_tmap(&map_col);
    for (int s = 0; s < kBtStages; ++s) mbar_init(&bars[s], 1);
    *cta_max = 0;
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (uint32_t s = 0; s < (uint32_t)kBtStages; ++s) {
    if (t == 0 && s < count) issue(s);
    ahead.advance();
  }
  const float v = *p.scale;
  const float scale = p.scale_kind == TNQ_SCALE_IS_AMAX ? scale_from_amax(v, Fp8Traits<OUT>::kMax) : v;
  uint32_t m = 0;

  // conversion: thread = 16-byte piece `piece` of rows r_in, r_in + 32, r_in + 64, r_in + 96
  const int piece = t & 15, r_in = t >> 4;
  // transposition: lane = group of four rows, warp = two groups of four columns
  const int rg = lane;

  uint32_t s = 0, phase = 0;
  for (uint32_t k = 0; k < count; ++k) {
    if (!mbar_wait(&bars[s], phase)) {
      if (t == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      break;
    }
    const uint32_t tile = tile0 + s * kTileBytes;
    const bool full = (int64_t)(cur.tr + 1) * kTileRows <= p.rows && (int64_t)(cur.tc + 1) * kTileCols <= p.cols;
    const int64_t c = (int64_t)cur.tc * kTileCols + piece * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = i * 32 + r_in;
      const int64_t r = (int64_t)cur.tr * kTileRows + row;
      const uint4 q = lds128(tile + row * 256 + piece * 16);  // zeros outside the matrix
      m = absmax_bf16x2_1op(absmax_bf16x2_1op(absmax_bf16x2_1op(absmax_bf16x2_1op(m, q.x), q.y), q.z), q.w);
      const uint2 o = quant8_bf16<OUT, SAT>(q, scale);
      if (full || (r < p.rows && c < p.cols)) stg64(p.out + r * p.cols + c, o);
      // words 2 piece, 2 piece + 1 of the row go to word positions (2 piece) ^ g and (2 piece + 1) ^ g, g = row >> 2:
      // the same aligned pair with g's low bit cleared, the two words swapped when g is odd
      const uint32_t g = (uint32_t)row >> 2;
      const uint32_t dst = stg_q + row * 128 + 4 * ((2 * piece) ^ (g & ~1u));
      const bool swap = (g & 1u) != 0;
      asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(dst), "r"(swap ? o.y : o.x), "r"(swap ? o.x : o.y) : "memory");
    }
    if (t == 0) bulk_group_wait_read();  // the previous tile's store has read the transposed staging tile
    __syncthreads();                     // tile converted: its stage is free, the fp8 tile is complete
    if (t == 0 && k + kBtStages < count) issue(s);  // `ahead` is the tile kBtStages after `cur`
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t cg = 2 * warp + h;  // columns 4 cg .. 4 cg + 3
      const uint32_t src = stg_q + (4 * rg) * 128 + 4 * (cg ^ (uint32_t)rg);
      const uint32_t a = lds32(src), b = lds32(src + 128), c4 = lds32(src + 256), d = lds32(src + 384);
      const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c4, d, 0x5140);
      const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c4, d, 0x7362);
      const uint32_t o[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632), __byte_perm(t2, t3, 0x5410),
                             __byte_perm(t2, t3, 0x7632)};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // column 4 cg + kk, rows 4 rg .. 4 rg + 3: chunk rg >> 2, swizzled by the column
        const uint32_t col = 4 * cg + kk;
        const uint32_t dst = stg_t + col * 128 + ((((uint32_t)rg >> 2) ^ (col & 7u)) << 4) + 4 * ((uint32_t)rg & 3u);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst), "r"(o[kk]) : "memory");
      }
    }
    fence_proxy_async();
    __syncthreads();  // transposed tile complete (and the fp8 tile may be overwritten by the next conversion)
    if (t == 0) {     // the part of the box outside the matrix is clipped by the copy engine
      tma_store_2d(&map_col, stg_t, (int32_t)(cur.tr * kTileRows), (int32_t)(cur.tc * kTileCols));
      bulk_group_commit();
    }
    cur.advance();
    ahead.advance();
    if (++s == (uint32_t)kBtStages) s = 0, phase ^= 1u;
  }
  if (t == 0) bulk_group_wait();  // shared memory must outlive the stores that read it
  if (p.abs_max != nullptr) {
    const uint32_t wm = warp_max_u32(fold_u16x2(m & 0x7fff7fffu));
    if (lane == 0 && wm != 0u) atomicMax(cta_max, wm);
    __syncthreads();
    if (t == 0) atomicMax(reinterpret_cast<int*>(p.abs_max), (int)(*cta_max << 16));
  }
}

}  // namespace tnq

// variant: 0 = both outputs converted separately and stored straight to global memory (the only path for
// shapes whose out_t row pitch is not a multiple of 16 bytes), 1 (default) = convert once, transpose the
// fp8 bytes in shared memory, TMA store
static std::atomic<int> g_ct_store_variant{1};
extern "C" int tnq_cast_transpose_set_store_variant(int v) {
  if (v < 0 || v > 1) return TNQ_EINVAL;
  g_ct_store_variant.store(v, std::memory_order_relaxed);
  return TNQ_OK;
}

template <int OUT, bool SAT>
static int launch_cast_transpose_bt(const CUtensorMap& map, const CastTParams& p, uint32_t* status, cudaStream_t stream) {
  const int cap = resident_ctas_smem<k_cast_transpose_bt<OUT, SAT>, 512, kBtSmemBytes>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  CUtensorMap map_col;
  int rc = make_byte_store_map(&map_col, p.out_t, p.cols, p.rows, true);
  if (rc != TNQ_OK) return rc;
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  return launch_chained(k_cast_transpose_bt<OUT, SAT>, dim3(grid), dim3(512), kBtSmemBytes, stream, map, map_col, p,
                        (uint32_t)tiles_r, (uint32_t)tiles_c, status);
}

template <int OUT, bool SAT>
static int launch_cast_transpose_any(const CUtensorMap& map, const CastTParams& p, uint32_t* status, cudaStream_t stream) {
  if (g_ct_store_variant.load(std::memory_order_relaxed) == 1 && p.rows % 16 == 0 && aligned16(p.out_t))
    return launch_cast_transpose_bt<OUT, SAT>(map, p, status, stream);
  return launch_cast_transpose<OUT, SAT>(map, p, status, stream);
}

// amax_workspace != null: the dynamic form - an amax pass into that workspace first; the scale is then read from its word 2.
static int cast_transpose(const void* x, int64_t rows, int64_t cols, int in_dtype, int out_dtype, const float* scale,
                          int scale_kind, int saturated, float* abs_max_inout, void* out, void* out_t, uint32_t* status,
                          cudaStream_t stream, void* amax_workspace, float* scale_out) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16) return TNQ_EUNSUPPORTED;
  if (out_dtype != TNQ_FP8_E4M3 && out_dtype != TNQ_FP8_E5M2) return TNQ_EINVAL;
  if (scale_kind != TNQ_SCALE_IS_SCALE && scale_kind != TNQ_SCALE_IS_AMAX) return TNQ_EINVAL;
  if (scale == nullptr) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (x == nullptr || out == nullptr || out_t == nullptr) return TNQ_EINVAL;
  if (cols % 8 != 0) return TNQ_ESHAPE;  // 16-byte row pitch for the tile loads, 8-byte output pieces
  if (rows > 0x7fffffff || cols > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (((rows + 127) / 128) * ((cols + 127) / 128) > 0x7fffffff) return TNQ_EUNSUPPORTED;  // 32-bit tile cursor
  if (!aligned16(x) || !aligned16(out)) return TNQ_EALIGN;
  CUtensorMap map;
  int rc = make_tile_map(&map, x, rows, cols);
  if (rc != TNQ_OK) return rc;
  CastTParams p;
  p.rows = rows, p.cols = cols;
  p.scale = scale, p.scale_kind = scale_kind;
  p.abs_max = abs_max_inout;
  p.out = static_cast<uint8_t*>(out), p.out_t = static_cast<uint8_t*>(out_t);
  p.t_aligned = (rows % 32 == 0) && ((reinterpret_cast<uintptr_t>(out_t) & 31u) == 0);
  if (amax_workspace != nullptr) {
    rc = amax_pass(x, rows * cols, in_dtype, amax_workspace, scale_out, out_dtype == TNQ_FP8_E4M3 ? 448.0f : 57344.0f, stream,
                   false);
    if (rc != TNQ_OK) return rc;
  }
  if (out_dtype == TNQ_FP8_E4M3)
    return saturated ? launch_cast_transpose_any<TNQ_FP8_E4M3, true>(map, p, status, stream)
                     : launch_cast_transpose_any<TNQ_FP8_E4M3, false>(map, p, status, stream);
  return saturated ? launch_cast_transpose_any<TNQ_FP8_E5M2, true>(map, p, status, stream)
                   : launch_cast_transpose_any<TNQ_FP8_E5M2, false>(map, p, status, stream);
}

extern "C" int tnq_fp8_cast_transpose(const void* x, int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                                      const float* scale, int scale_kind, int saturated, float* abs_max_inout,
                                      void* out, void* out_t, uint32_t* status, tnq_stream_t stream) {
  return cast_transpose(x, rows, cols, in_dtype, out_dtype, scale, scale_kind, saturated, abs_max_inout, out, out_t, status,
                        stream, nullptr, nullptr);
}

extern "C" int tnq_fp8_dynamic_cast_transpose(const void* x, int64_t rows, int64_t cols, int in_dtype, int out_dtype,
                                              void* workspace, void* out, void* out_t, float* scale_out,
                                              tnq_stream_t stream) {
  if (workspace == nullptr) return TNQ_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 31u) != 0) return TNQ_EALIGN;  // the amax pass reads 256-bit vectors
  uint32_t* words = static_cast<uint32_t*>(workspace);
  return cast_transpose(x, rows, cols, in_dtype, out_dtype, reinterpret_cast<const float*>(words + 2), TNQ_SCALE_IS_SCALE, 1,
                        nullptr, out, out_t, words + 3, stream, workspace, scale_out);
}
