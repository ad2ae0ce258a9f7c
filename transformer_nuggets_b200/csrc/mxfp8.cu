// MXFP8 quantizer: 32-element blocks, E8M0 scale byte, e4m3 payload; row-wise
// (blocks along the row) and column-wise (blocks along the column, stored
// transposed) outputs from ONE read of the input.
//
// A 128x128 tile staged in shared memory by TMA is consumed by two groups of warps
// at the same time.  Row pass (warps 0-7): four adjacent lanes own one 32-element
// block - conflict-free 16-byte shared loads, two shuffles for the block amax,
// 8-byte coalesced stores.  Column pass (warps 8-15): a thread owns two adjacent
// columns over 32 rows - conflict-free 4-byte shared loads, one 32-byte store per
// column.  One tile yields exactly one 512-byte atom of the swizzled 128x4 scale
// layout per direction; it is assembled in shared memory and leaves as 16-byte stores.
//
// The kernel is kept off the instruction-issue limit: |x| maxima and the power-of-two
// scaling run on packed bf16 pairs (abs/max.bf16x2, mul.bf16x2 - exact for a power of
// two), and only the final widening feeds cvt.rn.satfinite.e4m3x2.f32.
//
// Exponent rule on the bf16 amax bits m (15-bit magnitude): with
//   ceil : E' = (m + 0x1f) >> 7     (biased exponent, +1 when the mantissa is above 1.75)
//   floor: E' = m >> 7
// the stored byte is max(E' - 8, 1) (= clamp(e, -126, ..) + 127) and the multiplier
// 2^-e has the bf16 bits (254 - byte) << 7.  ceil equals ceil(log2(amax / 448)) and
// floor equals floor(log2(amax)) - 8 for every finite bf16 amax.
// A block that contains NaN or infinity is outside the contract (payload bytes are
// whatever the hardware cvt gives; the scale byte comes from the exponent rule).
#include <atomic>

#include "mx_scale.cuh"
#include "tile_pipeline.cuh"

#ifndef TNQ_MX_MIXED_FMA
#define TNQ_MX_MIXED_FMA 1
#endif

namespace tnq {


constexpr bool g_mixed_fma = TNQ_MX_MIXED_FMA != 0;

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

// Row pass by NW warps (warp index `warp` in 0..NW-1).  tile / sf_row are shared-space addresses.
template <int MODE, int NW, bool FULL>
__device__ __forceinline__ void mx_row_pass(const MxParams& p, uint32_t tile, uint32_t sf_row, uint32_t tr, uint32_t tc,
                                            int warp, int lane) {
  constexpr int R = kTileRows / NW;  // rows per warp, two per step
  const int chunk = lane & 15;
  const int r0 = warp * R + (lane >> 4);
  const uint32_t src = tile + r0 * 256 + chunk * 16;
  const int64_t grow0 = (int64_t)tr * kTileRows + r0, gcol = (int64_t)tc * kTileCols + chunk * 8;
  uint8_t* dst = p.q_row + grow0 * p.cols + gcol;
  const int64_t dstep = 2 * p.cols;
  const bool col_ok = FULL || gcol < p.cols;
  const bool sf_lane = (lane & 3) == 0;
  const uint32_t sf_dst = sf_row + (r0 & 31) * 16 + (r0 >> 5) * 4 + (chunk >> 2);  // row r0 + 2*it: + it*32 (R <= 16)
  static_for<R / 2>([&](auto I) {
    constexpr int it = decltype(I)::value;
    const uint4 v = lds128_at<it * 512>(src);
    // max of magnitudes in one instruction per word (the sign bits of the result are meaningless)
    uint32_t m = absmax_pk_bf16(absmax_pk_bf16(v.x, v.y), absmax_pk_bf16(v.z, v.w));
    m = absmax_pk_bf16(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = absmax_pk_bf16(m, __shfl_xor_sync(0xffffffffu, m, 2));
    uint32_t byte, s2;
    e8m0_from_amax<MODE>(fold_u16x2(m & 0x7fff7fffu), byte, s2);
    uint2 o;
    if (g_mixed_fma) {
      o.x = e4m3x4_scaled(v.x, v.y, (uint16_t)s2);
      o.y = e4m3x4_scaled(v.z, v.w, (uint16_t)s2);
    } else {
      o.x = e4m3x4_from_pk(mul_pk_bf16(v.x, s2), mul_pk_bf16(v.y, s2));
      o.y = e4m3x4_from_pk(mul_pk_bf16(v.z, s2), mul_pk_bf16(v.w, s2));
    }
    if constexpr (FULL) {
      stg64(dst, o);
      if (sf_lane) sts8_at<it * 32>(sf_dst, byte);
    } else {
      const bool ok = col_ok && grow0 + 2 * it < p.rows;
      if (ok) stg64(dst, o);
      if (sf_lane) sts8_at<it * 32>(sf_dst, ok ? byte : 0u);
    }
    dst += dstep;
  });
}

// Column pass by 256 threads (t in 0..255): columns 2w, 2w+1 and rows rb*32..rb*32+31.
// Computes the 32 payload bytes of each of the two columns (lo / hi) and stages the two scale bytes.
template <int MODE>
__device__ __forceinline__ void mx_col_compute(uint32_t tile, uint32_t sf_col, int t, bool ok, uint32_t (&lo)[8],
                                               uint32_t (&hi)[8]) {
  const int w = t & 63, rb = t >> 6;
  const uint32_t src = tile + rb * 32 * 256 + w * 4;
  uint32_t v[32];
  uint32_t m = 0;
  static_for<32>([&](auto I) {
    constexpr int i = decltype(I)::value;
    v[i] = lds32_at<i * 256>(src);
    m = absmax_pk_bf16(m, v[i]);  // one instruction; sign bits of m are meaningless
  });
  uint32_t byte_lo, byte_hi, s_lo, s_hi;
  e8m0_from_amax<MODE>(m & 0x7fffu, byte_lo, s_lo);
  e8m0_from_amax<MODE>((m >> 16) & 0x7fffu, byte_hi, s_hi);
  if (g_mixed_fma) {
    const uint16_t m_lo = (uint16_t)s_lo, m_hi = (uint16_t)s_hi;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a0, a1, a2, a3, b0, b1, b2, b3;
      widen_scale_pk2(v[4 * j], m_lo, m_hi, a0, b0);
      widen_scale_pk2(v[4 * j + 1], m_lo, m_hi, a1, b1);
      widen_scale_pk2(v[4 * j + 2], m_lo, m_hi, a2, b2);
      widen_scale_pk2(v[4 * j + 3], m_lo, m_hi, a3, b3);
      lo[j] = cvt_fp8x4<TNQ_FP8_E4M3>(a0, a1, a2, a3);
      hi[j] = cvt_fp8x4<TNQ_FP8_E4M3>(b0, b1, b2, b3);
    }
  } else {
    const uint32_t s2 = __byte_perm(s_lo, s_hi, 0x7610);  // low half from s_lo, high half from s_hi
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = mul_pk_bf16(v[i], s2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      lo[j] = cvt_fp8x4<TNQ_FP8_E4M3>(bf16lo(v[4 * j]), bf16lo(v[4 * j + 1]), bf16lo(v[4 * j + 2]), bf16lo(v[4 * j + 3]));
      hi[j] = cvt_fp8x4<TNQ_FP8_E4M3>(bf16hi(v[4 * j]), bf16hi(v[4 * j + 1]), bf16hi(v[4 * j + 2]), bf16hi(v[4 * j + 3]));
    }
  }
  // columns c0 = 2w, c1 = 2w + 1: (c & 31) * 16 + (c >> 5) * 4 + rb
  const uint32_t sf0 = sf_col + ((2 * w) & 31) * 16 + (w >> 4) * 4 + rb;
  sts8(sf0, ok ? byte_lo : 0u);
  sts8(sf0 + 16, ok ? byte_hi : 0u);
}

template <int MODE, bool FULL>
__device__ __forceinline__ void mx_col_pass(const MxParams& p, uint32_t tile, uint32_t sf_col, uint32_t tr, uint32_t tc,
                                            int t) {
  const int w = t & 63, rb = t >> 6;
  const int64_t c = (int64_t)tc * kTileCols + 2 * w;
  const int64_t r0 = (int64_t)tr * kTileRows + rb * 32;
  const bool ok = FULL || (c < p.cols && r0 < p.rows);
  uint32_t lo[8], hi[8];
  mx_col_compute<MODE>(tile, sf_col, t, ok, lo, hi);
  if (ok) {
    uint8_t* d0 = p.q_col + c * p.rows + r0;
    stg256(d0, lo[0], lo[1], lo[2], lo[3], lo[4], lo[5], lo[6], lo[7]);
    stg256(d0 + p.rows, hi[0], hi[1], hi[2], hi[3], hi[4], hi[5], hi[6], hi[7]);
  }
}

template <bool ROW, bool COL, int MODE>
struct MxOp {
  using Params = MxParams;
  // row + column: warps 0-7 row pass, warps 8-15 column pass; row only: 16 warps on the
  // row pass; column only: 8 warps
  static constexpr int kThreads = ROW ? 512 : 256;

  struct State {};
  __device__ static __forceinline__ State init(const Params&) { return State{}; }

  template <bool FULL>
  __device__ static __forceinline__ void process(const Params& p, const State&, uint32_t tile, uint32_t sf, uint32_t tr,
                                                 uint32_t tc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if constexpr (ROW && COL) {
      if (warp < 8) mx_row_pass<MODE, 8, FULL>(p, tile, sf, tr, tc, warp, lane);
      else mx_col_pass<MODE, FULL>(p, tile, sf + 512, tr, tc, (int)threadIdx.x - 256);
    } else if constexpr (ROW) {
      mx_row_pass<MODE, 16, FULL>(p, tile, sf, tr, tc, warp, lane);
    } else {
      mx_col_pass<MODE, FULL>(p, tile, sf + 512, tr, tc, (int)threadIdx.x);
    }
  }

  // One swizzled atom (scale rows ar*128.., scale columns ac*4.. of an [R, W] scale matrix) from
  // shared memory to its place: whole atom when swizzled (32 threads starting at t0), else row-major.
  // `t0`: first of the threads that take part (32 of them for the swizzled copy, `span` for raw).
  __device__ static __forceinline__ void flush_one(uint32_t atom, uint8_t* dst, int layout, int64_t R, int64_t W,
                                                   int64_t ar, int64_t ac, int t0, int span) {
    const int t = (int)threadIdx.x - t0;
    if (layout == TNQ_SCALES_SWIZZLED) {
      const int64_t ncb = (W + 3) / 4;
      if (t >= 0 && t < 32) stg128(dst + (ar * ncb + ac) * 512 + t * 16, lds128(atom + t * 16));
    } else {
      if (t < 0 || t >= span) return;
      for (int idx = t; idx < 128; idx += span) {  // one scale-matrix row (4 bytes) per thread
        const int64_t gr = ar * 128 + idx;
        if (gr >= R) continue;
        const uint32_t four = lds32(atom + (idx & 31) * 16 + (idx >> 5) * 4);
        for (int c = 0; c < 4; ++c)
          if (ac * 4 + c < W) dst[gr * W + ac * 4 + c] = (uint8_t)(four >> (8 * c));
      }
    }
  }

  __device__ static __forceinline__ void finish(const Params&, const State&) {}

  __device__ static __forceinline__ void flush(const Params& p, uint32_t sf, uint32_t tr, uint32_t tc) {
    if constexpr (ROW) flush_one(sf, p.sf_row, p.layout, p.rows, p.sf_row_w, tr, tc, 0, kThreads);
    if constexpr (COL) flush_one(sf + 512, p.sf_col, p.layout, p.cols, p.sf_col_w, tc, tr, 0, kThreads);
  }
};

// Row + column outputs with the two passes decoupled: warps 0-7 (row pass) and warps
// 8-15 (column pass) each walk the tile sequence at their own pace.  A group waits only
// for the tile's data (mbarrier) and for its own members (named barrier); whichever
// group finishes a stage second re-arms it and issues the next TMA load into it.
template <int MODE>
__global__ void __launch_bounds__(512, 2)
    k_mxfp8_dual(const __grid_constant__ CUtensorMap tmap, MxParams p, uint32_t tiles_r, uint32_t tiles_c, uint32_t* status) {
  extern __shared__ uint8_t tnq_dyn_smem[];
  uint8_t* const base = tile_smem_base(tnq_dyn_smem);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base + kStages * kTileBytes);       // kStages x 8 bytes
  uint32_t* const done = reinterpret_cast<uint32_t*>(base + kStages * kTileBytes + 32);  // kStages x 4 bytes
  const uint32_t tile0 = smem_u32(base);
  const uint32_t sf0 = tile0 + kStages * kTileBytes + 64;  // row atoms at +0 / +512, column atoms at +1024 / +1536
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
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  // every thread keeps `ahead` kStages tiles in front of `cur`; thread 0 also issues the first loads
  for (uint32_t s = 0; s < (uint32_t)kStages; ++s) {
    if (threadIdx.x == 0 && s < count) issue(s);
    ahead.advance();
  }

  uint32_t s = 0, phase = 0;
  for (uint32_t k = 0; k < count; ++k) {
    if (!mbar_wait(&bars[s], phase)) {
      if (gtid == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      return;
    }
    const uint32_t tile = tile0 + s * kTileBytes;
    const uint32_t sf = sf0 + (uint32_t)group * 1024u + (k & 1u) * 512u;
    const bool full = (int64_t)(cur.tr + 1) * kTileRows <= p.rows && (int64_t)(cur.tc + 1) * kTileCols <= p.cols;
    if (group == 0) {
      if (full) mx_row_pass<MODE, 8, true>(p, tile, sf, cur.tr, cur.tc, gtid >> 5, gtid & 31);
      else mx_row_pass<MODE, 8, false>(p, tile, sf, cur.tr, cur.tc, gtid >> 5, gtid & 31);
    } else {
      if (full) mx_col_pass<MODE, true>(p, tile, sf, cur.tr, cur.tc, gtid);
      else mx_col_pass<MODE, false>(p, tile, sf, cur.tr, cur.tc, gtid);
    }
    // the group is done with the tile and its scale atom is staged
    if (group == 0) named_barrier<1, 256>();
    else named_barrier<2, 256>();
    if (gtid == 0) {
      __threadfence_block();
      if (atomicAdd(&done[s], 1u) == 1u) {  // the other group released the stage earlier: reuse it
        atomicExch(&done[s], 0u);
        if (k + kStages < count) issue(s);  // `ahead` is the tile kStages after `cur`
      }
    }
    if (group == 0) MxOp<true, true, MODE>::flush_one(sf, p.sf_row, p.layout, p.rows, p.sf_row_w, cur.tr, cur.tc, 0, 512);
    else MxOp<true, true, MODE>::flush_one(sf, p.sf_col, p.layout, p.cols, p.sf_col_w, cur.tc, cur.tr, 256, 512);
    cur.advance();
    ahead.advance();
    if (++s == (uint32_t)kStages) s = 0, phase ^= 1u;
  }
}

// Row + column outputs with the transposed payload staged in shared memory and written by TMA
// stores: every q_col row receives its 128 bytes of a tile as one full line from the copy engine
// instead of four 32-byte pieces from four warps (49.6 -> 46.2 us at 8192 x 7168).  Two input
// stages: the staging tile takes the third stage's room so that two CTAs still fit on an SM.
// The two groups stay decoupled; the column group's elected thread issues its stores and waits
// until they have read the staging tile before the next tile overwrites it.  `tuning` bit 0: the
// input tiles are loaded with an L2 evict-first policy (they are never read again: 46.2 ->
// 45.1 us); bit 1: the stored lines carry the same policy (no gain measured).
template <int MODE>
__global__ void __launch_bounds__(512, 2)
    k_mxfp8_dual_ts(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap map_col, MxParams p,
                    uint32_t tiles_r, uint32_t tiles_c, uint32_t* status, int tuning) {
  extern __shared__ uint8_t tnq_dyn_smem[];
  const uint32_t raw = smem_u32(tnq_dyn_smem);
  uint8_t* const base = tnq_dyn_smem + ((1024u - (raw & 1023u)) & 1023u);
  const uint32_t stg_col = smem_u32(base);  // swizzled: needs the 1 KiB alignment
  uint8_t* const tiles = base + kStageOutBytes;
  const uint32_t tile0 = smem_u32(tiles);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(tiles + kStagesTs * kTileBytes);       // kStagesTs x 8 bytes
  uint32_t* const done = reinterpret_cast<uint32_t*>(tiles + kStagesTs * kTileBytes + 32);  // kStagesTs x 4 bytes
  const uint32_t sf0 = tile0 + kStagesTs * kTileBytes + 64;  // row atoms at +0 / +512, column atoms at +1024 / +1536
  const uint32_t ntiles = tiles_r * tiles_c;
  const uint32_t first = blockIdx.x;
  const uint32_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;
  const int group = threadIdx.x >> 8, gtid = threadIdx.x & 255;
  const bool hint_ld = (tuning & 1) != 0, hint_st = (tuning & 2) != 0;
  const uint64_t pol = l2_policy_evict_first();

  TileCursor cur, ahead;
  cur.init(first, gridDim.x, tiles_c);
  ahead = cur;
  auto issue = [&](uint32_t s) {  // one thread: arm stage s and load the tile at `ahead` into it
    mbar_expect_tx(&bars[s], kTileBytes);
    const int32_t x = (int32_t)(ahead.tc * kTileCols), y = (int32_t)(ahead.tr * kTileRows);
    if (hint_ld) tma_load_2d_hint(tiles + s * kTileBytes, &tmap, x, y, &bars[s], pol);
    else tma_load_2d(tiles + s * kTileBytes, &tmap, x, y, &bars[s]);
  };
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap);
    prefetch_tmap(&map_col);
    for (int s = 0; s < kStagesTs; ++s) {
      mbar_init(&bars[s], 1);
      done[s] = 0;
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (uint32_t s = 0; s < (uint32_t)kStagesTs; ++s) {
    if (threadIdx.x == 0 && s < count) issue(s);
    ahead.advance();
  }

  uint32_t s = 0, phase = 0;
  for (uint32_t k = 0; k < count; ++k) {
    if (!mbar_wait(&bars[s], phase)) {
      if (gtid == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      break;
    }
    const uint32_t tile = tile0 + s * kTileBytes;
    const uint32_t sf = sf0 + (uint32_t)group * 1024u + (k & 1u) * 512u;
    const bool full = (int64_t)(cur.tr + 1) * kTileRows <= p.rows && (int64_t)(cur.tc + 1) * kTileCols <= p.cols;
    auto release_stage = [&]() {  // gtid == 0, after the group's barrier: the group no longer reads the tile
      __threadfence_block();
      if (atomicAdd(&done[s], 1u) == 1u) {  // the other group released the stage earlier: reuse it
        atomicExch(&done[s], 0u);
        if (k + kStagesTs < count) issue(s);  // `ahead` is the tile kStagesTs after `cur`
      }
    };
    if (group == 0) {
      if (full) mx_row_pass<MODE, 8, true>(p, tile, sf, cur.tr, cur.tc, gtid >> 5, gtid & 31);
      else mx_row_pass<MODE, 8, false>(p, tile, sf, cur.tr, cur.tc, gtid >> 5, gtid & 31);
      named_barrier<1, 256>();
      if (gtid == 0) release_stage();
      MxOp<true, true, MODE>::flush_one(sf, p.sf_row, p.layout, p.rows, p.sf_row_w, cur.tr, cur.tc, 0, 512);
    } else {
      const int64_t c = (int64_t)cur.tc * kTileCols + 2 * (gtid & 63);
      const int64_t r0 = (int64_t)cur.tr * kTileRows + (gtid >> 6) * 32;
      const bool ok = full || (c < p.cols && r0 < p.rows);
      uint32_t lo[8], hi[8];
      mx_col_compute<MODE>(tile, sf, gtid, ok, lo, hi);
      if (gtid == 0) bulk_group_wait_read();  // the previous tile's store has read the staging tile
      named_barrier<2, 256>();                // everyone has its columns in registers; the staging tile is free
      if (gtid == 0) release_stage();
      stage_transposed(stg_col, gtid, lo, hi);
      fence_proxy_async();
      named_barrier<3, 256>();
      if (gtid == 0) {  // the part of the box outside the matrix is clipped by the copy engine
        const int32_t x = (int32_t)(cur.tr * kTileRows), y = (int32_t)(cur.tc * kTileCols);
        if (hint_st) tma_store_2d_hint(&map_col, stg_col, x, y, pol);
        else tma_store_2d(&map_col, stg_col, x, y);
        bulk_group_commit();
      }
      MxOp<true, true, MODE>::flush_one(sf, p.sf_col, p.layout, p.cols, p.sf_col_w, cur.tc, cur.tr, 256, 512);
    }
    cur.advance();
    ahead.advance();
    if (++s == (uint32_t)kStagesTs) s = 0, phase ^= 1u;
  }
  if (gtid == 0) bulk_group_wait();  // shared memory must outlive the stores that read it
}

template <bool ROW, bool COL, int MODE>
__global__ void __launch_bounds__((MxOp<ROW, COL, MODE>::kThreads), 2)
    k_mxfp8(const __grid_constant__ CUtensorMap tmap, MxParams p, uint32_t tiles_r, uint32_t tiles_c, uint32_t* status,
            int evict_first) {
  run_tile_pipeline<MxOp<ROW, COL, MODE>>(&tmap, p, tiles_r, tiles_c, status, evict_first != 0);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <bool ROW, bool COL, int MODE>
static int launch_mx(const CUtensorMap& map, const MxParams& p, uint32_t* status, cudaStream_t stream) {
  constexpr int kThreads = MxOp<ROW, COL, MODE>::kThreads;
  const int cap = tile_resident_ctas<k_mxfp8<ROW, COL, MODE>, kThreads>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  return launch_chained(k_mxfp8<ROW, COL, MODE>, dim3(grid), dim3(kThreads), kTileSmemBytes, stream, map, p, (uint32_t)tiles_r,
                        (uint32_t)tiles_c, status, tile_loads_evict_first() ? 1 : 0);
}

template <int MODE>
static int launch_mx_dual(const CUtensorMap& map, const MxParams& p, uint32_t* status, cudaStream_t stream) {
  const int cap = tile_resident_ctas<k_mxfp8_dual<MODE>, 512>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  return launch_chained(k_mxfp8_dual<MODE>, dim3(grid), dim3(512), kTileSmemBytes, stream, map, p, (uint32_t)tiles_r,
                        (uint32_t)tiles_c, status);
}

// variant: 0 = both passes store straight to global memory, 1 = transposed payload through shared
// memory + TMA stores; tuning: L2 policy bits of the TMA-store kernel (see k_mxfp8_dual_ts)
static std::atomic<int> g_mx_store_variant{1};
static std::atomic<int> g_mx_tuning{1};
extern "C" int tnq_mxfp8_set_store_variant(int v) {
  const int variant = v & 3, tuning = v >> 2;
  if (v < 0 || variant > 1 || tuning > 3) return TNQ_EINVAL;
  g_mx_store_variant.store(variant, std::memory_order_relaxed);
  g_mx_tuning.store(tuning, std::memory_order_relaxed);
  return TNQ_OK;
}

template <int MODE>
static int launch_mx_dual_ts(const CUtensorMap& map, const MxParams& p, uint32_t* status, cudaStream_t stream) {
  const int cap = resident_ctas_smem<k_mxfp8_dual_ts<MODE>, 512, kTsSmemBytes>();
  if (cap < 1) return cuda_fail(cudaGetLastError());
  CUtensorMap map_col;
  int rc = make_byte_store_map(&map_col, p.q_col, p.cols, p.rows, true);
  if (rc != TNQ_OK) return rc;
  const int64_t tiles_r = (p.rows + kTileRows - 1) / kTileRows, tiles_c = (p.cols + kTileCols - 1) / kTileCols;
  const int64_t ntiles = tiles_r * tiles_c;
  const int grid = (int)(ntiles < cap ? ntiles : cap);
  return launch_chained(k_mxfp8_dual_ts<MODE>, dim3(grid), dim3(512), kTsSmemBytes, stream, map, map_col, p, (uint32_t)tiles_r,
                        (uint32_t)tiles_c, status, g_mx_tuning.load(std::memory_order_relaxed));
}

template <int MODE>
static int launch_mx_mode(bool row, bool col, const CUtensorMap& map, const MxParams& p, uint32_t* status,
                          cudaStream_t stream) {
  if (row && col) {
    // the TMA store needs a 16-byte row pitch of q_col: rows % 32 == 0 holds whenever the column direction is asked for
    if (g_mx_store_variant.load(std::memory_order_relaxed) == 1) return launch_mx_dual_ts<MODE>(map, p, status, stream);
    return launch_mx_dual<MODE>(map, p, status, stream);
  }
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
  if (((rows + 127) / 128) * ((cols + 127) / 128) > 0x7fffffff) return TNQ_EUNSUPPORTED;  // 32-bit tile cursor
  if (!aligned16(x) || (row && (!aligned16(q_row) || !aligned16(sf_row))) ||
      (col && ((reinterpret_cast<uintptr_t>(q_col) & 31u) != 0 || !aligned16(sf_col))))
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
