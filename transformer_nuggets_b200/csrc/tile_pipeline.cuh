// Persistent 128x128 bf16 tile pipeline used by the block-scaled quantizers.
//
// Each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... of a row-major
// [rows, cols] bf16 matrix.  Tiles are brought into shared memory by 2-D TMA loads
// (cp.async.bulk.tensor, cluster size 1, one destination CTA) into a ring of kStages
// buffers, each guarded by an mbarrier; out-of-range parts of edge tiles arrive as
// zeros.  One elected thread issues the loads; all threads of the CTA consume.  A stage is
// re-armed after the __syncthreads that ends the tile that used it, so no "empty"
// barriers are needed.  Every wait is bounded: on expiry the CTA records
// TNQ_ETIMEOUT in the status word and leaves.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace tnq {

constexpr int kTileRows = 128;
constexpr int kTileCols = 128;
constexpr int kTileBytes = kTileRows * kTileCols * 2;  // 32 KiB
constexpr int kStages = 3;
constexpr int kSfBytes = 1024;  // per-tile scale staging (up to two 512-byte atoms)
// ring + alignment slack + barriers + two double-buffered scale staging areas
constexpr int kTileSmemBytes = kStages * kTileBytes + 128 + 64 + 2 * 2 * kSfBytes;

// Shared-memory layout behind a 128-byte aligned base: kStages tiles, kStages
// barriers (64 bytes reserved), two scale staging areas of 2 * kSfBytes each.
__device__ __forceinline__ uint8_t* tile_smem_base(uint8_t* raw) {
  const uint32_t a = smem_u32(raw);
  return raw + ((128u - (a & 127u)) & 127u);
}

// Op::kThreads                                  CTA size
// Op::init(params) -> Op::State                  once per thread, before the first tile
// Op::process<FULL>(params, state, tile, sf, tile_row, tile_col)
//                                                all threads; tile / sf are 32-bit shared-space
//                                                addresses; FULL = the tile lies inside the matrix
// Op::flush(params, sf, tile_row, tile_col)      all threads, after a __syncthreads
// Op::finish(params, state)                      all threads, after the last tile (state is mutable
//                                                across tiles: running maxima live there)
// Position of a CTA in its tile sequence (tiles blockIdx.x, + gridDim.x, ...), advanced
// without divisions: 32-bit tile coordinates, the ring stage and its phase bit.
struct TileCursor {
  uint32_t tr, tc;      // tile row / column
  uint32_t step_r, step_c, tiles_c;
  __device__ __forceinline__ void init(uint32_t first, uint32_t stride, uint32_t tiles_c_) {
    tiles_c = tiles_c_;
    tr = first / tiles_c, tc = first % tiles_c;
    step_r = stride / tiles_c, step_c = stride % tiles_c;
  }
  __device__ __forceinline__ void advance() {
    tc += step_c;
    tr += step_r;
    if (tc >= tiles_c) tc -= tiles_c, ++tr;
  }
};

// `evict_first`: the input tiles are loaded with an L2 evict-first policy (they are read exactly once).
template <class Op>
__device__ __forceinline__ void run_tile_pipeline(const CUtensorMap* tmap, const typename Op::Params& p,
                                                  uint32_t tiles_r, uint32_t tiles_c, uint32_t* status,
                                                  bool evict_first = false) {
  extern __shared__ uint8_t tnq_dyn_smem[];
  uint8_t* const base = tile_smem_base(tnq_dyn_smem);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base + kStages * kTileBytes);
  const uint32_t tile0 = smem_u32(base);
  const uint32_t sf0 = tile0 + kStages * kTileBytes + 64;
  const uint32_t ntiles = tiles_r * tiles_c;
  const uint32_t first = blockIdx.x;
  const uint32_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(tmap);
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  typename Op::State state = Op::init(p);
  TileCursor cur, ahead;  // tile being consumed / next tile to load
  cur.init(first, gridDim.x, tiles_c);
  ahead = cur;
  const uint64_t pol = l2_policy_evict_first();
  auto load = [&](uint32_t s) {  // thread 0: arm stage s and load the tile at `ahead` into it
    mbar_expect_tx(&bars[s], kTileBytes);
    const int32_t x = (int32_t)(ahead.tc * kTileCols), y = (int32_t)(ahead.tr * kTileRows);
    if (evict_first) tma_load_2d_hint(base + s * kTileBytes, tmap, x, y, &bars[s], pol);
    else tma_load_2d(base + s * kTileBytes, tmap, x, y, &bars[s]);
    ahead.advance();
  };
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < (uint32_t)kStages && s < count; ++s) load(s);
  }
  uint32_t s = 0, phase = 0;
  for (uint32_t k = 0; k < count; ++k) {
    if (!mbar_wait(&bars[s], phase)) {
      if (threadIdx.x == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      return;
    }
    const uint32_t sf = sf0 + (k & 1u) * (2 * kSfBytes);
    const uint32_t tile = tile0 + s * kTileBytes;
    const bool full = (int64_t)(cur.tr + 1) * kTileRows <= p.rows && (int64_t)(cur.tc + 1) * kTileCols <= p.cols;
    if (full) Op::template process<true>(p, state, tile, sf, cur.tr, cur.tc);
    else Op::template process<false>(p, state, tile, sf, cur.tr, cur.tc);
    __syncthreads();  // tile fully consumed, scale staging complete
    if (threadIdx.x == 0 && k + kStages < count) load(s);
    Op::flush(p, sf, cur.tr, cur.tc);
    cur.advance();
    if (++s == (uint32_t)kStages) s = 0, phase ^= 1u;
  }
  Op::finish(p, state);
}

// ---- outputs staged in shared memory and written by TMA stores (row + column kernels)
constexpr int kStagesTs = 2;
constexpr int kStageOutBytes = kTileCols * 128;  // transposed fp8 tile: 128 columns x 128 bytes
// 1 KiB alignment slack (the 128-byte swizzle of the staging tile), the staging tile, input stages,
// barriers + counters, four scale atoms
constexpr int kTsSmemBytes = 1024 + kStageOutBytes + kStagesTs * kTileBytes + 64 + 4 * 512;

// The 2 x 32 payload bytes of a column-pass thread into the transposed staging tile
// [128 columns][128 bytes] that a TMA store with the 128-byte swizzle reads: the 16-byte chunk j
// of staging row c lives at chunk j ^ (c & 7).  Two-way bank conflicts at most.
__device__ __forceinline__ void stage_transposed(uint32_t stg, int t, const uint32_t (&lo)[8], const uint32_t (&hi)[8]) {
  const int w = t & 63, rb = t >> 6;
  const uint32_t c0 = 2 * w, c1 = 2 * w + 1;
  const uint32_t r0 = stg + c0 * 128, r1 = stg + c1 * 128;
  const uint32_t j0 = 2 * rb, j1 = 2 * rb + 1;
  auto sts128 = [](uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
  };
  sts128(r0 + ((j0 ^ (c0 & 7)) << 4), lo[0], lo[1], lo[2], lo[3]);
  sts128(r0 + ((j1 ^ (c0 & 7)) << 4), lo[4], lo[5], lo[6], lo[7]);
  sts128(r1 + ((j0 ^ (c1 & 7)) << 4), hi[0], hi[1], hi[2], hi[3]);
  sts128(r1 + ((j1 ^ (c1 & 7)) << 4), hi[4], hi[5], hi[6], hi[7]);
}

}  // namespace tnq

// ------------------------------------------------------------------ host: tensor map
namespace tnq_host {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a row-major [rows, cols] matrix of 16-bit elements, box 128 x 128,
// zero fill outside.  Requires a 16-byte aligned base and cols % 8 == 0.
inline int make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return TNQ_ECUDA;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)tnq::kTileCols, (cuuint32_t)tnq::kTileRows};
  const cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return TNQ_ECUDA;
  }
  return TNQ_OK;
}

// Tensor map of a row-major [outer, inner] matrix of bytes for TMA stores of 128 x 128-byte
// boxes out of shared memory.  `swizzle128`: the shared-memory tile uses the 128-byte swizzle
// (16-byte chunk j of row r at chunk j ^ (r & 7); tile base 1 KiB aligned).  Requires a
// 16-byte aligned base and inner % 16 == 0.
inline int make_byte_store_map(CUtensorMap* map, void* base, int64_t outer, int64_t inner, bool swizzle128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return TNQ_ECUDA;
  const cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  const cuuint64_t gstride[1] = {(cuuint64_t)inner};
  const cuuint32_t box[2] = {128u, 128u};
  const cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return TNQ_ECUDA;
  }
  return TNQ_OK;
}

// resident CTAs of a kernel with `smem` bytes of dynamic shared memory (cached per device)
template <auto Kernel, int Threads, int Smem>
inline int resident_ctas_smem() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem) != cudaSuccess) return -1;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, Threads, Smem) != cudaSuccess || per_sm < 1)
      return -1;
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

template <auto Kernel, int Threads>
inline int tile_resident_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tnq::kTileSmemBytes) != cudaSuccess)
      return -1;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, Threads, tnq::kTileSmemBytes) !=
            cudaSuccess ||
        per_sm < 1)
      return -1;
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

}  // namespace tnq_host
