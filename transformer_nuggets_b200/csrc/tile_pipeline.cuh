// Persistent 128x128 bf16 tile pipeline used by the block-scaled quantizers.
//
// Each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... of a row-major
// [rows, cols] bf16 matrix.  Tiles are brought into shared memory by 2-D TMA loads
// (cp.async.bulk.tensor, cluster size 1, one destination CTA) into a ring of kStages
// buffers, each guarded by an mbarrier; out-of-range parts of edge tiles arrive as
// zeros.  One elected thread issues the loads; all 256 threads consume.  A stage is
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
constexpr int kTileThreads = 256;
constexpr int kSfBytes = 1024;  // per-tile scale staging (up to two 512-byte atoms)
// ring + alignment slack + barriers + two double-buffered scale staging areas
constexpr int kTileSmemBytes = kStages * kTileBytes + 128 + 64 + 2 * 2 * kSfBytes;

struct TileShared {
  uint8_t* tile[kStages];
  uint64_t* full;  // [kStages]
  uint8_t* sf[2];  // double-buffered, 2 * kSfBytes each
};

__device__ __forceinline__ TileShared carve_tile_smem(uint8_t* raw) {
  TileShared s;
  const uint32_t a = smem_u32(raw);
  uint8_t* base = raw + ((128u - (a & 127u)) & 127u);
#pragma unroll
  for (int i = 0; i < kStages; ++i) s.tile[i] = base + i * kTileBytes;
  s.full = reinterpret_cast<uint64_t*>(base + kStages * kTileBytes);
  s.sf[0] = base + kStages * kTileBytes + 64;
  s.sf[1] = s.sf[0] + 2 * kSfBytes;
  return s;
}

// Op::process(params, tile_smem, sf_smem, tile_row, tile_col)   all threads
// Op::flush(params, sf_smem, tile_row, tile_col)                 all threads, after a __syncthreads
template <class Op>
__device__ __forceinline__ void run_tile_pipeline(const CUtensorMap* tmap, const typename Op::Params& p,
                                                  int64_t tiles_r, int64_t tiles_c, uint32_t* status) {
  extern __shared__ uint8_t tnq_dyn_smem[];
  const TileShared sh = carve_tile_smem(tnq_dyn_smem);
  const int64_t ntiles = tiles_r * tiles_c;
  const int64_t first = blockIdx.x;
  const int64_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(tmap);
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(&sh.full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages && s < count; ++s) {
      const int64_t t = first + (int64_t)s * gridDim.x;
      mbar_expect_tx(&sh.full[s], kTileBytes);
      tma_load_2d(sh.tile[s], tmap, (int32_t)((t % tiles_c) * kTileCols), (int32_t)((t / tiles_c) * kTileRows),
                  &sh.full[s]);
    }
  }
  for (int64_t k = 0; k < count; ++k) {
    const int s = (int)(k % kStages);
    const uint32_t parity = (uint32_t)((k / kStages) & 1);
    if (!mbar_wait(&sh.full[s], parity)) {
      if (threadIdx.x == 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      return;
    }
    const int64_t t = first + k * gridDim.x;
    const int64_t tr = t / tiles_c, tc = t % tiles_c;
    uint8_t* sf = sh.sf[k & 1];
    Op::process(p, sh.tile[s], sf, tr, tc);
    __syncthreads();  // tile fully consumed, scale staging complete
    if (threadIdx.x == 0 && k + kStages < count) {
      const int64_t tn = first + (k + kStages) * gridDim.x;
      mbar_expect_tx(&sh.full[s], kTileBytes);
      tma_load_2d(sh.tile[s], tmap, (int32_t)((tn % tiles_c) * kTileCols), (int32_t)((tn / tiles_c) * kTileRows),
                  &sh.full[s]);
    }
    Op::flush(p, sf, tr, tc);
  }
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

template <auto Kernel>
inline int tile_resident_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tnq::kTileSmemBytes) != cudaSuccess)
      return -1;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, tnq::kTileThreads, tnq::kTileSmemBytes) !=
            cudaSuccess ||
        per_sm < 1)
      return -1;
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

}  // namespace tnq_host
