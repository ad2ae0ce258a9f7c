// Diagnostic: the tile pipeline of the block-scaled quantizers with the arithmetic taken out.
// A [rows, cols] bf16 matrix is copied tile by tile - 2-D TMA load of a 128 x 128 tile into a ring of
// shared-memory stages, 2-D TMA store of the same bytes - by persistent CTAs in which one thread does all
// the work.  What this takes is what a kernel that reads 128 x 128 tiles through TMA and writes the same
// number of bytes can reach at best on a given matrix; the quantizers' times are read against it.
#include "tile_pipeline.cuh"

namespace tnq {

__global__ void __launch_bounds__(128)
    k_tile_copy(const __grid_constant__ CUtensorMap in, const __grid_constant__ CUtensorMap out, uint32_t tiles_r,
                uint32_t tiles_c, int stages, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t tnq_copy_smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(tnq_copy_smem + stages * kTileBytes);
  const uint32_t ntiles = tiles_r * tiles_c;
  const uint32_t first = blockIdx.x;
  const uint32_t count = first < ntiles ? (ntiles - first + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x != 0) return;
  for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
  fence_mbar_init();
  pdl_wait();
  pdl_launch_dependents();
  auto issue = [&](uint32_t k) {  // tile k of this CTA into stage k % stages
    const uint32_t t = first + k * gridDim.x, s = k % stages;
    mbar_expect_tx(&bars[s], kTileBytes);
    tma_load_2d(tnq_copy_smem + s * kTileBytes, &in, (int32_t)((t % tiles_c) * kTileCols), (int32_t)((t / tiles_c) * kTileRows),
                &bars[s]);
  };
  for (uint32_t k = 0; k < (uint32_t)stages && k < count; ++k) issue(k);
  for (uint32_t k = 0; k < count; ++k) {
    const uint32_t s = k % stages, phase = (k / stages) & 1u;
    if (!mbar_wait(&bars[s], phase)) {
      if (status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      break;
    }
    const uint32_t t = first + k * gridDim.x;
    tma_store_2d(&out, smem_u32(tnq_copy_smem + s * kTileBytes), (int32_t)((t % tiles_c) * kTileCols),
                 (int32_t)((t / tiles_c) * kTileRows));
    bulk_group_commit();
    if (k >= 1 && k - 1 + stages < count) {  // the previous tile's store has read its stage: load into it
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue(k - 1 + stages);
    }
  }
  bulk_group_wait();
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

extern "C" int tnq_tile_copy(const void* x, void* y, int64_t rows, int64_t cols, int stages, int ctas_per_sm,
                             uint32_t* status, tnq_stream_t stream) {
  if (x == nullptr || y == nullptr || rows <= 0 || cols <= 0) return TNQ_EINVAL;
  if (rows % kTileRows != 0 || cols % kTileCols != 0) return TNQ_ESHAPE;
  if (stages < 2 || stages > 6 || ctas_per_sm < 1 || ctas_per_sm > 4) return TNQ_EINVAL;
  if (!aligned16(x) || !aligned16(y)) return TNQ_EALIGN;
  if ((rows / kTileRows) * (cols / kTileCols) > 0x7fffffff) return TNQ_EUNSUPPORTED;
  const int smem = stages * kTileBytes + 64;
  if (cudaFuncSetAttribute(k_tile_copy, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return cuda_fail(cudaGetLastError());
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_tile_copy, 128, smem) != cudaSuccess) return cuda_fail(cudaGetLastError());
  if (occ < ctas_per_sm) return TNQ_EUNSUPPORTED;
  CUtensorMap in, out;
  int rc = make_tile_map(&in, x, rows, cols);
  if (rc == TNQ_OK) rc = make_tile_map(&out, y, rows, cols);
  if (rc != TNQ_OK) return rc;
  const int64_t ntiles = (rows / kTileRows) * (cols / kTileCols);
  const int64_t cap = (int64_t)ctas_per_sm * sm_count();
  return launch_chained(k_tile_copy, dim3((unsigned)(ntiles < cap ? ntiles : cap)), dim3(128), smem, stream, in, out,
                        (uint32_t)(rows / kTileRows), (uint32_t)(cols / kTileCols), stages, status);
}
