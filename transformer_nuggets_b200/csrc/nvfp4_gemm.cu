// NVFP4 GEMM on the block-scaled tensor-core path: the consumer of the NVFP4 quantizer's outputs
// exactly as it writes them - packed e2m1 payload, E4M3 block scales in the swizzled 128x4
// layout, one fp32 global scale per tensor.
//     C[m, n] = bf16( ga * gb * sum_b sa[m,b] * sb[n,b] * sum_{k in block b} A[m, k] * B[n, k] )      (16-element blocks)
// A [M, K/2], B [N, K/2] bytes (two codes per byte, low nibble first), K contiguous.
//
// Same structure as the MXFP8 GEMM (mxfp8_gemm.cu).  A 128-byte K step of a tile row holds 256
// elements = 16 blocks = FOUR 512-byte scale atoms per 128 rows, contiguous in the swizzled
// buffer: one 2 KiB bulk copy for A and two for the 256 rows of B per stage.  Each of the four
// MMAs of a stage (tcgen05.mma kind::mxf4nvf4.block_scale.block16, K = 64) consumes one whole
// atom per 128 rows (four scale bytes per row), moved to tensor memory by tcgen05.cp.  The
// twelve copies of a stage are issued by a lane of their own, one stage ahead of the MMAs and
// into alternating sets of scale columns (its tcgen05.commit tells the MMA lane when a set is
// filled; the MMAs' commit on the stage tells it when a set may be overwritten): with the copies
// in front of the MMAs in one lane's instruction stream the kernel was 3-9 % slower.  The
// global scales are applied to the fp32 accumulator in the epilogue.
#include <cuda.h>

#include "common.cuh"

namespace tnq {

constexpr int kNvgBM = 128, kNvgBN = 256, kNvgBK = 128;  // BK in bytes = elements
constexpr int kNvgStages = 4;
constexpr int kNvgATile = kNvgBM * kNvgBK, kNvgBTile = kNvgBN * kNvgBK;
constexpr int kNvgSfA = 2048, kNvgSfB = 4096;  // four scale atoms (one per MMA) for the 128 rows of A, eight for B
constexpr int kNvgStageData = kNvgATile + kNvgBTile + kNvgSfA + kNvgSfB;
constexpr int kNvgStageBytes = 56320;  // kNvgStageData rounded up to a multiple of 1024 (tile alignment)
constexpr int kNvgEpilogueWarps = 8;  // two per tensor-memory lane quarter: columns 0..127 and 128..255 of the tile
constexpr int kNvgThreads = 96 + 32 * kNvgEpilogueWarps;  // + the loader warp, the MMA warp and the scale-copier warp
constexpr int kNvgTmemCols = 512;  // one 128 x 256 fp32 accumulator + two sets of 48 scale columns (power of two)
constexpr int kNvgSfCol = 256;     // scale set p at +64p: A at +4j (MMA j of a stage), B at +16 + 8j (+4 for rows 128..255)
constexpr int kNvgSmemBytes = kNvgStages * kNvgStageBytes + 1024 /* alignment */ + 128 /* barriers */;

// shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1
__device__ __forceinline__ uint64_t nvg_smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;             // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;             // version
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// block-scaled instruction descriptor: e2m1 x e2m1 (two per byte), both K-major, E4M3 scales,
// K = 64 per instruction, N and M
__device__ __forceinline__ uint32_t nvg_instr_desc() {
  return (1u << 7) | (1u << 10) | ((uint32_t)(kNvgBN >> 3) << 17) | ((uint32_t)(kNvgBM >> 4) << 24);
}
// scale atom in shared memory: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t nvg_sf_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;  // stride byte offset; one 16-byte column only, so no leading offset
  d |= (uint64_t)1 << 46;           // version
  return d;
}
__device__ __forceinline__ void nvg_sf_copy(uint32_t tmem_col, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tsfa,
                                          uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void nvg_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void nvg_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void nvg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void nvg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// Tile t of the (tiles_m x tiles_n) grid in a grouped order: kNvgGroupM consecutive row-tiles are
// swept across all column-tiles before the next group starts, so the tiles in flight at one
// time share a small set of A and B panels in L2.
#ifndef TNQ_NVG_GROUP_M
#define TNQ_NVG_GROUP_M 16
#endif
constexpr int kNvgGroupM = TNQ_NVG_GROUP_M;
__device__ __forceinline__ void nvg_tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kNvgGroupM * tiles_n;
  const int group = t / per_group, in_group = t % per_group;
  const int first_m = group * kNvgGroupM;
  const int rows_here = min(kNvgGroupM, tiles_m - first_m);
  tm = first_m + in_group % rows_here;
  tn = in_group / rows_here;
}
__device__ __forceinline__ void nvg_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent: CTA c computes tiles c, c + gridDim.x, ...  One accumulator (256 columns) plus the
// scale columns fill the tensor-memory allocation, so only the stores of a tile's epilogue are
// overlapped with the next tile's MMAs: eight warps first drain the accumulator into registers
// and release it.  Measured alternatives: 128 x 192 tiles with two accumulators
// (the scale columns of a tile then start 0 or 2 columns into an atom) overlap the epilogue but
// re-read more of A per output and were 13-16 % slower; 128 x 224 tiles would need scale columns
// starting on an odd column, which the MMA does not accept.
__global__ void __launch_bounds__(kNvgThreads, 1)
    k_nvfp4_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const uint8_t* __restrict__ sf_a, const uint8_t* __restrict__ sf_b, const float* __restrict__ a_global,
               const float* __restrict__ b_global, int m, int n, int k, uint16_t* __restrict__ out, uint32_t* status) {
  extern __shared__ uint8_t tnq_nvg_smem[];
  uint8_t* const base = tnq_nvg_smem + ((1024u - (smem_u32(tnq_nvg_smem) & 1023u)) & 1023u);
  uint64_t* const full = reinterpret_cast<uint64_t*>(base + kNvgStages * kNvgStageBytes);
  uint64_t* const empty = full + kNvgStages;
  uint64_t* const acc_full = empty + kNvgStages;  // [2]: MMA -> epilogue
  uint64_t* const acc_empty = acc_full + 2;        // [2]: epilogue (8 warps) -> MMA
  uint64_t* const sfready = acc_empty + 2;         // [2]: scale copier -> MMA, one per set of scale columns
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(sfready + 2);
  uint32_t* const failed = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + kNvgBM - 1) / kNvgBM, tiles_n = (n + kNvgBN - 1) / kNvgBN;
  const int tiles = tiles_m * tiles_n;
  const int kblocks = (k / 2 + kNvgBK - 1) / kNvgBK;  // 128 bytes = 256 elements per stage

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    for (int s = 0; s < kNvgStages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&acc_full[i], 1), mbar_init(&acc_empty[i], kNvgEpilogueWarps);
    for (int i = 0; i < 2; ++i) mbar_init(&sfready[i], 1);
    *failed = 0;
    fence_mbar_init();
  }
  if (warp == 1) {  // the warp that allocates tensor memory also frees it
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kNvgTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  nvg_fence_before();
  __syncthreads();
  nvg_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- loader
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        int tm, tn;
        nvg_tile_coords(t, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kNvgStages, ph = (it / kNvgStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) {
            atomicExch(failed, 1u);
            ok = false;
            break;
          }
          uint8_t* stage = base + s * kNvgStageBytes;
          const bool second = tn * kNvgBN + 128 < n;  // the tile's rows 128..255 of B exist
          mbar_expect_tx(&full[s], kNvgATile + kNvgBTile + kNvgSfA + (second ? 4096 : 2048));
          tma_load_2d(stage, &map_a, kb * kNvgBK, tm * kNvgBM, &full[s]);
          tma_load_2d(stage + kNvgATile, &map_b, kb * kNvgBK, tn * kNvgBN, &full[s]);
          // four 512-byte atoms per 128 rows and stage, contiguous: atoms (row tile, 4 kb .. 4 kb + 3) of a
          // [rows, K/16] scale matrix with K/64 atoms per row tile
          uint8_t* sfs = stage + kNvgATile + kNvgBTile;
          const int64_t per_tile = (int64_t)kblocks * 4;
          bulk_g2s(sfs, sf_a + ((int64_t)tm * per_tile + 4 * kb) * 512, 2048, &full[s]);
          bulk_g2s(sfs + 2048, sf_b + ((int64_t)(2 * tn) * per_tile + 4 * kb) * 512, 2048, &full[s]);
          if (second) bulk_g2s(sfs + 4096, sf_b + ((int64_t)(2 * tn + 1) * per_tile + 4 * kb) * 512, 2048, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer; the scale columns are filled by the copier warp
      const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
      const uint32_t total = (uint32_t)my_tiles * (uint32_t)kblocks;
      const uint32_t idesc = nvg_instr_desc();
      uint32_t tile_i = 0;
      for (uint32_t it = 0; it < total; ++it) {
        const uint32_t kb = it % (uint32_t)kblocks;
        if (kb == 0) {
          if (!mbar_wait(&acc_empty[0], (tile_i & 1u) ^ 1u)) { atomicExch(failed, 1u); break; }
        }
        const uint32_t s = it % kNvgStages, ph = (it / kNvgStages) & 1u;
        if (!mbar_wait(&full[s], ph) || !mbar_wait(&sfready[it & 1u], (it >> 1) & 1u)) { atomicExch(failed, 1u); break; }
        nvg_fence_after();
        const uint32_t sa = smem_u32(base + s * kNvgStageBytes);
        const uint64_t da = nvg_smem_desc(sa), db = nvg_smem_desc(sa + kNvgATile);
        const uint32_t set = tmem + kNvgSfCol + 64u * (it & 1u);
#pragma unroll
        for (int j = 0; j < kNvgBK / 32; ++j)
          umma_nvf4(tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, set + 4 * j, set + 16 + 8 * j,
                    (kb > 0 || j > 0) ? 1u : 0u);
        nvg_commit(&empty[s]);
        if (kb == (uint32_t)kblocks - 1) { nvg_commit(&acc_full[0]); ++tile_i; }
      }
    }
  } else if (warp == 2 + kNvgEpilogueWarps) {
    if (lane == 0) {  // ---- scale copier: shared memory -> the set of scale columns of iteration it
      const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
      const uint32_t total = (uint32_t)my_tiles * (uint32_t)kblocks;
      for (uint32_t it = 0; it < total; ++it) {
        const uint32_t s = it % kNvgStages, ph = (it / kNvgStages) & 1u;
        bool ok = mbar_wait(&full[s], ph);
        // the MMAs of iteration it - 2 read this set of columns: their commit completes empty[(it - 2) % stages]
        if (ok && it >= 2) ok = mbar_wait(&empty[(it - 2) % kNvgStages], ((it - 2) / kNvgStages) & 1u);
        if (!ok) { atomicExch(failed, 1u); break; }
        nvg_fence_after();
        const uint32_t sfs = smem_u32(base + s * kNvgStageBytes) + kNvgATile + kNvgBTile;
        const uint32_t set = tmem + kNvgSfCol + 64u * (it & 1u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          nvg_sf_copy(set + 4 * j, nvg_sf_desc(sfs + 512 * j));
          nvg_sf_copy(set + 16 + 8 * j, nvg_sf_desc(sfs + 2048 + 512 * j));
          nvg_sf_copy(set + 16 + 8 * j + 4, nvg_sf_desc(sfs + 4096 + 512 * j));
        }
        nvg_commit(&sfready[it & 1u]);
      }
    }
  } else {  // ---- epilogue: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31
    // every output row starts on a 32-byte boundary: 256-bit stores are legal
    const bool wide_rows = (n % 16) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const float gscale = __fmul_rn(a_global ? *a_global : 1.0f, b_global ? *b_global : 1.0f);
    int i = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++i) {
      int tm, tn;
      nvg_tile_coords(t, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = 0u, aph = (uint32_t)i & 1u;
      bool ok = mbar_wait(&acc_full[buf], aph);
      if (!ok) atomicExch(failed, 1u);
      if (!__all_sync(0xffffffffu, ok)) break;
      nvg_fence_after();
      const int row = tm * kNvgBM + quarter * 32 + lane;
      // Drain this warp's 32 rows x 128 columns into registers as packed bf16, hand the accumulator
      // back to the MMA issuer, then store: the stores overlap the next tile's MMAs.
      uint32_t o[kNvgBN / 4];
#pragma unroll
      for (int c = 0; c < kNvgBN / 64; ++c) {
        uint32_t r[32];
        nvg_tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)kNvgBN + (uint32_t)(128 * half + 32 * c), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[16 * c + j]) : "f"(__fmul_rn(__uint_as_float(r[2 * j + 1]), gscale)), "f"(__fmul_rn(__uint_as_float(r[2 * j]), gscale)));
        }
      }
      nvg_fence_before();
      __syncwarp();
      if (lane == 0) nvg_mbar_arrive(&acc_empty[buf]);  // this warp's part of the accumulator has been read
      if (row < m) {
#pragma unroll
        for (int c = 0; c < kNvgBN / 64; ++c) {
          const int col0 = tn * kNvgBN + 128 * half + 32 * c;
          if (col0 < n) {
            uint16_t* dst = out + (int64_t)row * n + col0;
            const uint32_t* oc = o + 16 * c;
            if (col0 + 32 <= n && wide_rows) {  // two whole 32-byte sectors per lane and instruction
              stg256(dst, oc[0], oc[1], oc[2], oc[3], oc[4], oc[5], oc[6], oc[7]);
              stg256(dst + 16, oc[8], oc[9], oc[10], oc[11], oc[12], oc[13], oc[14], oc[15]);
            } else if (col0 + 32 <= n && (n % 8) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) stg128(dst + 8 * j, make_uint4(oc[4 * j], oc[4 * j + 1], oc[4 * j + 2], oc[4 * j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < n) dst[j] = (uint16_t)(oc[j >> 1] >> (16 * (j & 1)));
            }
          }
        }
      }
    }
  }
  nvg_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kNvgTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && *failed != 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

typedef CUresult (*NvgEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, k] bytes, K contiguous, box 128 bytes x box_rows, 128-byte swizzle, zero fill outside
static int nvg_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  static NvgEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return TNQ_ECUDA;
    fn = reinterpret_cast<NvgEncodeFn>(p);
  }
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {(cuuint32_t)kNvgBK, (cuuint32_t)box_rows};
  const cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return TNQ_ECUDA;
  }
  return TNQ_OK;
}

extern "C" int tnq_nvfp4_gemm(const void* a_packed, const void* b_packed, const void* sf_a, const void* sf_b,
                              const float* a_global, const float* b_global, int64_t m, int64_t n, int64_t k, void* out_bf16,
                              uint32_t* status, tnq_stream_t stream) {
  if (m < 0 || n < 0 || k < 0) return TNQ_EINVAL;
  if (m == 0 || n == 0) return TNQ_OK;
  if (!a_packed || !b_packed || !sf_a || !sf_b || !out_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 256 != 0) return TNQ_ESHAPE;  // whole stages: 128 bytes of codes and four scale atoms along K
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return TNQ_EUNSUPPORTED;
  const int64_t tiles = ((m + kNvgBM - 1) / kNvgBM) * ((n + kNvgBN - 1) / kNvgBN);
  if (tiles > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (!aligned16(a_packed) || !aligned16(b_packed) || !aligned16(out_bf16) || !aligned16(sf_a) || !aligned16(sf_b))
    return TNQ_EALIGN;
  CUtensorMap map_a, map_b;
  int rc = nvg_operand_map(&map_a, a_packed, m, k / 2, kNvgBM);
  if (rc != TNQ_OK) return rc;
  rc = nvg_operand_map(&map_b, b_packed, n, k / 2, kNvgBN);
  if (rc != TNQ_OK) return rc;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(k_nvfp4_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kNvgSmemBytes) != cudaSuccess)
      return cuda_fail(cudaGetLastError());
    configured[dev] = 1;
  }
  const int64_t sms = sm_count();
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  k_nvfp4_gemm<<<grid, kNvgThreads, kNvgSmemBytes, stream>>>(map_a, map_b, static_cast<const uint8_t*>(sf_a),
                                                             static_cast<const uint8_t*>(sf_b), a_global, b_global, (int)m,
                                                             (int)n, (int)k, static_cast<uint16_t*>(out_bf16), status);
  return check_launch();
}
