// MXFP8 GEMM on the block-scaled tensor-core path: the consumer of the MXFP8 quantizer's outputs
// exactly as it writes them - e4m3 payload and E8M0 scales in the swizzled 128x4 layout.
//     C[m, n] = bf16( sum_b 2^(sa[m,b]-127) * 2^(sb[n,b]-127) * sum_{k in block b} A[m, k] * B[n, k] )
// A [M, K], B [N, K] e4m3 with K contiguous; sa, sb the flat swizzled scale buffers of
// [M, K/32] and [N, K/32] (to_blocked / quantize_mxfp8(..., swizzle=True)).
//
// Structure of the per-tensor FP8 GEMM (fp8_gemm.cu): persistent CTAs, 128 x 256 output tiles,
// TMA ring, one lane issuing tcgen05.mma, accumulator in tensor memory, bounded waits.
// What the block scaling adds: a 128-element K step of a 128-row operand tile needs 128 x 4
// scale bytes, which is exactly ONE 512-byte atom of the swizzled layout, contiguous in the
// scale buffer - so each stage also receives three 512-byte bulk copies (one atom for A, two
// for the 256 rows of B).  An atom is 32 rows of 16 bytes; `tcgen05.cp.32x128b.warpx4` copies
// it from shared memory into four columns of tensor memory (lane r of every 32-lane quarter
// gets row r: bytes [quad * 4 + k step] for the rows r, r + 32, r + 64, r + 96), which is the
// operand layout of `tcgen05.mma.kind::mxf8f6f4.block_scale`; the K step within the atom is
// selected by the scale-factor id in the instruction descriptor.  No shuffling of scale bytes
// anywhere between the quantizer's store and the tensor core.
#include <cuda.h>

#include "common.cuh"

namespace tnq {

constexpr int kMxgBM = 128, kMxgBN = 256, kMxgBK = 128;  // BK in bytes = elements
constexpr int kMxgStages = 4;
constexpr int kMxgATile = kMxgBM * kMxgBK, kMxgBTile = kMxgBN * kMxgBK;
constexpr int kMxgSfA = 512, kMxgSfB = 1024;  // one scale atom for the 128 rows of A, two for the 256 rows of B
constexpr int kMxgStageData = kMxgATile + kMxgBTile + kMxgSfA + kMxgSfB;
constexpr int kMxgStageBytes = 51200;  // kMxgStageData rounded up to a multiple of 1024 (tile alignment)
constexpr int kMxgEpilogueWarps = 8;  // two per tensor-memory lane quarter: columns 0..127 and 128..255 of the tile
constexpr int kMxgThreads = 64 + 32 * kMxgEpilogueWarps;  // + the loader warp and the MMA warp
constexpr int kMxgTmemCols = 512;  // one 128 x 256 fp32 accumulator + 12 columns of scale bytes (power of two)
constexpr int kMxgSfCol = 256;     // scale columns: A at +0 .. +3, B at +4 .. +11
constexpr int kMxgSmemBytes = kMxgStages * kMxgStageBytes + 1024 /* alignment */ + 128 /* barriers */;

// shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1
__device__ __forceinline__ uint64_t mxg_smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;             // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;             // version
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// block-scaled instruction descriptor: e4m3 x e4m3, both K-major, E8M0 scales, N and M, and the
// index (0..3) of the K step within the scale atom for A and for B
__device__ __forceinline__ uint32_t mxg_instr_desc(uint32_t sf_id) {
  return (sf_id << 4) | ((uint32_t)(kMxgBN >> 3) << 17) | (1u << 23) | ((uint32_t)(kMxgBM >> 4) << 24) | (sf_id << 29);
}
// scale atom in shared memory: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t mxg_sf_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;  // stride byte offset; one 16-byte column only, so no leading offset
  d |= (uint64_t)1 << 46;           // version
  return d;
}
__device__ __forceinline__ void mxg_sf_copy(uint32_t tmem_col, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t tsfa,
                                          uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tsfa), "r"(tsfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mxg_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mxg_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void mxg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mxg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// Tile t of the (tiles_m x tiles_n) grid in a grouped order: kMxgGroupM consecutive row-tiles are
// swept across all column-tiles before the next group starts, so the tiles in flight at one
// time share a small set of A and B panels in L2.
#ifndef TNQ_MXG_GROUP_M
#define TNQ_MXG_GROUP_M 16
#endif
constexpr int kMxgGroupM = TNQ_MXG_GROUP_M;
__device__ __forceinline__ void mxg_tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kMxgGroupM * tiles_n;
  const int group = t / per_group, in_group = t % per_group;
  const int first_m = group * kMxgGroupM;
  const int rows_here = min(kMxgGroupM, tiles_m - first_m);
  tm = first_m + in_group % rows_here;
  tn = in_group / rows_here;
}
__device__ __forceinline__ void mxg_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent: CTA c computes tiles c, c + gridDim.x, ...  One accumulator (256 columns) plus the
// scale columns fill the tensor-memory allocation, so only the stores of a tile's epilogue are
// overlapped with the next tile's MMAs: eight warps first drain the accumulator into registers
// and release it.  Measured alternatives: 128 x 192 tiles with two accumulators
// (the scale columns of a tile then start 0 or 2 columns into an atom) overlap the epilogue but
// re-read more of A per output and were 13-16 % slower; 128 x 224 tiles would need scale columns
// starting on an odd column, which the MMA does not accept.
__global__ void __launch_bounds__(kMxgThreads, 1)
    k_mxfp8_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const uint8_t* __restrict__ sf_a, const uint8_t* __restrict__ sf_b, int m, int n, int k,
               uint16_t* __restrict__ out, uint32_t* status) {
  extern __shared__ uint8_t tnq_mxg_smem[];
  uint8_t* const base = tnq_mxg_smem + ((1024u - (smem_u32(tnq_mxg_smem) & 1023u)) & 1023u);
  uint64_t* const full = reinterpret_cast<uint64_t*>(base + kMxgStages * kMxgStageBytes);
  uint64_t* const empty = full + kMxgStages;
  uint64_t* const acc_full = empty + kMxgStages;  // [2]: MMA -> epilogue
  uint64_t* const acc_empty = acc_full + 2;        // [2]: epilogue (8 warps) -> MMA
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint32_t* const failed = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + kMxgBM - 1) / kMxgBM, tiles_n = (n + kMxgBN - 1) / kMxgBN;
  const int tiles = tiles_m * tiles_n;
  const int kblocks = (k + kMxgBK - 1) / kMxgBK;

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    for (int s = 0; s < kMxgStages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&acc_full[i], 1), mbar_init(&acc_empty[i], kMxgEpilogueWarps);
    *failed = 0;
    fence_mbar_init();
  }
  if (warp == 1) {  // the warp that allocates tensor memory also frees it
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kMxgTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  mxg_fence_before();
  __syncthreads();
  mxg_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- loader
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        int tm, tn;
        mxg_tile_coords(t, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kMxgStages, ph = (it / kMxgStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) {
            atomicExch(failed, 1u);
            ok = false;
            break;
          }
          uint8_t* stage = base + s * kMxgStageBytes;
          const bool second = tn * kMxgBN + 128 < n;  // the tile's rows 128..255 of B exist
          mbar_expect_tx(&full[s], kMxgATile + kMxgBTile + kMxgSfA + (second ? 1024 : 512));
          tma_load_2d(stage, &map_a, kb * kMxgBK, tm * kMxgBM, &full[s]);
          tma_load_2d(stage + kMxgATile, &map_b, kb * kMxgBK, tn * kMxgBN, &full[s]);
          // one 512-byte atom per 128 rows and K step: atom (row tile, kb) of a [rows, K/32] scale matrix
          uint8_t* sfs = stage + kMxgATile + kMxgBTile;
          bulk_g2s(sfs, sf_a + ((int64_t)tm * kblocks + kb) * 512, 512, &full[s]);
          bulk_g2s(sfs + 512, sf_b + ((int64_t)(2 * tn) * kblocks + kb) * 512, 512, &full[s]);
          if (second) bulk_g2s(sfs + 1024, sf_b + ((int64_t)(2 * tn + 1) * kblocks + kb) * 512, 512, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      uint32_t it = 0;
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++i) {
        const uint32_t buf = 0u, aph = (uint32_t)i & 1u;  // one accumulator: tensor memory also holds the scales
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u)) {  // the epilogue has drained the accumulator
          atomicExch(failed, 1u);
          break;
        }
        mxg_fence_after();
        const uint32_t acc = tmem + buf * (uint32_t)kMxgBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kMxgStages, ph = (it / kMxgStages) & 1u;
          if (!mbar_wait(&full[s], ph)) {
            atomicExch(failed, 1u);
            ok = false;
            break;
          }
          mxg_fence_after();
          const uint32_t sa = smem_u32(base + s * kMxgStageBytes);
          const uint64_t da = mxg_smem_desc(sa), db = mxg_smem_desc(sa + kMxgATile);
          // this K step's scale atoms -> tensor memory (executed in order with the MMAs that read them)
          const uint32_t sfs = sa + kMxgATile + kMxgBTile;
          mxg_sf_copy(tmem + kMxgSfCol, mxg_sf_desc(sfs));
          mxg_sf_copy(tmem + kMxgSfCol + 4, mxg_sf_desc(sfs + 512));
          mxg_sf_copy(tmem + kMxgSfCol + 8, mxg_sf_desc(sfs + 1024));
#pragma unroll
          for (int j = 0; j < kMxgBK / 32; ++j)  // one 32-element block per instruction; scale id j = byte j of the atom's words
            umma_mxf8(acc, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), mxg_instr_desc((uint32_t)j),
                      (tmem + kMxgSfCol) | ((uint32_t)j << 30), (tmem + kMxgSfCol + 4) | ((uint32_t)j << 30),
                      (kb > 0 || j > 0) ? 1u : 0u);
          mxg_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        if (ok) mxg_commit(&acc_full[buf]);  // complete once every MMA issued so far has finished
      }
    }
  } else {  // ---- epilogue: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31
    // every output row starts on a 32-byte boundary: 256-bit stores are legal
    const bool wide_rows = (n % 16) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    int i = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++i) {
      int tm, tn;
      mxg_tile_coords(t, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = 0u, aph = (uint32_t)i & 1u;
      bool ok = mbar_wait(&acc_full[buf], aph);
      if (!ok) atomicExch(failed, 1u);
      if (!__all_sync(0xffffffffu, ok)) break;
      mxg_fence_after();
      const int row = tm * kMxgBM + quarter * 32 + lane;
      // Drain this warp's 32 rows x 128 columns into registers as packed bf16, hand the accumulator
      // back to the MMA issuer, then store: the stores overlap the next tile's MMAs.
      uint32_t o[kMxgBN / 4];
#pragma unroll
      for (int c = 0; c < kMxgBN / 64; ++c) {
        uint32_t r[32];
        mxg_tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)kMxgBN + (uint32_t)(128 * half + 32 * c), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[16 * c + j]) : "f"(__uint_as_float(r[2 * j + 1])), "f"(__uint_as_float(r[2 * j])));
        }
      }
      mxg_fence_before();
      __syncwarp();
      if (lane == 0) mxg_mbar_arrive(&acc_empty[buf]);  // this warp's part of the accumulator has been read
      if (row < m) {
#pragma unroll
        for (int c = 0; c < kMxgBN / 64; ++c) {
          const int col0 = tn * kMxgBN + 128 * half + 32 * c;
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
  mxg_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kMxgTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && *failed != 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

typedef CUresult (*MxgEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, k] bytes, K contiguous, box 128 bytes x box_rows, 128-byte swizzle, zero fill outside
static int mxg_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  static MxgEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return TNQ_ECUDA;
    fn = reinterpret_cast<MxgEncodeFn>(p);
  }
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {(cuuint32_t)kMxgBK, (cuuint32_t)box_rows};
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

extern "C" int tnq_mxfp8_gemm(const void* a, const void* b, const void* sf_a, const void* sf_b, int64_t m, int64_t n,
                              int64_t k, void* out_bf16, uint32_t* status, tnq_stream_t stream) {
  if (m < 0 || n < 0 || k < 0) return TNQ_EINVAL;
  if (m == 0 || n == 0) return TNQ_OK;
  if (!a || !b || !sf_a || !sf_b || !out_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 128 != 0) return TNQ_ESHAPE;  // whole scale atoms (four 32-element blocks) along K
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return TNQ_EUNSUPPORTED;
  const int64_t tiles = ((m + kMxgBM - 1) / kMxgBM) * ((n + kMxgBN - 1) / kMxgBN);
  if (tiles > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (!aligned16(a) || !aligned16(b) || !aligned16(out_bf16) || !aligned16(sf_a) || !aligned16(sf_b)) return TNQ_EALIGN;
  CUtensorMap map_a, map_b;
  int rc = mxg_operand_map(&map_a, a, m, k, kMxgBM);
  if (rc != TNQ_OK) return rc;
  rc = mxg_operand_map(&map_b, b, n, k, kMxgBN);
  if (rc != TNQ_OK) return rc;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(k_mxfp8_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxgSmemBytes) != cudaSuccess)
      return cuda_fail(cudaGetLastError());
    configured[dev] = 1;
  }
  const int64_t sms = sm_count();
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  k_mxfp8_gemm<<<grid, kMxgThreads, kMxgSmemBytes, stream>>>(map_a, map_b, static_cast<const uint8_t*>(sf_a),
                                                             static_cast<const uint8_t*>(sf_b), (int)m, (int)n, (int)k,
                                                             static_cast<uint16_t*>(out_bf16), status);
  return check_launch();
}
