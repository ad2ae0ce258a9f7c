// FP8 GEMM with a per-tensor or per-row scale epilogue on the 5th-generation tensor cores:
//     C[m, n] = bf16( (sum_k A[m, k] * B[n, k]) * a_scale[m or 0] * b_scale[n or 0] )
// A [M, K] and B [N, K] are e4m3 (or e5m2), K contiguous in both - the layout the casts of this
// library produce for an activation and for a weight.  The consumer of the per-tensor and
// row-wise casts.
//
// A CTA computes 128 x 256 tiles of C, one after another (persistent grid, one CTA per SM, grouped
// tile order for L2 reuse).  Warp 0 (one elected lane) streams 128 x 128-byte
// tiles of A and 256 x 128-byte tiles of B into a ring of shared-memory stages with 2-D TMA
// loads (128-byte swizzle, one mbarrier per stage).  Warp 1 (one elected lane) issues
// tcgen05.mma (kind::f8f6f4, M = 128, N = 256, K = 32 per instruction, four per stage) with
// both operands read from shared memory through matrix descriptors and the fp32 accumulator
// in tensor memory (two accumulators of 256 columns: the epilogue of one tile overlaps the MMAs of
// the next); tcgen05.commit hands a finished stage back to the loader and, after a tile's last
// one, the accumulator to the epilogue.  Warps 2-5 (one
// per 32-lane quarter of tensor memory) read the accumulator with tcgen05.ld, apply the
// scales, round to bf16 and store rows.  Every wait is bounded (about one second): on expiry
// the CTA records TNQ_ETIMEOUT, the roles fall through to the common exit and the tensor
// memory is released.
#include <cuda.h>

#include "common.cuh"

namespace tnq {

constexpr int kGemmBM = 128, kGemmBN = 256, kGemmBK = 128;  // BK in bytes = elements
constexpr int kGemmStages = 4;
constexpr int kGemmATile = kGemmBM * kGemmBK, kGemmBTile = kGemmBN * kGemmBK;
constexpr int kGemmStageBytes = kGemmATile + kGemmBTile;
constexpr int kGemmThreads = 192;
constexpr int kGemmTmemCols = 512;  // two 128 x 256 fp32 accumulators
constexpr int kGemmSmemBytes = kGemmStages * kGemmStageBytes + 1024 /* alignment */ + 128 /* barriers */;

// shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1
__device__ __forceinline__ uint64_t gemm_smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;             // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;             // version
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// instruction descriptor: fp32 accumulator, A and B in the given 8-bit float format, both K-major
__host__ __device__ constexpr uint32_t gemm_instr_desc(int fmt /* 0 e4m3, 1 e5m2 */) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(kGemmBN >> 3) << 17) |
         ((uint32_t)(kGemmBM >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// Tile t of the (tiles_m x tiles_n) grid in a grouped order: kGemmGroupM consecutive row-tiles are
// swept across all column-tiles before the next group starts, so the tiles in flight at one
// time share a small set of A and B panels in L2.
#ifndef TNQ_GEMM_GROUP_M
#define TNQ_GEMM_GROUP_M 16
#endif
constexpr int kGemmGroupM = TNQ_GEMM_GROUP_M;
__device__ __forceinline__ void gemm_tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kGemmGroupM * tiles_n;
  const int group = t / per_group, in_group = t % per_group;
  const int first_m = group * kGemmGroupM;
  const int rows_here = min(kGemmGroupM, tiles_m - first_m);
  tm = first_m + in_group % rows_here;
  tn = in_group / rows_here;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent: CTA c computes tiles c, c + gridDim.x, ...  The accumulator is double-buffered in
// tensor memory (2 x 256 columns) so that the epilogue of one tile overlaps the MMAs of the next.
__global__ void __launch_bounds__(kGemmThreads, 1)
    k_fp8_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const float* __restrict__ a_scale, const float* __restrict__ b_scale, int rowwise, int fmt, int m, int n,
               int k, uint16_t* __restrict__ out, uint32_t* status) {
  extern __shared__ uint8_t tnq_gemm_smem[];
  uint8_t* const base = tnq_gemm_smem + ((1024u - (smem_u32(tnq_gemm_smem) & 1023u)) & 1023u);
  uint64_t* const full = reinterpret_cast<uint64_t*>(base + kGemmStages * kGemmStageBytes);
  uint64_t* const empty = full + kGemmStages;
  uint64_t* const acc_full = empty + kGemmStages;  // [2]: MMA -> epilogue
  uint64_t* const acc_empty = acc_full + 2;        // [2]: epilogue (4 warps) -> MMA
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint32_t* const failed = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (m + kGemmBM - 1) / kGemmBM, tiles_n = (n + kGemmBN - 1) / kGemmBN;
  const int tiles = tiles_m * tiles_n;
  const int kblocks = (k + kGemmBK - 1) / kGemmBK;

  if (threadIdx.x == 0) {
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
    for (int s = 0; s < kGemmStages; ++s) mbar_init(&full[s], 1), mbar_init(&empty[s], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&acc_full[i], 1), mbar_init(&acc_empty[i], 4);
    *failed = 0;
    fence_mbar_init();
  }
  if (warp == 1) {  // the warp that allocates tensor memory also frees it
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kGemmTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {  // ---- loader
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        int tm, tn;
        gemm_tile_coords(t, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kGemmStages, ph = (it / kGemmStages) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u)) {
            atomicExch(failed, 1u);
            ok = false;
            break;
          }
          uint8_t* stage = base + s * kGemmStageBytes;
          mbar_expect_tx(&full[s], kGemmStageBytes);
          tma_load_2d(stage, &map_a, kb * kGemmBK, tm * kGemmBM, &full[s]);
          tma_load_2d(stage + kGemmATile, &map_b, kb * kGemmBK, tn * kGemmBN, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer
      const uint32_t idesc = gemm_instr_desc(fmt);
      uint32_t it = 0;
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++i) {
        const uint32_t buf = (uint32_t)i & 1u, aph = ((uint32_t)i >> 1) & 1u;
        if (!mbar_wait(&acc_empty[buf], aph ^ 1u)) {  // the epilogue has drained this accumulator
          atomicExch(failed, 1u);
          break;
        }
        tcgen05_fence_after();
        const uint32_t acc = tmem + buf * (uint32_t)kGemmBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kGemmStages, ph = (it / kGemmStages) & 1u;
          if (!mbar_wait(&full[s], ph)) {
            atomicExch(failed, 1u);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(base + s * kGemmStageBytes);
          const uint64_t da = gemm_smem_desc(sa), db = gemm_smem_desc(sa + kGemmATile);
#pragma unroll
          for (int j = 0; j < kGemmBK / 32; ++j)  // 32 bytes of K per instruction: the descriptor start moves by 32 >> 4
            umma_f8(acc, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (kb > 0 || j > 0) ? 1u : 0u);
          umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);  // complete once every MMA issued so far has finished
      }
    }
  } else {  // ---- epilogue: warp w may read tensor-memory lanes 32 * (w % 4) .. + 31
    // every output row starts on a 32-byte boundary: 256-bit stores are legal
    const bool wide_rows = (n % 16) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
    const int quarter = warp & 3;
    const float sb0 = rowwise ? 0.0f : b_scale[0];
    int i = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++i) {
      int tm, tn;
      gemm_tile_coords(t, tiles_m, tiles_n, tm, tn);
      const uint32_t buf = (uint32_t)i & 1u, aph = ((uint32_t)i >> 1) & 1u;
      bool ok = mbar_wait(&acc_full[buf], aph);
      if (!ok) atomicExch(failed, 1u);
      if (!__all_sync(0xffffffffu, ok)) break;
      tcgen05_fence_after();
      const int row = tm * kGemmBM + quarter * 32 + lane;
      const float sa = rowwise ? (row < m ? a_scale[row] : 0.0f) : a_scale[0];
#pragma unroll 1
      for (int c0 = 0; c0 < kGemmBN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * (uint32_t)kGemmBN + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = tn * kGemmBN + c0;
        if (row < m && col0 < n) {
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int c = col0 + 2 * j;
            const float s0 = rowwise ? __fmul_rn(sa, c < n ? b_scale[c] : 0.0f) : __fmul_rn(sa, sb0);
            const float s1 = rowwise ? __fmul_rn(sa, c + 1 < n ? b_scale[c + 1] : 0.0f) : s0;
            const float v0 = __fmul_rn(__uint_as_float(r[2 * j]), s0), v1 = __fmul_rn(__uint_as_float(r[2 * j + 1]), s1);
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[j]) : "f"(v1), "f"(v0));
          }
          uint16_t* dst = out + (int64_t)row * n + col0;
          if (col0 + 32 <= n && wide_rows) {  // two whole 32-byte sectors per lane and instruction
            stg256(dst, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
            stg256(dst + 16, o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]);
          } else if (col0 + 32 <= n && (n % 8) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) stg128(dst + 8 * j, make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < n) dst[j] = (uint16_t)(o[j >> 1] >> (16 * (j & 1)));
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // this warp's quarter of the accumulator has been read
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGemmTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && *failed != 0 && status != nullptr) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

typedef CUresult (*GemmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, k] bytes, K contiguous, box 128 bytes x box_rows, 128-byte swizzle, zero fill outside
static int gemm_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  static GemmEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return TNQ_ECUDA;
    fn = reinterpret_cast<GemmEncodeFn>(p);
  }
  const cuuint64_t gdim[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)box_rows};
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

extern "C" int tnq_fp8_gemm(const void* a, const void* b, const float* a_scale, const float* b_scale, int rowwise,
                            int fp8_dtype, int64_t m, int64_t n, int64_t k, void* out_bf16, uint32_t* status,
                            tnq_stream_t stream) {
  if (m < 0 || n < 0 || k < 0) return TNQ_EINVAL;
  if (fp8_dtype != TNQ_FP8_E4M3 && fp8_dtype != TNQ_FP8_E5M2) return TNQ_EINVAL;
  if (m == 0 || n == 0) return TNQ_OK;
  if (!a || !b || !a_scale || !b_scale || !out_bf16) return TNQ_EINVAL;
  if (k == 0 || k % 16 != 0) return TNQ_ESHAPE;  // 16-byte row pitch for the tile loads
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return TNQ_EUNSUPPORTED;
  const int64_t tiles = ((m + kGemmBM - 1) / kGemmBM) * ((n + kGemmBN - 1) / kGemmBN);
  if (tiles > 0x7fffffff) return TNQ_EUNSUPPORTED;
  if (!aligned16(a) || !aligned16(b) || !aligned16(out_bf16)) return TNQ_EALIGN;
  CUtensorMap map_a, map_b;
  int rc = gemm_operand_map(&map_a, a, m, k, kGemmBM);
  if (rc != TNQ_OK) return rc;
  rc = gemm_operand_map(&map_b, b, n, k, kGemmBN);
  if (rc != TNQ_OK) return rc;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(k_fp8_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes) != cudaSuccess)
      return cuda_fail(cudaGetLastError());
    configured[dev] = 1;
  }
  const int64_t sms = sm_count();
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  k_fp8_gemm<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(
      map_a, map_b, a_scale, b_scale, rowwise ? 1 : 0, fp8_dtype == TNQ_FP8_E4M3 ? 0 : 1, (int)m, (int)n, (int)k,
      static_cast<uint16_t*>(out_bf16), status);
  return check_launch();
}
