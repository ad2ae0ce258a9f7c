// Single-launch dynamic per-tensor FP8 cast for tensors that fit in the shared
// memory of the whole GPU (148 SMs x ~226 KB = 33.5 MB: a 4096 x 4096 bf16 tensor
// just fits).
//
// One CTA per SM, launched cooperatively so that all CTAs are resident.  Each CTA
// owns a contiguous slab of the tensor and brings it into shared memory with bulk
// async copies (cp.async.bulk, 32 KiB pieces, one mbarrier each, all in flight at
// once).  As pieces land the CTA folds |x| maxima; a grid-wide barrier (ticket +
// generation word, bounded wait) exchanges the per-CTA maxima; then every CTA casts
// its slab straight out of shared memory.  The input crosses HBM exactly once and the
// two-launch gap of the general path disappears.
#include "common.cuh"

namespace tnq {

constexpr int kFusedThreads = 1024;
constexpr int kPieceBytes = 32768;
constexpr int kMaxPieces = 8;
constexpr int kFusedHeaderBytes = 512;  // barriers + reduction scratch in front of the slab

struct FusedWorkspace {  // same memory as the per-tensor Workspace of fp8_tensor.cu
  uint32_t ticket;
  uint32_t amax_bits;
  float scale;
  uint32_t status;
  uint32_t bar_count;  // pad[0]
  uint32_t bar_gen;    // pad[1]
  uint32_t gmax[2];    // pad[2..3]: tensor-wide maximum, one slot per barrier generation parity
  uint32_t pad[8];
  uint32_t partial[(TNQ_WORKSPACE_BYTES - 64) / 4];
};

// All CTAs of a cooperative grid meet here and leave with the maximum of their
// contributions.  One atomicMax into the slot of the current generation, a ticket, and
// a generation word that the last arriver bumps (after clearing the other slot for the
// next call).  Returns false if the others did not show up within about a second.
__device__ __forceinline__ bool grid_max_barrier(FusedWorkspace* ws, uint32_t cta_max, uint32_t* result, int* s_flag,
                                                 uint32_t* s_val) {
  if (threadIdx.x == 0) {
    int ok = 1;
    volatile uint32_t* gen = &ws->bar_gen;
    const uint32_t my_gen = *gen;
    atomicMax(&ws->gmax[my_gen & 1u], cta_max);
    __threadfence();
    const uint32_t t = atomicInc(&ws->bar_count, gridDim.x - 1);  // wraps to 0 for the next use
    if (t == gridDim.x - 1) {
      ws->gmax[(my_gen + 1u) & 1u] = 0u;
      __threadfence();
      atomicAdd(const_cast<uint32_t*>(gen), 1u);
    } else {
      uint64_t t0 = 0;
      for (uint32_t it = 0; *gen == my_gen; ++it) {
        if ((it & 255u) == 255u) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > 1000000000ull) {
            ok = 0;
            break;
          }
        }
      }
    }
    __threadfence();
    *s_val = __ldcg(&ws->gmax[my_gen & 1u]);
    *s_flag = ok;
  }
  __syncthreads();
  *result = *s_val;
  return *s_flag != 0;
}

template <int IN, int OUT>
__global__ void __launch_bounds__(kFusedThreads, 1)
    k_dynamic_fused(const uint8_t* __restrict__ x, uint8_t* __restrict__ out, int64_t total_bytes, uint32_t slab_bytes,
                    FusedWorkspace* ws, float* scale_out) {
  extern __shared__ uint8_t tnq_fused_smem[];
  const uint32_t a = smem_u32(tnq_fused_smem);
  uint8_t* base = tnq_fused_smem + ((128u - (a & 127u)) & 127u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base);              // kMaxPieces barriers
  uint32_t* red = reinterpret_cast<uint32_t*>(base + 128);         // 33 words
  int* flag = reinterpret_cast<int*>(base + 384);
  uint8_t* slab = base + kFusedHeaderBytes;

  const int64_t begin = (int64_t)blockIdx.x * slab_bytes;
  int64_t my_bytes64 = total_bytes - begin;
  if (my_bytes64 > (int64_t)slab_bytes) my_bytes64 = slab_bytes;
  if (my_bytes64 < 0) my_bytes64 = 0;
  const uint32_t my_bytes = (uint32_t)my_bytes64;  // multiple of 16
  const int pieces = (int)((my_bytes + kPieceBytes - 1) / kPieceBytes);

  if (threadIdx.x == 0) {
    for (int p = 0; p < kMaxPieces; ++p) mbar_init(&bars[p], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int p = 0; p < pieces; ++p) {
      const uint32_t off = (uint32_t)p * kPieceBytes;
      const uint32_t len = (my_bytes - off < (uint32_t)kPieceBytes) ? my_bytes - off : (uint32_t)kPieceBytes;
      mbar_expect_tx(&bars[p], len);
      bulk_g2s(slab + off, x + begin + off, len, &bars[p]);
    }
  }

  // ---- amax over the slab, piece by piece as it lands
  uint32_t m = 0;
  bool ok = true;
  for (int p = 0; p < pieces && ok; ++p) {
    ok = mbar_wait(&bars[p], 0);
    if (!ok) break;
    const uint32_t off = (uint32_t)p * kPieceBytes;
    const uint32_t len = (my_bytes - off < (uint32_t)kPieceBytes) ? my_bytes - off : (uint32_t)kPieceBytes;
    for (uint32_t v = threadIdx.x * 16u; v < len; v += kFusedThreads * 16u) {
      const uint4 q = *reinterpret_cast<const uint4*>(slab + off + v);
      if constexpr (IN == TNQ_IN_BF16) {
        m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m, q.x), q.y), q.z), q.w);
      } else {
        m = max(max(m, q.x & 0x7fffffffu), max(max(q.y & 0x7fffffffu, q.z & 0x7fffffffu), q.w & 0x7fffffffu));
      }
    }
  }
  if (__syncthreads_or(!ok)) {  // a copy never arrived: flag it and leave together
    if (threadIdx.x == 0) atomicExch(&ws->status, (uint32_t)TNQ_ETIMEOUT);
    return;
  }
  if constexpr (IN == TNQ_IN_BF16) m = fold_u16x2(m) << 16;
  m = block_max_u32(m, red);
  uint32_t g = 0;
  if (!grid_max_barrier(ws, m, &g, flag, reinterpret_cast<uint32_t*>(flag) + 1)) {
    if (threadIdx.x == 0) atomicExch(&ws->status, (uint32_t)TNQ_ETIMEOUT);
    return;
  }
  const float amax = __uint_as_float(g);
  const float s = scale_from_amax(amax, Fp8Traits<OUT>::kMax);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    ws->amax_bits = g;
    ws->scale = s;
    if (scale_out) *scale_out = s;
  }
  const bool finite = g < 0x7f800000u;

  // ---- cast the slab out of shared memory
  if constexpr (IN == TNQ_IN_BF16) {
    uint8_t* dst = out + begin / 2;
    for (uint32_t v = threadIdx.x * 16u; v < my_bytes; v += kFusedThreads * 16u) {
      const uint4 q = *reinterpret_cast<const uint4*>(slab + v);
      const uint2 o = finite ? quant8_bf16_finite<OUT>(q, s) : quant8_bf16<OUT, true>(q, s);
      stg64(dst + v / 2, o);
    }
  } else {
    uint8_t* dst = out + begin / 4;
    for (uint32_t v = threadIdx.x * 16u; v < my_bytes; v += kFusedThreads * 16u) {
      const uint4 q = *reinterpret_cast<const uint4*>(slab + v);
      const uint32_t o = finite ? quant4_f32_finite<OUT>(q, s) : quant4_f32<OUT, true>(q, s);
      stg32(dst + v / 4, o);
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

namespace tnq_host {

struct FusedLimits {
  int sms = 0;
  int max_smem = 0;
  int coop = 0;
};

static FusedLimits fused_limits() {
  static FusedLimits cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FusedLimits{};
  if (cached[dev].sms == 0) {
    FusedLimits l;
    l.sms = sm_count();
    if (cudaDeviceGetAttribute(&l.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) l.max_smem = 0;
    if (cudaDeviceGetAttribute(&l.coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) l.coop = 0;
    cached[dev] = l;
  }
  return cached[dev];
}

template <int IN, int OUT>
static int launch_fused(const uint8_t* x, uint8_t* out, int64_t total_bytes, int grid, uint32_t slab_bytes, void* ws,
                        float* scale_out, cudaStream_t stream) {
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem = (int)slab_bytes + kFusedHeaderBytes + 128;
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(k_dynamic_fused<IN, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fused_limits().max_smem);
    if (e != cudaSuccess) return cuda_fail(e);
    configured[dev] = fused_limits().max_smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFusedThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k_dynamic_fused<IN, OUT>, x, out, total_bytes, slab_bytes,
                                     static_cast<FusedWorkspace*>(ws), scale_out);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

// Whether the single-launch kernel can take this tensor; fills grid and slab size.
bool fused_plan(int64_t total_bytes, int* grid, uint32_t* slab_bytes) {
  const FusedLimits l = fused_limits();
  if (l.sms <= 0 || !l.coop || total_bytes <= 0 || (total_bytes & 15) != 0) return false;
  const int64_t max_slab = ((int64_t)l.max_smem - kFusedHeaderBytes - 128) & ~127ll;
  if (max_slab < kPieceBytes || max_slab > (int64_t)kMaxPieces * kPieceBytes) return false;
  if (total_bytes > max_slab * l.sms) return false;
  int g = l.sms;
  int64_t slab = (total_bytes + g - 1) / g;
  slab = (slab + 127) & ~127ll;
  if (slab < 4096) {  // small tensors: fewer CTAs, at least 4 KiB each
    slab = 4096;
    g = (int)((total_bytes + slab - 1) / slab);
  }
  *grid = g;
  *slab_bytes = (uint32_t)slab;
  return true;
}

int fused_dynamic_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype, void* workspace,
                       float* scale_out, cudaStream_t stream, int grid, uint32_t slab_bytes) {
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  uint8_t* op = static_cast<uint8_t*>(out);
  const int64_t bytes = n * (in_dtype == TNQ_IN_BF16 ? 2 : 4);
  if (in_dtype == TNQ_IN_BF16) {
    if (out_dtype == TNQ_FP8_E4M3)
      return launch_fused<TNQ_IN_BF16, TNQ_FP8_E4M3>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, stream);
    return launch_fused<TNQ_IN_BF16, TNQ_FP8_E5M2>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, stream);
  }
  if (out_dtype == TNQ_FP8_E4M3)
    return launch_fused<TNQ_IN_F32, TNQ_FP8_E4M3>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, stream);
  return launch_fused<TNQ_IN_F32, TNQ_FP8_E5M2>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, stream);
}

}  // namespace tnq_host
