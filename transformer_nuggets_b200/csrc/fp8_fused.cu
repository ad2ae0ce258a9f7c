// Single-launch dynamic per-tensor FP8 cast for tensors that fit in the shared
// memory of the whole GPU (148 SMs x ~226 KB = 33.5 MB: a 4096 x 4096 bf16 tensor
// just fits).
//
// One CTA per SM, all resident together (see launch_fused for how that is ensured).  Each CTA
// owns a contiguous slab of the tensor and brings it into shared memory with bulk
// async copies (cp.async.bulk, 32 KiB pieces, one mbarrier each, all in flight at
// once).  As pieces land the CTA folds |x| maxima; a grid-wide exchange (one max, one
// arrival counter, one polled 64-bit word; bounded wait) gives every CTA the tensor's
// maximum; then every CTA casts its slab straight out of shared memory.  The input
// crosses HBM exactly once and the two-launch gap of the general path disappears.
#include "common.cuh"

namespace tnq {

constexpr int kFusedThreads = 1024;
constexpr int kPieceBytes = 32768;
constexpr int kMaxPieces = 8;
constexpr int kFusedHeaderBytes = 512;  // barriers + reduction scratch in front of the slab
constexpr int kFusedStamps = 8;         // uint64 words per CTA written by the profiled build

// Same memory as the per-tensor Workspace of fp8_tensor.cu.  Words 4..9 belong to this kernel.
struct FusedWorkspace {
  uint32_t ticket;
  uint32_t amax_bits;
  float scale;
  uint32_t status;
  uint32_t reserved0;
  uint32_t bar_gen;  // number of single-launch casts that have run on this workspace (its parity picks the pair)
  // one pair per parity, 8-byte aligned so that one 64-bit load reads both halves:
  // low word = arrivals (wraps to 0 when the last CTA arrives), high word = tensor-wide maximum
  unsigned long long pair[2];
  uint32_t pad[6];
  uint32_t partial[(TNQ_WORKSPACE_BYTES - 64) / 4];
};
static_assert(sizeof(FusedWorkspace) == TNQ_WORKSPACE_BYTES, "workspace layout");

// All CTAs of the grid meet here and leave with the maximum of their contributions.
// Thread 0 of every CTA: a max into the high word of this call's pair, a fence, an increment of the
// low word (which wraps to zero when the last CTA arrives), then it polls the pair with ONE 64-bit
// load until the low word reads zero - the same load delivers the maximum.  Measured beside a
// variant in which every CTA posted its maximum into a slot of its own and all CTAs polled all
// slots: the 740 polling warps queued up on the ten L2 lines that hold the slots and the exchange took
// 5.5 us instead of 2.2 us.  Returns false if the others did not show up within about a second.
__device__ __forceinline__ bool grid_exchange_max(FusedWorkspace* ws, uint32_t parity, uint32_t cta_max, uint32_t* red,
                                                  uint32_t* result) {
  uint32_t& s_val = red[40];  // behind the 33 reduction words (no static shared memory: the slab takes it all)
  uint32_t& s_ok = red[41];
  if (threadIdx.x == 0) {
    uint32_t ok = 1, val = 0;
    uint32_t* words = reinterpret_cast<uint32_t*>(&ws->pair[parity]);  // little endian: [0] arrivals, [1] maximum
    atomicMax(&words[1], cta_max);
    __threadfence();
    const uint32_t t = atomicInc(&words[0], gridDim.x - 1);
    if (t == gridDim.x - 1) {
      val = __ldcg(&words[1]);
    } else {
      uint64_t t0 = 0;
      for (uint32_t it = 0;; ++it) {
        unsigned long long w;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(&ws->pair[parity]) : "memory");
        if ((uint32_t)w == 0u) {
          val = (uint32_t)(w >> 32);
          break;
        }
        if ((it & 63u) == 63u) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > 1000000000ull) {
            ok = 0;
            break;
          }
        }
      }
    }
    s_val = val;
    s_ok = ok;
  }
  __syncthreads();
  *result = s_val;
  return s_ok != 0;
}

template <int IN>
__device__ __forceinline__ uint32_t fused_absmax(uint32_t m, const uint4& q) {
  if constexpr (IN == TNQ_IN_BF16) return absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m, q.x), q.y), q.z), q.w);
  else return max(max(m, q.x & 0x7fffffffu), max(max(q.y & 0x7fffffffu, q.z & 0x7fffffffu), q.w & 0x7fffffffu));
}

template <int IN, int OUT, bool PROF>
__global__ void __launch_bounds__(kFusedThreads, 1)
    k_dynamic_fused(const uint8_t* __restrict__ x, uint8_t* __restrict__ out, int64_t total_bytes, uint32_t slab_bytes,
                    FusedWorkspace* ws, float* scale_out, unsigned long long* stamps) {
  extern __shared__ uint8_t tnq_fused_smem[];
  const uint32_t a = smem_u32(tnq_fused_smem);
  uint8_t* base = tnq_fused_smem + ((128u - (a & 127u)) & 127u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base);       // kMaxPieces barriers
  uint32_t* red = reinterpret_cast<uint32_t*>(base + 128);  // 33 words + 2 for the exchange
  uint8_t* slab = base + kFusedHeaderBytes;
  const uint32_t slab_s = smem_u32(slab);
  unsigned long long t_start = 0, t_loaded = 0, t_exchanged = 0, g_start = 0, g_loaded = 0, g_exchanged = 0;

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
  // launched with programmatic stream serialization the CTA may get here while the previous kernel of the
  // stream still runs: everything that reads what that kernel wrote (the input, the workspace) stays behind this
  pdl_wait();
  pdl_launch_dependents();
  if constexpr (PROF) t_start = clock64(), g_start = globaltimer_ns();  // the stream's previous kernel has finished
  uint32_t gen = 0;
  if (threadIdx.x == 0) {
    for (int p = 0; p < pieces; ++p) {
      const uint32_t off = (uint32_t)p * kPieceBytes;
      const uint32_t len = (my_bytes - off < (uint32_t)kPieceBytes) ? my_bytes - off : (uint32_t)kPieceBytes;
      mbar_expect_tx(&bars[p], len);
      bulk_g2s(slab + off, x + begin + off, len, &bars[p]);
    }
    // written by CTA 0 at the very end of the previous call on this workspace, so stable here
    gen = __ldcg(&ws->bar_gen) + 1u;
  }
  auto close_generation = [&]() {  // CTA 0, thread 0: clear the pair the NEXT call will use, then hand over
    ws->pair[(gen + 1u) & 1u] = 0ull;
    __threadfence();
    ws->bar_gen = gen;
  };

  // ---- amax over the slab, piece by piece as it lands
  uint32_t m = 0;
  bool ok = true;
  for (int p = 0; p < pieces && ok; ++p) {
    ok = mbar_wait(&bars[p], 0);
    if (!ok) break;
    const uint32_t off = (uint32_t)p * kPieceBytes;
    const uint32_t len = (my_bytes - off < (uint32_t)kPieceBytes) ? my_bytes - off : (uint32_t)kPieceBytes;
    for (uint32_t v = threadIdx.x * 16u; v < len; v += kFusedThreads * 16u)
      m = fused_absmax<IN>(m, lds128(slab_s + off + v));
  }
  if (__syncthreads_or(!ok)) {  // a copy never arrived: flag it and leave together
    if (threadIdx.x == 0) atomicExch(&ws->status, (uint32_t)TNQ_ETIMEOUT);
    return;
  }
  if constexpr (IN == TNQ_IN_BF16) m = fold_u16x2(m) << 16;
  m = block_max_u32(m, red);
  if constexpr (PROF) t_loaded = clock64(), g_loaded = globaltimer_ns();
  uint32_t g = 0;
  const bool met = grid_exchange_max(ws, gen & 1u, m, red, &g);
  if (!met) {
    if (threadIdx.x == 0) atomicExch(&ws->status, (uint32_t)TNQ_ETIMEOUT);
    return;
  }
  if constexpr (PROF) t_exchanged = clock64(), g_exchanged = globaltimer_ns();
  const float amax = __uint_as_float(g);
  const float s = scale_from_amax(amax, Fp8Traits<OUT>::kMax);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    close_generation();
    ws->amax_bits = g;
    ws->scale = s;
    if (scale_out) *scale_out = s;
  }
  const bool finite = g < 0x7f800000u;

  // ---- cast the slab out of shared memory: two independent 16-byte pieces per thread and step.
  // Measured beside three other ways out (16-byte stores with lane pairs swapping halves: 3.0 us;
  // converting in place and sending the results off as bulk copies shared -> global: 4.1-4.4 us): these
  // plain 8-byte stores are the fastest (2.4 us for the 16 MiB of output).
  constexpr uint32_t kStep = kFusedThreads * 16u;
  if constexpr (IN == TNQ_IN_BF16) {
    uint8_t* dst = out + begin / 2;
    uint32_t v = threadIdx.x * 16u;
    for (; v + kStep < my_bytes; v += 2 * kStep) {
      const uint4 q0 = lds128(slab_s + v), q1 = lds128(slab_s + v + kStep);
      const uint2 o0 = finite ? quant8_bf16_finite<OUT>(q0, s) : quant8_bf16<OUT, true>(q0, s);
      const uint2 o1 = finite ? quant8_bf16_finite<OUT>(q1, s) : quant8_bf16<OUT, true>(q1, s);
      stg64(dst + v / 2, o0);
      stg64(dst + (v + kStep) / 2, o1);
    }
    if (v < my_bytes) {
      const uint4 q = lds128(slab_s + v);
      stg64(dst + v / 2, finite ? quant8_bf16_finite<OUT>(q, s) : quant8_bf16<OUT, true>(q, s));
    }
  } else {
    uint8_t* dst = out + begin / 4;
    for (uint32_t v = threadIdx.x * 16u; v < my_bytes; v += kStep) {
      const uint4 q = lds128(slab_s + v);
      stg32(dst + v / 4, finite ? quant4_f32_finite<OUT>(q, s) : quant4_f32<OUT, true>(q, s));
    }
  }
  if constexpr (PROF) {
    if (threadIdx.x == 0) {
      unsigned long long* w = stamps + (size_t)blockIdx.x * kFusedStamps;
      w[0] = t_start, w[1] = t_loaded, w[2] = t_exchanged, w[3] = clock64();
      w[4] = g_start, w[5] = g_loaded, w[6] = g_exchanged, w[7] = globaltimer_ns();
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

namespace tnq_host {

int fused_launch_mode();  // fp8_tensor.cu, TNQ_OPT_FUSED_LAUNCH

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

template <int IN, int OUT, bool PROF>
static int launch_fused(const uint8_t* x, uint8_t* out, int64_t total_bytes, int grid, uint32_t slab_bytes, void* ws,
                        float* scale_out, unsigned long long* stamps, cudaStream_t stream) {
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem = (int)slab_bytes + kFusedHeaderBytes + 128;
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(k_dynamic_fused<IN, OUT, PROF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fused_limits().max_smem);
    if (e != cudaSuccess) return cuda_fail(e);
    configured[dev] = fused_limits().max_smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFusedThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // The grid never exceeds one CTA per SM, so a plain launch places every CTA as soon as the SMs are free, and
  // the block scheduler hands out all CTAs of one grid before it turns to the next grid: the CTAs of a call
  // meet in the exchange without the cooperative attribute.  What the attribute adds is a guarantee when
  // other streams hold SMs; without it a call whose CTAs cannot all be placed within the exchange's bound
  // (about a second) reports TNQ_ETIMEOUT in the status word instead of waiting.  What it costs is the
  // chained launch: the runtime honours programmatic stream serialization on a cooperative launch only inside
  // a CUDA graph (measured per call at 4096 x 4096: cooperative 14.4 us eager / 12.6 us replayed, plain +
  // chained 12.5 us / 12.6 us).  TNQ_OPT_FUSED_LAUNCH picks: 1 = plain (default), 0 = cooperative.
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (fused_launch_mode() == 0) {
    attr[na].id = cudaLaunchAttributeCooperative;
    attr[na].val.cooperative = 1;
    ++na;
  }
  if (pdl_chain()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k_dynamic_fused<IN, OUT, PROF>, x, out, total_bytes, slab_bytes,
                                     static_cast<FusedWorkspace*>(ws), scale_out, stamps);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

// Whether the single-launch kernel can take this tensor; fills grid and slab size.
bool fused_plan(int64_t total_bytes, int* grid, uint32_t* slab_bytes) {
  const FusedLimits l = fused_limits();
  if (l.sms <= 0 || l.sms > 256 || !l.coop || total_bytes <= 0 || (total_bytes & 15) != 0) return false;
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
      return launch_fused<TNQ_IN_BF16, TNQ_FP8_E4M3, false>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, nullptr, stream);
    return launch_fused<TNQ_IN_BF16, TNQ_FP8_E5M2, false>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, nullptr, stream);
  }
  if (out_dtype == TNQ_FP8_E4M3)
    return launch_fused<TNQ_IN_F32, TNQ_FP8_E4M3, false>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, nullptr, stream);
  return launch_fused<TNQ_IN_F32, TNQ_FP8_E5M2, false>(xp, op, bytes, grid, slab_bytes, workspace, scale_out, nullptr, stream);
}

}  // namespace tnq_host

// Diagnostic twin of tnq_fp8_dynamic_cast for the single-launch path (bf16 -> e4m3): the same kernel
// compiled with time stamps.  stamps[cta * 8 + i]: SM clock at kernel entry (0), slab loaded and CTA
// maximum known (1), grid-wide exchange done (2), last store issued (3); words 4..7: the global
// nanosecond timer at the same four points.
extern "C" int tnq_fp8_dynamic_cast_profile(const void* x, void* out, int64_t n, void* workspace, float* scale_out,
                                            unsigned long long* stamps, int* grid_out, tnq_stream_t stream) {
  if (x == nullptr || out == nullptr || workspace == nullptr || stamps == nullptr || n <= 0) return TNQ_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 31u) != 0 || !aligned16(out)) return TNQ_EALIGN;
  int grid = 0;
  uint32_t slab = 0;
  if (!fused_plan(n * 2, &grid, &slab)) return TNQ_EUNSUPPORTED;
  if (grid_out) *grid_out = grid;
  return launch_fused<TNQ_IN_BF16, TNQ_FP8_E4M3, true>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), n * 2, grid,
                                                       slab, workspace, scale_out, stamps, stream);
}
