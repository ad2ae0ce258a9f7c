// Row-wise dynamic FP8 cast: per-row amax -> per-row scale -> saturated cast, with
// e4m3 and e5m2 outputs produced from a single read of the row.
//
// A row is owned by a group of G threads (32..256) that keeps its share of the row
// in registers between the amax reduction and the cast, so the input crosses HBM
// once.  Groups of 32 reduce with warp shuffles only; larger groups add one shared
// memory exchange.  The grid is persistent (resident CTAs only) and strides over
// row groups.  The default kernel loads rows straight into registers with 256-bit
// global loads; a variant that stages rows in shared memory with bulk async copies
// (TMA) ahead of the consumers is kept behind tnq_rowwise_set_tma (slower here).
// Rows longer than 32 KiB take a two-pass kernel whose second read comes from L1/L2.
#include <atomic>

#include "common.cuh"

namespace tnq {

constexpr int kRowThreads = 256;
#ifndef TNQ_ROW_PREFETCH
#define TNQ_ROW_PREFETCH 1
#endif

template <int IN>
struct RowIn;
template <>
struct RowIn<TNQ_IN_BF16> {
  static constexpr int kElemsPerVec = 16;
  // integer max on the magnitude bits: a NaN (bits above infinity) wins, which is what
  // marks a row as non-finite below
  __device__ static __forceinline__ uint32_t absmax(uint32_t m, const Vec32B& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = absmax_bf16x2(m, v.w[i]);
    return m;
  }
  __device__ static __forceinline__ uint32_t fold(uint32_t m) { return fold_u16x2(m) << 16; }
};
template <>
struct RowIn<TNQ_IN_F32> {
  static constexpr int kElemsPerVec = 8;
  __device__ static __forceinline__ uint32_t absmax(uint32_t m, const Vec32B& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = max(m, v.w[i] & 0x7fffffffu);
    return m;
  }
  __device__ static __forceinline__ uint32_t fold(uint32_t m) { return m; }
};

// FINITE: the row's amax is finite, so no product can be NaN and the per-word NaN
// check (needed to give a NaN the sign the CPU cast gives it) is skipped.
template <int IN, int OUT, bool FINITE>
__device__ __forceinline__ void row_quant_store(const Vec32B& v, float s, uint8_t* q_row, int64_t vec) {
  const uint4 lo = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]), hi = make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]);
  if constexpr (IN == TNQ_IN_BF16) {
    const uint2 a = FINITE ? quant8_bf16_finite<OUT>(lo, s) : quant8_bf16<OUT, true>(lo, s);
    const uint2 b = FINITE ? quant8_bf16_finite<OUT>(hi, s) : quant8_bf16<OUT, true>(hi, s);
    stg128(q_row + vec * 16, make_uint4(a.x, a.y, b.x, b.y));
  } else {
    uint2 o;
    o.x = FINITE ? quant4_f32_finite<OUT>(lo, s) : quant4_f32<OUT, true>(lo, s);
    o.y = FINITE ? quant4_f32_finite<OUT>(hi, s) : quant4_f32<OUT, true>(hi, s);
    stg64(q_row + vec * 8, o);
  }
}

// Both formats from one widening of the input (finite rows only): 16 bf16 -> 16 e4m3 + 16 e5m2.
__device__ __forceinline__ void row_quant_store_both_bf16(const Vec32B& v, float s43, float s52, uint8_t* q43_row,
                                                          uint8_t* q52_row, int64_t vec) {
  uint32_t a[4], b[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float x0 = bf16lo(v.w[2 * i]), x1 = bf16hi(v.w[2 * i]), x2 = bf16lo(v.w[2 * i + 1]), x3 = bf16hi(v.w[2 * i + 1]);
    a[i] = cvt_fp8x4<TNQ_FP8_E4M3>(__fmul_rn(x0, s43), __fmul_rn(x1, s43), __fmul_rn(x2, s43), __fmul_rn(x3, s43));
    b[i] = cvt_fp8x4<TNQ_FP8_E5M2>(__fmul_rn(x0, s52), __fmul_rn(x1, s52), __fmul_rn(x2, s52), __fmul_rn(x3, s52));
  }
  stg128(q43_row + vec * 16, make_uint4(a[0], a[1], a[2], a[3]));
  stg128(q52_row + vec * 16, make_uint4(b[0], b[1], b[2], b[3]));
}

// G threads per row, up to VPT 32-byte vectors per thread held in registers.
template <int IN, int G, int VPT>
__global__ void __launch_bounds__(kRowThreads)
    k_rowwise(const uint8_t* __restrict__ x, int64_t rows, int64_t cols, int nvec_row, uint8_t* __restrict__ q43,
              float* __restrict__ s43, uint8_t* __restrict__ q52, float* __restrict__ s52) {
  using T = RowIn<IN>;
  constexpr int kGroups = kRowThreads / G;
  __shared__ uint32_t s_part[kRowThreads / 32];
  const int g = threadIdx.x / G;
  const int t = threadIdx.x % G;
  const int64_t row_bytes = (int64_t)nvec_row * 32;
  const int64_t n_steps = (rows + kGroups - 1) / kGroups;  // identical trip count for every thread of a CTA

  // Where the registers allow (bf16, VPT <= 2) the next row's loads are issued before this row's
  // reduction and cast, so a CTA always has two rows of reads in flight.
  constexpr bool kPrefetch = TNQ_ROW_PREFETCH && VPT <= 2;
  auto load_row = [&](Vec32B (&dst)[VPT], int64_t step) {
    const int64_t r = step * kGroups + g;
    const bool ok = step < n_steps && r < rows;
    const uint8_t* xr = x + r * row_bytes;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = t + k * G;
      if (ok && vi < nvec_row) {
        dst[k] = ldg256(xr + (int64_t)vi * 32);
      } else {
#pragma unroll
        for (int w = 0; w < 8; ++w) dst[k].w[w] = 0u;
      }
    }
  };
  Vec32B v[VPT], vn[kPrefetch ? VPT : 1];
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  load_row(v, blockIdx.x);
  for (int64_t step = blockIdx.x; step < n_steps; step += gridDim.x) {
    const int64_t r = step * kGroups + g;
    const bool live = r < rows;
    if constexpr (kPrefetch) load_row(vn, step + gridDim.x);
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < VPT; ++k) m = T::absmax(m, v[k]);
    m = T::fold(m);
    if constexpr (G == 32) {
      m = warp_max_u32(m);
    } else {
      constexpr int kWarpsPerGroup = G / 32;
      m = warp_max_u32(m);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
      __syncthreads();
      uint32_t mm = 0;
#pragma unroll
      for (int w = 0; w < kWarpsPerGroup; ++w) mm = max(mm, s_part[g * kWarpsPerGroup + w]);
      m = mm;
    }
    do {
    if (!live) break;
    const float amax = __uint_as_float(m);
    const bool finite = m < 0x7f800000u;  // uniform over the row's threads
    if constexpr (IN == TNQ_IN_BF16) {
      if (finite && q43 && q52) {
        const float sa = scale_from_amax(amax, 448.0f), sb = scale_from_amax(amax, 57344.0f);
        if (t == 0) s43[r] = sa, s52[r] = sb;
        uint8_t* qa = q43 + r * cols;
        uint8_t* qb = q52 + r * cols;
#pragma unroll
        for (int k = 0; k < VPT; ++k)
          if (t + k * G < nvec_row) row_quant_store_both_bf16(v[k], sa, sb, qa, qb, t + k * G);
        break;
      }
    }
    if (q43) {
      const float s = scale_from_amax(amax, 448.0f);
      if (t == 0) s43[r] = s;
      uint8_t* qr = q43 + r * cols;
      if (finite) {
#pragma unroll
        for (int k = 0; k < VPT; ++k)
          if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E4M3, true>(v[k], s, qr, t + k * G);
      } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k)
          if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E4M3, false>(v[k], s, qr, t + k * G);
      }
    }
    if (q52) {
      const float s = scale_from_amax(amax, 57344.0f);
      if (t == 0) s52[r] = s;
      uint8_t* qr = q52 + r * cols;
      if (finite) {
#pragma unroll
        for (int k = 0; k < VPT; ++k)
          if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E5M2, true>(v[k], s, qr, t + k * G);
      } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k)
          if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E5M2, false>(v[k], s, qr, t + k * G);
      }
    }
    } while (false);
    if constexpr (kPrefetch) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) v[k] = vn[k];
    } else {
      load_row(v, step + gridDim.x);
    }
  }
}

// ---------------------------------------------------------------- TMA-staged variant
// Same ownership (G threads per row, the row's share in registers between amax and
// cast) but the rows reach the CTA through a ring of shared-memory stages filled by
// bulk async copies (cp.async.bulk + mbarrier): one elected thread keeps kStages - 1
// row groups in flight ahead of the consumers, so HBM latency is hidden by the ring
// depth instead of by occupancy.  Threads read 16-byte units (consecutive lanes,
// consecutive units: conflict-free) and write 8-byte units.
template <int IN, int OUT, bool FINITE>
__device__ __forceinline__ void unit_quant_store(const uint4& v, float s, uint8_t* q_row, int unit) {
  if constexpr (IN == TNQ_IN_BF16) {
    stg64(q_row + unit * 8, FINITE ? quant8_bf16_finite<OUT>(v, s) : quant8_bf16<OUT, true>(v, s));
  } else {
    stg32(q_row + unit * 4, FINITE ? quant4_f32_finite<OUT>(v, s) : quant4_f32<OUT, true>(v, s));
  }
}

template <int IN, int G, int UPT>
__global__ void __launch_bounds__(kRowThreads)
    k_rowwise_tma(const uint8_t* __restrict__ x, int64_t rows, int64_t cols, int nunit_row, int stages,
                  uint8_t* __restrict__ q43, float* __restrict__ s43, uint8_t* __restrict__ q52,
                  float* __restrict__ s52, uint32_t* status) {
  constexpr int kGroups = kRowThreads / G;
  extern __shared__ uint8_t tnq_row_smem[];
  __shared__ uint32_t s_part[kRowThreads / 32];
  const uint32_t a0 = smem_u32(tnq_row_smem);
  uint8_t* base = tnq_row_smem + ((128u - (a0 & 127u)) & 127u);
  uint64_t* full = reinterpret_cast<uint64_t*>(base);  // up to 16 barriers
  uint8_t* ring = base + 128;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const uint32_t row_bytes = (uint32_t)nunit_row * 16u;
  const uint32_t stage_bytes = row_bytes * kGroups;
  const int64_t n_steps = (rows + kGroups - 1) / kGroups;
  const int64_t first = blockIdx.x;
  const int64_t count = first < n_steps ? (n_steps - first + gridDim.x - 1) / gridDim.x : 0;

  auto issue = [&](int64_t k) {  // thread 0 only: load the rows of this CTA's k-th step
    const int s = (int)(k % stages);
    const int64_t r0 = (first + k * gridDim.x) * kGroups;
    const int64_t live = (rows - r0 < kGroups) ? rows - r0 : kGroups;
    const uint32_t bytes = (uint32_t)live * row_bytes;
    mbar_expect_tx(&full[s], bytes);
    bulk_g2s(ring + (size_t)s * stage_bytes, x + r0 * row_bytes, bytes, &full[s]);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  if (threadIdx.x == 0)
    for (int64_t k = 0; k < stages && k < count; ++k) issue(k);

  for (int64_t k = 0; k < count; ++k) {
    const int s = (int)(k % stages);
    if (!mbar_wait(&full[s], (uint32_t)((k / stages) & 1))) {
      if (threadIdx.x == 0 && status) atomicExch(status, (uint32_t)TNQ_ETIMEOUT);
      return;
    }
    const int64_t r = (first + k * gridDim.x) * kGroups + g;
    const bool live = r < rows;
    const uint8_t* src = ring + (size_t)s * stage_bytes + (size_t)g * row_bytes;
    uint4 v[UPT];
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < UPT; ++j) {
      const int u = t + j * G;
      if (live && u < nunit_row) {
        v[j] = *reinterpret_cast<const uint4*>(src + u * 16);
      } else {
        v[j] = make_uint4(0u, 0u, 0u, 0u);
      }
      if constexpr (IN == TNQ_IN_BF16) {
        m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(m, v[j].x), v[j].y), v[j].z), v[j].w);
      } else {
        m = max(max(m, v[j].x & 0x7fffffffu), max(max(v[j].y & 0x7fffffffu, v[j].z & 0x7fffffffu), v[j].w & 0x7fffffffu));
      }
    }
    if constexpr (IN == TNQ_IN_BF16) m = fold_u16x2(m) << 16;
    m = warp_max_u32(m);
    __syncthreads();  // every thread has consumed its units of stage s (and s_part of the previous step)
    if (threadIdx.x == 0 && k + stages < count) issue(k + stages);
    if constexpr (G > 32) {
      constexpr int kWarpsPerGroup = G / 32;
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
      __syncthreads();
      uint32_t mm = 0;
#pragma unroll
      for (int w = 0; w < kWarpsPerGroup; ++w) mm = max(mm, s_part[g * kWarpsPerGroup + w]);
      m = mm;
    }
    if (!live) continue;
    const float amax = __uint_as_float(m);
    const bool finite = m < 0x7f800000u;
    if (q43) {
      const float sc = scale_from_amax(amax, 448.0f);
      if (t == 0) s43[r] = sc;
      uint8_t* qr = q43 + r * cols;
      if (finite) {
#pragma unroll
        for (int j = 0; j < UPT; ++j)
          if (t + j * G < nunit_row) unit_quant_store<IN, TNQ_FP8_E4M3, true>(v[j], sc, qr, t + j * G);
      } else {
#pragma unroll
        for (int j = 0; j < UPT; ++j)
          if (t + j * G < nunit_row) unit_quant_store<IN, TNQ_FP8_E4M3, false>(v[j], sc, qr, t + j * G);
      }
    }
    if (q52) {
      const float sc = scale_from_amax(amax, 57344.0f);
      if (t == 0) s52[r] = sc;
      uint8_t* qr = q52 + r * cols;
      if (finite) {
#pragma unroll
        for (int j = 0; j < UPT; ++j)
          if (t + j * G < nunit_row) unit_quant_store<IN, TNQ_FP8_E5M2, true>(v[j], sc, qr, t + j * G);
      } else {
#pragma unroll
        for (int j = 0; j < UPT; ++j)
          if (t + j * G < nunit_row) unit_quant_store<IN, TNQ_FP8_E5M2, false>(v[j], sc, qr, t + j * G);
      }
    }
  }
}

// Any row length that is a whole number of 32-byte vectors: one CTA per row, two
// passes over the row (the second one is served by L1/L2).
template <int IN>
__global__ void __launch_bounds__(kRowThreads)
    k_rowwise_long(const uint8_t* __restrict__ x, int64_t rows, int64_t cols, int64_t nvec_row,
                   uint8_t* __restrict__ q43, float* __restrict__ s43, uint8_t* __restrict__ q52,
                   float* __restrict__ s52) {
  using T = RowIn<IN>;
  __shared__ uint32_t smem32[33];
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint8_t* xr = x + r * nvec_row * 32;
    uint32_t m = 0;
    for (int64_t vi = threadIdx.x; vi < nvec_row; vi += blockDim.x) {
      Vec32B v;
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(xr + vi * 32));
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(xr + vi * 32 + 16));
      v.w[0] = a.x, v.w[1] = a.y, v.w[2] = a.z, v.w[3] = a.w, v.w[4] = b.x, v.w[5] = b.y, v.w[6] = b.z, v.w[7] = b.w;
      m = T::absmax(m, v);
    }
    m = block_max_u32(T::fold(m), smem32);
    const float amax = __uint_as_float(m);
    const float sa = scale_from_amax(amax, 448.0f), sb = scale_from_amax(amax, 57344.0f);
    if (threadIdx.x == 0) {
      if (q43) s43[r] = sa;
      if (q52) s52[r] = sb;
    }
    for (int64_t vi = threadIdx.x; vi < nvec_row; vi += blockDim.x) {
      Vec32B v;
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(xr + vi * 32));
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(xr + vi * 32 + 16));
      v.w[0] = a.x, v.w[1] = a.y, v.w[2] = a.z, v.w[3] = a.w, v.w[4] = b.x, v.w[5] = b.y, v.w[6] = b.z, v.w[7] = b.w;
      if (q43) row_quant_store<IN, TNQ_FP8_E4M3, false>(v, sa, q43 + r * cols, vi);
      if (q52) row_quant_store<IN, TNQ_FP8_E5M2, false>(v, sb, q52 + r * cols, vi);
    }
  }
}

}  // namespace tnq

using namespace tnq;
using namespace tnq_host;

template <auto Kernel>
static int row_resident_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, kRowThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

template <int IN, int G, int VPT>
static int launch_rowwise(const uint8_t* x, int64_t rows, int64_t cols, int nvec_row, uint8_t* q43, float* s43,
                          uint8_t* q52, float* s52, cudaStream_t stream) {
  constexpr int kGroups = kRowThreads / G;
  const int64_t steps = (rows + kGroups - 1) / kGroups;
  const int64_t cap = row_resident_ctas<k_rowwise<IN, G, VPT>>();
  const int grid = (int)(steps < cap ? steps : cap);
  return launch_chained(k_rowwise<IN, G, VPT>, dim3(grid), dim3(kRowThreads), 0, stream, x, rows, cols, nvec_row, q43, s43, q52, s52);
}

template <int IN, int G>
static int pick_vpt(int per_thread, const uint8_t* x, int64_t rows, int64_t cols, int nvec_row, uint8_t* q43,
                    float* s43, uint8_t* q52, float* s52, cudaStream_t stream) {
  if (per_thread <= 1) return launch_rowwise<IN, G, 1>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
  if (per_thread <= 2) return launch_rowwise<IN, G, 2>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
  return launch_rowwise<IN, G, 4>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
}

static std::atomic<int> g_rowwise_tma{0};
static std::atomic<int> g_rowwise_group{0};  // 0 = automatic, else force 32/64/128/256 threads per row where legal
extern "C" int tnq_rowwise_set_tma(int on) {
  g_rowwise_tma = on ? 1 : 0;
  return TNQ_OK;
}
extern "C" int tnq_rowwise_set_group(int threads_per_row) {
  if (threads_per_row != 0 && threads_per_row != 32 && threads_per_row != 64 && threads_per_row != 128 &&
      threads_per_row != 256)
    return TNQ_EINVAL;
  g_rowwise_group = threads_per_row;
  return TNQ_OK;
}

template <int IN, int G, int UPT>
static int launch_rowwise_tma(const uint8_t* x, int64_t rows, int64_t cols, int nunit_row, uint8_t* q43, float* s43,
                              uint8_t* q52, float* s52, uint32_t* status, cudaStream_t stream) {
  constexpr int kGroups = kRowThreads / G;
  const int64_t stage_bytes = (int64_t)nunit_row * 16 * kGroups;
  int stages = (int)(49152 / stage_bytes);
  if (stages < 2) stages = 2;
  if (stages > 8) stages = 8;
  const int smem = (int)(stages * stage_bytes) + 256;
  static int configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(k_rowwise_tma<IN, G, UPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cuda_fail(e);
    configured[dev] = 200 * 1024;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_rowwise_tma<IN, G, UPT>, kRowThreads, smem) != cudaSuccess ||
      per_sm < 1)
    per_sm = 1;
  const int64_t steps = (rows + kGroups - 1) / kGroups;
  const int64_t cap = (int64_t)per_sm * sm_count();
  const int grid = (int)(steps < cap ? steps : cap);
  return launch_chained(k_rowwise_tma<IN, G, UPT>, dim3(grid), dim3(kRowThreads), smem, stream, x, rows, cols, nunit_row, stages, q43,
                        s43, q52, s52, status);
}

template <int IN, int G>
static int pick_upt(int per_thread, const uint8_t* x, int64_t rows, int64_t cols, int nunit_row, uint8_t* q43, float* s43,
                    uint8_t* q52, float* s52, uint32_t* status, cudaStream_t stream) {
  if (per_thread <= 1) return launch_rowwise_tma<IN, G, 1>(x, rows, cols, nunit_row, q43, s43, q52, s52, status, stream);
  if (per_thread <= 2) return launch_rowwise_tma<IN, G, 2>(x, rows, cols, nunit_row, q43, s43, q52, s52, status, stream);
  if (per_thread <= 4) return launch_rowwise_tma<IN, G, 4>(x, rows, cols, nunit_row, q43, s43, q52, s52, status, stream);
  return launch_rowwise_tma<IN, G, 8>(x, rows, cols, nunit_row, q43, s43, q52, s52, status, stream);
}

// rows of up to 2048 16-byte units (32 KiB) through the TMA ring
template <int IN>
static int rowwise_tma_in(const uint8_t* x, int64_t rows, int64_t cols, int nunit, uint8_t* q43, float* s43, uint8_t* q52,
                          float* s52, uint32_t* status, cudaStream_t stream) {
  if (nunit >= 256) return pick_upt<IN, 256>((nunit + 255) / 256, x, rows, cols, nunit, q43, s43, q52, s52, status, stream);
  if (nunit >= 128) return pick_upt<IN, 128>((nunit + 127) / 128, x, rows, cols, nunit, q43, s43, q52, s52, status, stream);
  if (nunit >= 64) return pick_upt<IN, 64>((nunit + 63) / 64, x, rows, cols, nunit, q43, s43, q52, s52, status, stream);
  return pick_upt<IN, 32>((nunit + 31) / 32, x, rows, cols, nunit, q43, s43, q52, s52, status, stream);
}

template <int IN>
static int rowwise_in(const uint8_t* x, int64_t rows, int64_t cols, uint8_t* q43, float* s43, uint8_t* q52,
                      float* s52, uint32_t* status, cudaStream_t stream) {
  const int64_t nvec_row = cols / RowIn<IN>::kElemsPerVec;
  if (g_rowwise_tma && nvec_row * 2 <= 2048)
    return rowwise_tma_in<IN>(x, rows, cols, (int)(nvec_row * 2), q43, s43, q52, s52, status, stream);
  if (nvec_row > 4 * 256) {
    const int64_t cap = row_resident_ctas<k_rowwise_long<IN>>();
    const int grid = (int)(rows < cap ? rows : cap);
    return launch_chained(k_rowwise_long<IN>, dim3(grid), dim3(kRowThreads), 0, stream, x, rows, cols, nvec_row, q43, s43, q52, s52);
  }
  const int nv = (int)nvec_row;
  // largest group that still gives every thread a vector: more threads per row means fewer
  // registers per thread and more resident CTAs to overlap one row's loads with another's math
  const int gsel = g_rowwise_group;
  if ((gsel == 0 && nv >= 256) || gsel == 256 || nv > 4 * 128)
    return pick_vpt<IN, 256>((nv + 255) / 256, x, rows, cols, nv, q43, s43, q52, s52, stream);
  if ((gsel == 0 && nv >= 128) || gsel == 128 || nv > 4 * 64)
    return pick_vpt<IN, 128>((nv + 127) / 128, x, rows, cols, nv, q43, s43, q52, s52, stream);
  if ((gsel == 0 && nv >= 64) || gsel == 64 || nv > 4 * 32)
    return pick_vpt<IN, 64>((nv + 63) / 64, x, rows, cols, nv, q43, s43, q52, s52, stream);
  return pick_vpt<IN, 32>((nv + 31) / 32, x, rows, cols, nv, q43, s43, q52, s52, stream);
}

extern "C" int tnq_fp8_rowwise(const void* x, int64_t rows, int64_t cols, int in_dtype, void* q_e4m3,
                               float* scale_e4m3, void* q_e5m2, float* scale_e5m2, uint32_t* status,
                               tnq_stream_t stream) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16 && in_dtype != TNQ_IN_F32) return TNQ_EUNSUPPORTED;
  if (q_e4m3 == nullptr && q_e5m2 == nullptr) return TNQ_EINVAL;
  if ((q_e4m3 && !scale_e4m3) || (q_e5m2 && !scale_e5m2)) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (x == nullptr) return TNQ_EINVAL;
  const int epv = in_dtype == TNQ_IN_BF16 ? 16 : 8;
  if (cols % epv != 0) return TNQ_ESHAPE;  // rows must be whole 32-byte vectors
  if ((reinterpret_cast<uintptr_t>(x) & 31u) != 0) return TNQ_EALIGN;
  if ((q_e4m3 && !aligned16(q_e4m3)) || (q_e5m2 && !aligned16(q_e5m2))) return TNQ_EALIGN;
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  uint8_t* a = static_cast<uint8_t*>(q_e4m3);
  uint8_t* b = static_cast<uint8_t*>(q_e5m2);
  if (in_dtype == TNQ_IN_BF16) return rowwise_in<TNQ_IN_BF16>(xp, rows, cols, a, scale_e4m3, b, scale_e5m2, status, stream);
  return rowwise_in<TNQ_IN_F32>(xp, rows, cols, a, scale_e4m3, b, scale_e5m2, status, stream);
}
