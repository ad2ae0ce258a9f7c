// Row-wise dynamic FP8 cast: per-row amax -> per-row scale -> saturated cast, with
// e4m3 and e5m2 outputs produced from a single read of the row.
//
// A row is owned by a group of G threads (32..256) that keeps its share of the row
// in registers between the amax reduction and the cast, so the input crosses HBM
// once.  Groups of 32 reduce with warp shuffles only; larger groups add one shared
// memory exchange.  The grid is persistent (resident CTAs only) and strides over
// row groups.  Rows longer than the register budget take a two-pass kernel whose
// second read comes from L1/L2.
#include "common.cuh"

namespace tnq {

constexpr int kRowThreads = 256;

template <int IN>
struct RowIn;
template <>
struct RowIn<TNQ_IN_BF16> {
  static constexpr int kElemsPerVec = 16;
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

template <int IN, int OUT>
__device__ __forceinline__ void row_quant_store(const Vec32B& v, float s, uint8_t* q_row, int64_t vec) {
  if constexpr (IN == TNQ_IN_BF16) {
    const uint2 a = quant8_bf16<OUT, true>(make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]), s);
    const uint2 b = quant8_bf16<OUT, true>(make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]), s);
    stg128(q_row + vec * 16, make_uint4(a.x, a.y, b.x, b.y));
  } else {
    uint2 o;
    o.x = quant4_f32<OUT, true>(make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]), s);
    o.y = quant4_f32<OUT, true>(make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]), s);
    stg64(q_row + vec * 8, o);
  }
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

  for (int64_t step = blockIdx.x; step < n_steps; step += gridDim.x) {
    const int64_t r = step * kGroups + g;
    const bool live = r < rows;
    const uint8_t* xr = x + r * row_bytes;
    Vec32B v[VPT];
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = t + k * G;
      if (live && vi < nvec_row) {
        v[k] = ldg256(xr + (int64_t)vi * 32);
      } else {
#pragma unroll
        for (int w = 0; w < 8; ++w) v[k].w[w] = 0u;
      }
    }
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
    if (!live) continue;
    const float amax = __uint_as_float(m);
    if (q43) {
      const float s = scale_from_amax(amax, 448.0f);
      if (t == 0) s43[r] = s;
      uint8_t* qr = q43 + r * cols;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E4M3>(v[k], s, qr, t + k * G);
    }
    if (q52) {
      const float s = scale_from_amax(amax, 57344.0f);
      if (t == 0) s52[r] = s;
      uint8_t* qr = q52 + r * cols;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        if (t + k * G < nvec_row) row_quant_store<IN, TNQ_FP8_E5M2>(v[k], s, qr, t + k * G);
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
      if (q43) row_quant_store<IN, TNQ_FP8_E4M3>(v, sa, q43 + r * cols, vi);
      if (q52) row_quant_store<IN, TNQ_FP8_E5M2>(v, sb, q52 + r * cols, vi);
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
  k_rowwise<IN, G, VPT><<<grid, kRowThreads, 0, stream>>>(x, rows, cols, nvec_row, q43, s43, q52, s52);
  return check_launch();
}

template <int IN, int G>
static int pick_vpt(int per_thread, const uint8_t* x, int64_t rows, int64_t cols, int nvec_row, uint8_t* q43,
                    float* s43, uint8_t* q52, float* s52, cudaStream_t stream) {
  if (per_thread <= 1) return launch_rowwise<IN, G, 1>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
  if (per_thread <= 2) return launch_rowwise<IN, G, 2>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
  return launch_rowwise<IN, G, 4>(x, rows, cols, nvec_row, q43, s43, q52, s52, stream);
}

template <int IN>
static int rowwise_in(const uint8_t* x, int64_t rows, int64_t cols, uint8_t* q43, float* s43, uint8_t* q52,
                      float* s52, cudaStream_t stream) {
  const int64_t nvec_row = cols / RowIn<IN>::kElemsPerVec;
  if (nvec_row > 4 * 256) {
    const int64_t cap = row_resident_ctas<k_rowwise_long<IN>>();
    const int grid = (int)(rows < cap ? rows : cap);
    k_rowwise_long<IN><<<grid, kRowThreads, 0, stream>>>(x, rows, cols, nvec_row, q43, s43, q52, s52);
    return check_launch();
  }
  const int nv = (int)nvec_row;
  if (nv <= 4 * 32) return pick_vpt<IN, 32>((nv + 31) / 32, x, rows, cols, nv, q43, s43, q52, s52, stream);
  if (nv <= 4 * 64) return pick_vpt<IN, 64>((nv + 63) / 64, x, rows, cols, nv, q43, s43, q52, s52, stream);
  if (nv <= 4 * 128) return pick_vpt<IN, 128>((nv + 127) / 128, x, rows, cols, nv, q43, s43, q52, s52, stream);
  return pick_vpt<IN, 256>((nv + 255) / 256, x, rows, cols, nv, q43, s43, q52, s52, stream);
}

extern "C" int tnq_fp8_rowwise(const void* x, int64_t rows, int64_t cols, int in_dtype, void* q_e4m3,
                               float* scale_e4m3, void* q_e5m2, float* scale_e5m2, tnq_stream_t stream) {
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
  if (in_dtype == TNQ_IN_BF16) return rowwise_in<TNQ_IN_BF16>(xp, rows, cols, a, scale_e4m3, b, scale_e5m2, stream);
  return rowwise_in<TNQ_IN_F32>(xp, rows, cols, a, scale_e4m3, b, scale_e5m2, stream);
}
