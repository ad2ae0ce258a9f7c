// Per-tensor FP8 casts: amax reduction, scaled cast (delayed scale, optional amax
// side output) and the dynamic cast (amax -> scale -> saturated cast).
//
// All three are HBM streaming kernels.  Persistent grids (a multiple of the SM
// count), grid-stride over 32-byte vectors, 512-thread CTAs with two independent
// 256-bit loads in flight per thread (the best of a sweep over 128..1024 threads and
// unroll 1..8; 640- and 768-thread CTAs lose 7-12 %), |x| maxima on the integer view, one warp `redux` + one shared
// memory step per CTA, and a self-resetting ticket so that the last CTA to finish
// combines the per-CTA partial maxima (no float atomics, no memset between calls).
#include <atomic>

#include "common.cuh"

namespace tnq {

#ifndef TNQ_STREAM_THREADS
#define TNQ_STREAM_THREADS 512
#endif
#ifndef TNQ_STREAM_UNROLL
#define TNQ_STREAM_UNROLL 2
#endif
constexpr int kThreads = TNQ_STREAM_THREADS;
constexpr int kUnroll = TNQ_STREAM_UNROLL;
constexpr int kMaxPartials = (TNQ_WORKSPACE_BYTES - 64) / 4;

struct Workspace {
  uint32_t ticket;
  uint32_t amax_bits;  // fp32 bit pattern
  float scale;
  uint32_t status;
  uint32_t pad[12];
  uint32_t partial[kMaxPartials];
};

// Cross-GPU amax exchange (row-sharded cast).  Every rank owns a slot array in its
// own memory: slot[parity][r] holds rank r's amax for the call with that sequence
// parity as one 64-bit word (sequence number << 32 | fp32 bits), so a single aligned
// store publishes value and flag together.  A rank STORES its word into every peer's
// array (plain peer stores over NVLink, one store per peer) and only ever
// LOADS from its own memory.  Two parities suffice: a rank cannot publish call k+2
// before every peer has consumed call k, because its own call k+1 needs theirs.
constexpr int kMaxRanks = 16;
constexpr int kSlotStride = 64;          // slots per parity in the buffer
constexpr int kExchangeStatusWord = 512; // uint32 index of the status word (byte 2048)
struct PeerSlots {
  uint64_t* base[kMaxRanks];  // base[r] = rank r's slot buffer as seen from this GPU
  int world;
  int rank;
  uint32_t seq;
};
struct ExchangeWait {
  const uint64_t* slots;  // this rank's own buffer; nullptr = not used
  int world;
  uint32_t seq;
  uint32_t* status;
  float* amax_out;
};

// All ranks' amax for sequence `seq` from this GPU's own slots; bounded wait of about
// one second.  Returns false on expiry.
__device__ __forceinline__ bool exchange_collect(const ExchangeWait& ex, float* amax) {
  const uint64_t* slot = ex.slots + (ex.seq & 1u) * kSlotStride;
  uint32_t m = 0;
  uint64_t t0 = 0;
  for (int r = 0; r < ex.world; ++r) {
    for (uint32_t it = 0;; ++it) {
      uint64_t w;
      asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(slot + r) : "memory");
      if ((uint32_t)(w >> 32) == ex.seq) {
        m = max(m, (uint32_t)w);
        break;
      }
      if ((it & 63u) == 63u) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 1000000000ull) return false;
      }
    }
  }
  *amax = __uint_as_float(m);
  return true;
}

template <int IN>
struct InTraits;
template <>
struct InTraits<TNQ_IN_BF16> {
  static constexpr int kElemsPerVec = 16;  // per 32-byte vector
  static constexpr int kElemBytes = 2;
  __device__ static __forceinline__ uint32_t absmax(uint32_t m, const Vec32B& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = absmax_bf16x2_1op(m, v.w[i]);  // sign bits of m are meaningless until fold()
    return m;
  }
  __device__ static __forceinline__ uint32_t fold(uint32_t m) { return fold_u16x2(m & 0x7fff7fffu) << 16; }  // -> fp32 bits
  // both halves of an accumulator below the infinity pattern: everything it saw was finite
  __device__ static __forceinline__ bool all_finite(uint32_t m) { return (((m & 0x7fff7fffu) + 0x00800080u) & 0x80008000u) == 0u; }
  __device__ static __forceinline__ uint32_t merge(uint32_t m, uint32_t vm) { return absmax_bf16x2_1op(m, vm); }
  __device__ static __forceinline__ float load_scalar(const void* x, int64_t i) {
    return bf16bits_to_f32(reinterpret_cast<const uint16_t*>(x)[i]);
  }
};
template <>
struct InTraits<TNQ_IN_F32> {
  static constexpr int kElemsPerVec = 8;
  static constexpr int kElemBytes = 4;
  __device__ static __forceinline__ uint32_t absmax(uint32_t m, const Vec32B& v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = absmax_f32_1op(m, v.w[i]);  // sign bit of m is meaningless until fold()
    return m;
  }
  __device__ static __forceinline__ uint32_t fold(uint32_t m) { return m & 0x7fffffffu; }
  __device__ static __forceinline__ bool all_finite(uint32_t m) { return (m & 0x7fffffffu) < 0x7f800000u; }
  __device__ static __forceinline__ uint32_t merge(uint32_t m, uint32_t vm) { return absmax_f32_1op(m, vm); }
  __device__ static __forceinline__ float load_scalar(const void* x, int64_t i) {
    return reinterpret_cast<const float*>(x)[i];
  }
};

// 32 input bytes -> fp8 bytes, stored.  CHECKED = false skips the per-word NaN test: for callers that have
// established that the vector and the scale are finite (saturated casts only: nothing can then be NaN).
template <int IN, int OUT, bool SAT, bool CHECKED = true>
__device__ __forceinline__ void quant_store(const Vec32B& v, float s, uint8_t* out, int64_t vec_index, bool hint,
                                            uint64_t policy) {
  static_assert(CHECKED || SAT, "the unchecked conversion is for saturated casts");
  if constexpr (IN == TNQ_IN_BF16) {
    const uint4 lo4 = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]), hi4 = make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]);
    uint2 a, b;
    if constexpr (CHECKED) a = quant8_bf16<OUT, SAT>(lo4, s), b = quant8_bf16<OUT, SAT>(hi4, s);
    else a = quant8_bf16_finite<OUT>(lo4, s), b = quant8_bf16_finite<OUT>(hi4, s);
    if (hint) stg128_hint(out + vec_index * 16, make_uint4(a.x, a.y, b.x, b.y), policy);
    else stg128(out + vec_index * 16, make_uint4(a.x, a.y, b.x, b.y));
  } else {
    const uint4 lo4 = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]), hi4 = make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]);
    uint2 o;
    if constexpr (CHECKED) o.x = quant4_f32<OUT, SAT>(lo4, s), o.y = quant4_f32<OUT, SAT>(hi4, s);
    else o.x = quant4_f32_finite<OUT>(lo4, s), o.y = quant4_f32_finite<OUT>(hi4, s);
    if (hint) stg64_hint(out + vec_index * 8, o, policy);
    else stg64(out + vec_index * 8, o);
  }
}

// ADJACENT 32-byte vectors -> 32 fp8 bytes in one store (a 256-bit store when `wide`, i.e. the
// destination is 32-byte aligned): two vectors of bf16 input (64 contiguous bytes), four of fp32 (128).
template <int IN>
struct GroupTraits {
  static constexpr int kVecs = (IN == TNQ_IN_BF16) ? 2 : 4;
};
template <int IN, int OUT, bool SAT, bool CHECKED = true>
__device__ __forceinline__ void quant_store_group(const Vec32B* v, float s, uint8_t* out, int64_t group_index, bool wide) {
  static_assert(CHECKED || SAT, "the unchecked conversion is for saturated casts");
  uint32_t o[8];
  if constexpr (IN == TNQ_IN_BF16) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint4 lo4 = make_uint4(v[k].w[0], v[k].w[1], v[k].w[2], v[k].w[3]), hi4 = make_uint4(v[k].w[4], v[k].w[5], v[k].w[6], v[k].w[7]);
      uint2 a, b;
      if constexpr (CHECKED) a = quant8_bf16<OUT, SAT>(lo4, s), b = quant8_bf16<OUT, SAT>(hi4, s);
      else a = quant8_bf16_finite<OUT>(lo4, s), b = quant8_bf16_finite<OUT>(hi4, s);
      o[4 * k] = a.x, o[4 * k + 1] = a.y, o[4 * k + 2] = b.x, o[4 * k + 3] = b.y;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint4 lo4 = make_uint4(v[k].w[0], v[k].w[1], v[k].w[2], v[k].w[3]), hi4 = make_uint4(v[k].w[4], v[k].w[5], v[k].w[6], v[k].w[7]);
      if constexpr (CHECKED) o[2 * k] = quant4_f32<OUT, SAT>(lo4, s), o[2 * k + 1] = quant4_f32<OUT, SAT>(hi4, s);
      else o[2 * k] = quant4_f32_finite<OUT>(lo4, s), o[2 * k + 1] = quant4_f32_finite<OUT>(hi4, s);
    }
  }
  uint8_t* dst = out + group_index * 32;
  if (wide) {
    stg256(dst, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
  } else {
    stg128(dst, make_uint4(o[0], o[1], o[2], o[3]));
    stg128(dst + 16, make_uint4(o[4], o[5], o[6], o[7]));
  }
}

// Combine the CTA maxima: every CTA publishes its partial, takes a ticket, and the
// CTA holding the last ticket folds all partials.  Returns true (in thread 0 of that
// CTA only) with the tensor-wide maximum as fp32 bits.
__device__ __forceinline__ bool grid_max(uint32_t cta_max_bits, Workspace* ws, uint32_t* smem32,
                                         uint32_t* result_bits) {
  __shared__ uint32_t s_last;
  if (threadIdx.x == 0) {
    ws->partial[blockIdx.x] = cta_max_bits;
    __threadfence();
    const uint32_t t = atomicInc(&ws->ticket, gridDim.x - 1);  // wraps to 0: ready for the next call
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return false;
  __threadfence();
  uint32_t m = 0;
  for (uint32_t i = threadIdx.x; i < gridDim.x; i += blockDim.x) m = max(m, __ldcg(&ws->partial[i]));
  m = block_max_u32(m, smem32);
  *result_bits = m;
  return threadIdx.x == 0;
}

// ---------------------------------------------------------------- amax
template <int IN, bool PUBLISH>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads)
    k_amax(const uint8_t* __restrict__ x, int64_t n, Workspace* ws, float* amax_out, float* scale_out, float fp8_max,
           PeerSlots peers, int64_t keep_from) {
  using T = InTraits<IN>;
  __shared__ uint32_t smem32[33];
  const int64_t nvec = n / T::kElemsPerVec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t m = 0;
  pdl_wait();  // chained launch: the input may come from the stream's previous kernel
  if (keep_from < nvec) {
    // A cast pass over the same tensor follows and walks it from the end: ask L2 to
    // hold on to the tail (vectors >= keep_from) and to let go of the rest first.
    const uint64_t keep = l2_policy_evict_last(), stream = l2_policy_evict_first();
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
      Vec32B v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t j = i + u * stride;
        v[u] = ldg256_hint(x + j * 32, j >= keep_from ? keep : stream);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) m = T::absmax(m, v[u]);
    }
    for (; i < nvec; i += stride) m = T::absmax(m, ldg256_hint(x + i * 32, i >= keep_from ? keep : stream));
  } else {
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
      Vec32B v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) v[u] = ldg256(x + (i + u * stride) * 32);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) m = T::absmax(m, v[u]);
    }
    for (; i < nvec; i += stride) m = T::absmax(m, ldg256(x + i * 32));
  }
  m = T::fold(m);
  if (blockIdx.x == 0) {  // ragged tail, fewer than one vector
    for (int64_t j = nvec * T::kElemsPerVec + threadIdx.x; j < n; j += blockDim.x)
      m = max(m, __float_as_uint(T::load_scalar(x, j)) & 0x7fffffffu);
  }
  m = block_max_u32(m, smem32);
  pdl_launch_dependents();
  uint32_t total;
  if (grid_max(m, ws, smem32, &total)) {
    const float amax = __uint_as_float(total);
    ws->amax_bits = total;
    const float scale = scale_from_amax(amax, fp8_max);
    ws->scale = scale;
    if (amax_out) *amax_out = amax;
    if (scale_out) *scale_out = scale;
    if constexpr (PUBLISH) {
      const uint64_t word = ((uint64_t)peers.seq << 32) | total;
      const int idx = (int)(peers.seq & 1u) * kSlotStride + peers.rank;
      for (int r = 0; r < peers.world; ++r)
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peers.base[r] + idx), "l"(word) : "memory");
    }
  }
}

// One CTA: wait (bounded) for every rank's amax word of this sequence number in this GPU's
// own slot buffer and write their maximum.
__global__ void k_exchange_collect(ExchangeWait ex) {
  pdl_wait();
  if (threadIdx.x == 0) {
    float a = 0.0f;
    if (exchange_collect(ex, &a)) {
      if (ex.amax_out) *ex.amax_out = a;
    } else {
      atomicExch(ex.status, (uint32_t)TNQ_ETIMEOUT);
    }
  }
}

// ---------------------------------------------------------------- cast (optionally + amax)
// The streaming loop of k_cast.  A saturated cast skips the per-word NaN test (`fast`) for a vector when
// nothing in it can become NaN: either everything is known to be finite (`known_finite`, uniform), or - with
// the abs_max side output, where the vector's own maximum is at hand - that maximum and the scale are
// finite.  Returns the thread's running |x| maximum (meaningful with AMAX; sign bits are meaningless).
template <int IN, int OUT, bool SAT, bool AMAX, bool PAIR>
__device__ __forceinline__ uint32_t cast_loop(const uint8_t* __restrict__ x, uint8_t* __restrict__ out, int64_t nvec, float s,
                                              int reverse, int l2_mode, bool known_finite, bool scale_finite) {
  using T = InTraits<IN>;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // reverse != 0 walks the tensor from its end: after an amax pass over the same tensor
  // the most recently read (last) part is the part still in L2.
  const int64_t first = reverse ? nvec - 1 : 0, dir = reverse ? -1 : 1;
  // l2_mode bit 0: loads are last uses (evict first); bit 1: stores are never re-read (evict first)
  const bool hint_ld = (l2_mode & 1) != 0, hint_st = (l2_mode & 2) != 0;
  const uint64_t pol = l2_policy_evict_first();
  uint32_t m = 0;
  auto one_vector = [&](const Vec32B& v, int64_t j) {
    bool fast = known_finite;
    if constexpr (AMAX) {
      const uint32_t vm = T::absmax(0u, v);
      m = T::merge(m, vm);
      fast = fast || (scale_finite && T::all_finite(vm));
    }
    if constexpr (SAT) {
      if (fast) {
        quant_store<IN, OUT, SAT, !SAT>(v, s, out, j, hint_st, pol);
        return;
      }
    }
    quant_store<IN, OUT, SAT>(v, s, out, j, hint_st, pol);
  };
  if constexpr (PAIR) {
    constexpr int K = GroupTraits<IN>::kVecs;
    const int64_t ngroup = nvec / K;
    const bool wide = (reinterpret_cast<uintptr_t>(out) & 31u) == 0;
    for (; i < ngroup; i += stride) {
      const int64_t j = reverse ? ngroup - 1 - i : i;
      Vec32B v[K];
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = ldg256(x + (j * K + k) * 32);
      bool fast = known_finite;
      if constexpr (AMAX) {
        uint32_t vm = 0;
#pragma unroll
        for (int k = 0; k < K; ++k) vm = T::absmax(vm, v[k]);
        m = T::merge(m, vm);
        fast = fast || (scale_finite && T::all_finite(vm));
      }
      if (SAT && fast) quant_store_group<IN, OUT, SAT, !SAT>(v, s, out, j, wide);
      else quant_store_group<IN, OUT, SAT>(v, s, out, j, wide);
    }
    if (blockIdx.x == 0 && threadIdx.x < (unsigned)(nvec - ngroup * K)) {  // fewer than K vectors are left over
      const int64_t j = ngroup * K + threadIdx.x;
      one_vector(ldg256(x + j * 32), j);
    }
  } else {
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
      Vec32B v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const uint8_t* src = x + (first + dir * (i + u * stride)) * 32;
        v[u] = hint_ld ? ldg256_hint(src, pol) : ldg256(src);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) one_vector(v[u], first + dir * (i + u * stride));
    }
    for (; i < nvec; i += stride) {
      const int64_t j = first + dir * i;
      one_vector(hint_ld ? ldg256_hint(x + j * 32, pol) : ldg256(x + j * 32), j);
    }
  }
  return m;
}

// PAIR: a thread takes adjacent vectors per step (64 contiguous bytes of bf16 input) and writes their
// 32 fp8 bytes with one 256-bit store; a warp then reads 2 KiB in one piece.  Used for the forward walk
// over bf16 input (delayed-scale and plain casts: 72.0 -> 66.2 us at 16384 x 8192 with the abs_max side
// output); the reversed walk behind an amax pass keeps two independent far-apart vectors per thread.
template <int IN, int OUT, bool SAT, bool AMAX, bool PAIR>
__global__ void __launch_bounds__(kThreads)
    k_cast(const uint8_t* __restrict__ x, uint8_t* __restrict__ out, int64_t n, const float* scale_ptr,
           int scale_source, float* abs_max_inout, Workspace* ws, ExchangeWait ex, int reverse, int l2_mode) {
  using T = InTraits<IN>;
  __shared__ uint32_t smem32[33];
  // The scale may come from the preceding amax launch: wait for it - except on the exchange path.  There the cast
  // takes nothing from that launch but the slot words it polls below, and everything older in the stream was complete
  // before the amax launch got past its own wait.  Without the wait the cast does not sit behind the amax kernel's
  // completion, which includes the acknowledgement of its stores into the peers' memory (one per rank).
  // The abs_max variants never run on the exchange path and keep the unconditional wait: with the condition in
  // them the compiler allocates the kernel differently (32 instead of 39 registers) and the delayed-scale cast
  // loses 2 % (64.8-65.1 -> 66.2-66.8 us at 16384 x 8192).
  if constexpr (AMAX) pdl_wait();
  else pdl_wait_if(ex.slots == nullptr || (l2_mode & 8) != 0);
  pdl_launch_dependents();
  float s;
  if (ex.slots != nullptr) {  // amax of all ranks, read from this GPU's own slots
    __shared__ float s_amax;
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
      float a = 0.0f;
      s_ok = exchange_collect(ex, &a) ? 1 : 0;
      s_amax = a;
      if (!s_ok) atomicExch(ex.status, (uint32_t)TNQ_ETIMEOUT);
      else if (blockIdx.x == 0 && ex.amax_out) *ex.amax_out = a;
    }
    __syncthreads();
    if (!s_ok) return;
    s = scale_from_amax(s_amax, Fp8Traits<OUT>::kMax);
  } else {
    s = *reinterpret_cast<const volatile float*>(scale_ptr);
    if (scale_source == TNQ_SCALE_IS_AMAX) s = scale_from_amax(s, Fp8Traits<OUT>::kMax);
  }

  const int64_t nvec = n / T::kElemsPerVec;
  // A saturated cast whose scale is this tensor's own fp8_max / amax (the caller says so: l2_mode bit 2) and is
  // finite and non-zero had a finite, non-zero amax: every element is finite and no product can be NaN.
  const bool scale_finite = (__float_as_uint(s) & 0x7fffffffu) < 0x7f800000u;
  const bool known_finite = SAT && (l2_mode & 4) != 0 && scale_finite && s != 0.0f;
  uint32_t m = cast_loop<IN, OUT, SAT, AMAX, PAIR>(x, out, nvec, s, reverse, l2_mode, known_finite, scale_finite);
  if constexpr (AMAX) m = T::fold(m);
  if (blockIdx.x == 0) {
    for (int64_t j = nvec * T::kElemsPerVec + threadIdx.x; j < n; j += blockDim.x) {
      const float xv = T::load_scalar(x, j);
      if constexpr (AMAX) m = max(m, __float_as_uint(xv) & 0x7fffffffu);
      out[j] = (uint8_t)fp8_scalar_exact<OUT, SAT>(xv, s);
    }
  }
  if constexpr (AMAX) {
    // abs_max = max(abs_max, max|x|): one atomic max per CTA on the bit patterns, compared as signed
    // integers - non-negative floats order like their bits with NaN on top (a NaN stays), and a negative
    // starting value (callers start from -1.0) loses to any magnitude.  No ticket, no last-CTA pass: the
    // kernel has no tail behind its last store.
    m = block_max_u32(m, smem32);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(abs_max_inout), (int)m);
  }
}

}  // namespace tnq

// ================================================================= host side
using namespace tnq;

namespace tnq_host {
thread_local int g_last_cuda_error = 0;

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace tnq_host
using namespace tnq_host;

// Persistent grid: as many CTAs as are resident at once (occupancy * SMs), fewer
// for small inputs.
template <auto Kernel>
static int resident_ctas() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kernel, kThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

template <auto Kernel>
static int stream_grid(int64_t n_vec) {
  int64_t want = (n_vec + kThreads - 1) / kThreads;
  int64_t cap = resident_ctas<Kernel>();
  if (cap > kMaxPartials) cap = kMaxPartials;
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

// tuning switches: read by any thread that launches, written by tnq_set_option (relaxed atomics:
// a launch sees either the old or the new value, never a torn one)
static std::atomic<int> g_cast_reverse{1};
static std::atomic<int> g_fused_small{1};
static std::atomic<int> g_l2_keep_mb{64};
static std::atomic<int> g_cast_l2_mode{0};
static std::atomic<int> g_cast_pair{1};
static std::atomic<int> g_tile_evict_first{0};  // measured: NVFP4 205.6 -> 209.5 us with it, MXFP8 one direction 31.3 -> 31.1
static std::atomic<int> g_fused_launch{1};
static std::atomic<int> g_pdl_chain{1};
static std::atomic<int> g_exchange_cast_waits{0};
namespace tnq_host {
bool pdl_chain() { return g_pdl_chain.load(std::memory_order_relaxed) != 0; }
int fused_launch_mode() { return g_fused_launch.load(std::memory_order_relaxed); }
bool tile_loads_evict_first() { return g_tile_evict_first.load(std::memory_order_relaxed) != 0; }
}  // namespace tnq_host
// Walking backwards only pays once the tensor no longer fits in L2 as a whole, and only while the tail that L2 keeps
// (64 MiB) is a noticeable part of it.  Measured on two tensors cast in turn, keep-and-walk-back against the plain
// forward walk: 256 MiB 112.0 -> 106.2 us, 512 MiB 216.7 -> 208.4, 1 GiB 421.1 -> 415.5, 1.5 GiB 625.6 -> 624.1,
// 2 GiB 821-836 -> 827-843 (the eviction priorities then cost more than the 3 % of the reads they save).
constexpr int64_t kReverseMinBytes = 96ll << 20;
constexpr int64_t kReverseMaxBytes = 1536ll << 20;
static bool reverse_pays(int64_t bytes) { return bytes > kReverseMinBytes && bytes <= kReverseMaxBytes; }

// First vector of the tail that the amax pass asks L2 to keep for the cast pass.
static int64_t keep_from_vec(int64_t n, int in_dtype) {
  const int64_t bytes = n * (in_dtype == TNQ_IN_BF16 ? 2 : 4), nvec = bytes / 32;
  const int keep_mb = g_l2_keep_mb.load(std::memory_order_relaxed);
  if (!g_cast_reverse.load(std::memory_order_relaxed) || keep_mb <= 0 || !reverse_pays(bytes)) return nvec;
  const int64_t keep_vec = ((int64_t)keep_mb << 20) / 32;
  return keep_vec >= nvec ? 0 : nvec - keep_vec;
}

extern "C" int tnq_set_option(int option, int value) {
  switch (option) {
    case TNQ_OPT_CAST_REVERSE: g_cast_reverse.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_FUSED_SMALL: g_fused_small.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_L2_KEEP_MB: g_l2_keep_mb.store(value < 0 ? 0 : value, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_CAST_L2_MODE: g_cast_l2_mode.store(value & 3, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_CAST_PAIR: g_cast_pair.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_TILE_EVICT_FIRST: g_tile_evict_first.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_EXCHANGE_CAST_WAITS: g_exchange_cast_waits.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_PDL_CHAIN: g_pdl_chain.store(value ? 1 : 0, std::memory_order_relaxed); return TNQ_OK;
    case TNQ_OPT_FUSED_LAUNCH:
      if (value != 0 && value != 1) return TNQ_EINVAL;
      g_fused_launch.store(value, std::memory_order_relaxed);
      return TNQ_OK;
    default: return TNQ_EINVAL;
  }
}

static int check_common(const void* x, int64_t n, int in_dtype, int out_dtype) {
  if (n < 0 || (n > 0 && x == nullptr)) return TNQ_EINVAL;
  if (in_dtype != TNQ_IN_BF16 && in_dtype != TNQ_IN_F32) return TNQ_EUNSUPPORTED;
  if (out_dtype != TNQ_FP8_E4M3 && out_dtype != TNQ_FP8_E5M2) return TNQ_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 31u) != 0) return TNQ_EALIGN;  // 256-bit loads
  return TNQ_OK;
}

static float fp8_max_of(int out_dtype) { return out_dtype == TNQ_FP8_E4M3 ? 448.0f : 57344.0f; }

template <auto Kernel, typename... Args>
static int launch(int64_t n_vec, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(stream_grid<Kernel>(n_vec));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl || pdl_chain()) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, Kernel, args...);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

static int amax_launch(const uint8_t* xp, int64_t n, int in_dtype, Workspace* ws, float* amax_out, float* scale_out,
                       float fmax, cudaStream_t stream, bool cast_follows = false) {
  const PeerSlots none = {};
  const int64_t keep = cast_follows ? keep_from_vec(n, in_dtype) : INT64_MAX;
  if (in_dtype == TNQ_IN_BF16)
    return launch<k_amax<TNQ_IN_BF16, false>>(n / 16, stream, false, xp, n, ws, amax_out, scale_out, fmax, none, keep);
  return launch<k_amax<TNQ_IN_F32, false>>(n / 8, stream, false, xp, n, ws, amax_out, scale_out, fmax, none, keep);
}

namespace tnq_host {
int amax_pass(const void* x, int64_t n, int in_dtype, void* workspace, float* scale_out, float fp8_max, cudaStream_t stream,
              bool tail_stays) {
  return amax_launch(static_cast<const uint8_t*>(x), n, in_dtype, static_cast<Workspace*>(workspace), nullptr, scale_out,
                     fp8_max, stream, tail_stays);
}
}  // namespace tnq_host

extern "C" int tnq_fp8_amax(const void* x, int64_t n, int in_dtype, int out_dtype, void* workspace,
                            float* amax_out, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, out_dtype);
  if (rc != TNQ_OK) return rc;
  if (workspace == nullptr) return TNQ_EINVAL;
  Workspace* ws = static_cast<Workspace*>(workspace);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  const float fmax = fp8_max_of(out_dtype);
  return amax_launch(xp, n, in_dtype, ws, amax_out, nullptr, fmax, stream);
}

template <int IN, int OUT, bool PAIR>
static int cast_dispatch_pair(const uint8_t* x, uint8_t* out, int64_t n, const float* scale, int scale_source,
                              int saturated, float* abs_max, Workspace* ws, cudaStream_t stream, bool pdl,
                              const ExchangeWait& ex, int reverse, int l2_mode) {
  const int64_t nv = n / InTraits<IN>::kElemsPerVec / (PAIR ? GroupTraits<IN>::kVecs : 1);  // units per launch -> grid size
  if (abs_max) {
    if (saturated) return launch<k_cast<IN, OUT, true, true, PAIR>>(nv, stream, pdl, x, out, n, scale, scale_source, abs_max, ws, ex, reverse, l2_mode);
    return launch<k_cast<IN, OUT, false, true, PAIR>>(nv, stream, pdl, x, out, n, scale, scale_source, abs_max, ws, ex, reverse, l2_mode);
  }
  if (saturated) return launch<k_cast<IN, OUT, true, false, PAIR>>(nv, stream, pdl, x, out, n, scale, scale_source, abs_max, ws, ex, reverse, l2_mode);
  return launch<k_cast<IN, OUT, false, false, PAIR>>(nv, stream, pdl, x, out, n, scale, scale_source, abs_max, ws, ex, reverse, l2_mode);
}

template <int IN, int OUT>
static int cast_dispatch(const uint8_t* x, uint8_t* out, int64_t n, const float* scale, int scale_source,
                         int saturated, float* abs_max, Workspace* ws, cudaStream_t stream, bool pdl,
                         const ExchangeWait& ex, int reverse, int l2_mode) {
  // forward walks over bf16 input take adjacent vectors per thread (tuning switch, on by default); the reversed
  // walk does not, and fp32 input measured slower that way (four adjacent vectors per thread: 101 -> 123 us)
  const bool pair = IN == TNQ_IN_BF16 && !reverse && g_cast_pair.load(std::memory_order_relaxed) != 0;
  if (pair) return cast_dispatch_pair<IN, OUT, true>(x, out, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
  return cast_dispatch_pair<IN, OUT, false>(x, out, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
}

static int cast_any(const void* x, void* out, int64_t n, int in_dtype, int out_dtype, const float* scale,
                    int scale_source, int saturated, float* abs_max, void* workspace, cudaStream_t stream,
                    bool pdl, const ExchangeWait& ex = ExchangeWait{}) {
  // a cast that follows an amax pass over the same tensor may walk it backwards
  const int64_t in_bytes = n * (in_dtype == TNQ_IN_BF16 ? 2 : 4);
  const bool after_amax = pdl || scale_source == TNQ_SCALE_IS_AMAX;
  const int reverse = (after_amax && g_cast_reverse.load(std::memory_order_relaxed) && reverse_pays(in_bytes)) ? 1 : 0;
  // bit 2: the scale is this very tensor's fp8_max / amax (dynamic and sharded casts), see k_cast
  const int l2_mode = (reverse ? g_cast_l2_mode.load(std::memory_order_relaxed) : 0) | ((pdl || ex.slots != nullptr) ? 4 : 0) |
                      (g_exchange_cast_waits.load(std::memory_order_relaxed) ? 8 : 0);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  uint8_t* op = static_cast<uint8_t*>(out);
  Workspace* ws = static_cast<Workspace*>(workspace);
  if (in_dtype == TNQ_IN_BF16) {
    if (out_dtype == TNQ_FP8_E4M3)
      return cast_dispatch<TNQ_IN_BF16, TNQ_FP8_E4M3>(xp, op, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
    return cast_dispatch<TNQ_IN_BF16, TNQ_FP8_E5M2>(xp, op, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
  }
  if (out_dtype == TNQ_FP8_E4M3)
    return cast_dispatch<TNQ_IN_F32, TNQ_FP8_E4M3>(xp, op, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
  return cast_dispatch<TNQ_IN_F32, TNQ_FP8_E5M2>(xp, op, n, scale, scale_source, saturated, abs_max, ws, stream, pdl, ex, reverse, l2_mode);
}

extern "C" int tnq_fp8_scaled_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                                   const float* scale, int scale_source, int saturated,
                                   float* abs_max_inout, void* workspace, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, out_dtype);
  if (rc != TNQ_OK) return rc;
  if (scale == nullptr || (n > 0 && out == nullptr)) return TNQ_EINVAL;
  if (scale_source != TNQ_SCALE_IS_SCALE && scale_source != TNQ_SCALE_IS_AMAX) return TNQ_EINVAL;
  if (abs_max_inout != nullptr && workspace == nullptr) return TNQ_EINVAL;
  if (!aligned16(out)) return TNQ_EALIGN;
  return cast_any(x, out, n, in_dtype, out_dtype, scale, scale_source, saturated, abs_max_inout, workspace,
                  stream, false);
}

extern "C" int tnq_fp8_dynamic_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                                    void* workspace, float* scale_out, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, out_dtype);
  if (rc != TNQ_OK) return rc;
  if (workspace == nullptr || (n > 0 && out == nullptr)) return TNQ_EINVAL;
  if (!aligned16(out)) return TNQ_EALIGN;
  if (g_fused_small.load(std::memory_order_relaxed)) {  // the whole tensor fits in shared memory: one launch, one HBM read
    int grid = 0;
    uint32_t slab = 0;
    if (fused_plan(n * (in_dtype == TNQ_IN_BF16 ? 2 : 4), &grid, &slab))
      return fused_dynamic_cast(x, out, n, in_dtype, out_dtype, workspace, scale_out, stream, grid, slab);
  }
  Workspace* ws = static_cast<Workspace*>(workspace);
  rc = amax_launch(static_cast<const uint8_t*>(x), n, in_dtype, ws, nullptr, scale_out, fp8_max_of(out_dtype), stream, true);
  if (rc != TNQ_OK) return rc;
  return cast_any(x, out, n, in_dtype, out_dtype, &ws->scale, TNQ_SCALE_IS_SCALE, 1, nullptr, workspace, stream,
                  true);
}

extern "C" int tnq_fp8_sharded_cast(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                                    void* workspace, void* const* slot_buffers, int world_size, int rank,
                                    uint32_t seq, float* amax_out, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, out_dtype);
  if (rc != TNQ_OK) return rc;
  if (workspace == nullptr || slot_buffers == nullptr || (n > 0 && out == nullptr)) return TNQ_EINVAL;
  if (world_size < 1 || world_size > kMaxRanks || rank < 0 || rank >= world_size || seq == 0) return TNQ_EINVAL;
  if (!aligned16(out)) return TNQ_EALIGN;
  PeerSlots peers = {};
  for (int r = 0; r < world_size; ++r) {
    if (slot_buffers[r] == nullptr) return TNQ_EINVAL;
    peers.base[r] = static_cast<uint64_t*>(slot_buffers[r]);
  }
  peers.world = world_size, peers.rank = rank, peers.seq = seq;
  Workspace* ws = static_cast<Workspace*>(workspace);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  const float fmax = fp8_max_of(out_dtype);
  if (in_dtype == TNQ_IN_BF16)
    rc = launch<k_amax<TNQ_IN_BF16, true>>(n / 16, stream, false, xp, n, ws, (float*)nullptr, (float*)nullptr, fmax, peers,
                                           keep_from_vec(n, in_dtype));
  else
    rc = launch<k_amax<TNQ_IN_F32, true>>(n / 8, stream, false, xp, n, ws, (float*)nullptr, (float*)nullptr, fmax, peers,
                                          keep_from_vec(n, in_dtype));
  if (rc != TNQ_OK) return rc;
  ExchangeWait ex;
  ex.slots = peers.base[rank];
  ex.world = world_size;
  ex.seq = seq;
  ex.status = reinterpret_cast<uint32_t*>(peers.base[rank]) + kExchangeStatusWord;
  ex.amax_out = amax_out;
  return cast_any(x, out, n, in_dtype, out_dtype, &ws->scale, TNQ_SCALE_IS_SCALE, 1, nullptr, workspace, stream,
                  true, ex);
}

// ================================================================= no-allocation variant
// Dynamic per-tensor cast for callers that own no device scratch and may not create
// any: a plug-in that is handed input and output buffers and a stream by a host
// framework but no allocator, a serving process that gave all device memory to its
// own pool at start-up (a later cudaMalloc fails or stalls every stream while it
// runs), or a latency-critical loop that cannot afford cudaMalloc's implicit
// device-wide synchronisation.  The reduction scratch that tnq_fp8_dynamic_cast takes
// from the caller lives here in a fixed array inside the library image: every GPU
// that loads libtnq.so carries these 4 KiB until the process exits.
namespace tnq {
constexpr int kStaticScratchBytes = 4096;
constexpr int kStaticMaxCtas = (kStaticScratchBytes - 64) / 4;  // per-CTA partial maxima that fit: 1008
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
}  // namespace tnq

// Device address of g_static_scratch on the current device.  In host code the name of
// a __device__ array is only a handle for the runtime, not an address a kernel can
// use, so the address is asked for once per device (with that device current).
static int static_scratch_address(void** out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return TNQ_EUNSUPPORTED;
  void* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress((void**)&p, tnq::g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e);
    if (p == nullptr) return TNQ_ECUDA;
    __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);  // every thread would store the same value
  }
  *out = p;
  return TNQ_OK;
}

extern "C" int64_t tnq_fp8_dynamic_cast_static_max_elements(void) { return TNQ_STATIC_MAX_ELEMENTS; }

extern "C" int tnq_fp8_dynamic_cast_static(const void* x, void* out, int64_t n, int in_dtype, int out_dtype,
                                           float* scale_out, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, out_dtype);
  if (rc != TNQ_OK) return rc;
  if (n > 0 && out == nullptr) return TNQ_EINVAL;
  if (!aligned16(out)) return TNQ_EALIGN;
  if (n > TNQ_STATIC_MAX_ELEMENTS) return TNQ_EUNSUPPORTED;  // beyond what the fixed scratch is specified for
  // one partial-maximum slot per CTA of the amax launch must fit in the fixed array
  const int amax_ctas = in_dtype == TNQ_IN_BF16 ? resident_ctas<k_amax<TNQ_IN_BF16, false>>()
                                                : resident_ctas<k_amax<TNQ_IN_F32, false>>();
  if (amax_ctas > kStaticMaxCtas) return TNQ_EUNSUPPORTED;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != TNQ_OK) return rc;
  // The array keeps whatever the previous call left.  The ticket counter and the
  // status word must start at zero (a call that was abandoned half way would
  // otherwise poison the next one); the partial slots are overwritten before use.
  cudaError_t e = cudaMemsetAsync(scratch, 0, 64, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  Workspace* ws = static_cast<Workspace*>(scratch);
  rc = amax_launch(static_cast<const uint8_t*>(x), n, in_dtype, ws, nullptr, scale_out, fp8_max_of(out_dtype), stream, true);
  if (rc != TNQ_OK) return rc;
  return cast_any(x, out, n, in_dtype, out_dtype, &ws->scale, TNQ_SCALE_IS_SCALE, 1, nullptr, scratch, stream, true);
}

extern "C" int tnq_sharded_amax(const void* x, int64_t n, int in_dtype, void* workspace, void* const* slot_buffers,
                                int world_size, int rank, uint32_t seq, float* amax_out, tnq_stream_t stream) {
  int rc = check_common(x, n, in_dtype, TNQ_FP8_E4M3);
  if (rc != TNQ_OK) return rc;
  if (workspace == nullptr || slot_buffers == nullptr || amax_out == nullptr) return TNQ_EINVAL;
  if (world_size < 1 || world_size > kMaxRanks || rank < 0 || rank >= world_size || seq == 0) return TNQ_EINVAL;
  PeerSlots peers = {};
  for (int r = 0; r < world_size; ++r) {
    if (slot_buffers[r] == nullptr) return TNQ_EINVAL;
    peers.base[r] = static_cast<uint64_t*>(slot_buffers[r]);
  }
  peers.world = world_size, peers.rank = rank, peers.seq = seq;
  Workspace* ws = static_cast<Workspace*>(workspace);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  if (in_dtype == TNQ_IN_BF16)
    rc = launch<k_amax<TNQ_IN_BF16, true>>(n / 16, stream, false, xp, n, ws, (float*)nullptr, (float*)nullptr, 448.0f, peers,
                                           (int64_t)INT64_MAX);
  else
    rc = launch<k_amax<TNQ_IN_F32, true>>(n / 8, stream, false, xp, n, ws, (float*)nullptr, (float*)nullptr, 448.0f, peers,
                                          (int64_t)INT64_MAX);
  if (rc != TNQ_OK) return rc;
  ExchangeWait ex;
  ex.slots = peers.base[rank];
  ex.world = world_size;
  ex.seq = seq;
  ex.status = reinterpret_cast<uint32_t*>(peers.base[rank]) + kExchangeStatusWord;
  ex.amax_out = amax_out;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k_exchange_collect, ex);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

extern "C" const char* tnq_status_str(int status) {
  switch (status) {
    case TNQ_OK: return "ok";
    case TNQ_EINVAL: return "invalid argument";
    case TNQ_EALIGN: return "pointer or pitch not sufficiently aligned";
    case TNQ_ESHAPE: return "shape is not a multiple of the block size";
    case TNQ_EUNSUPPORTED: return "unsupported dtype or size";
    case TNQ_ECUDA: return "CUDA runtime error";
    case TNQ_ETIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}
extern "C" int tnq_last_cuda_error(void) { return tnq_host::g_last_cuda_error; }
extern "C" int tnq_abi_version(void) { return 1; }
