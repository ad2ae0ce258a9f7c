// Delayed-scaling state update: the step between two delayed-scale casts.
//
// `tnq_fp8_scaled_cast` casts with a scale fixed before the step and leaves max|x| of the
// step in an fp32 word.  Between steps every tensor's amax word is pushed into its amax
// history and the next scale is taken from the history:
//
//     history[t] = [amax[t], history[t][0 .. L-2]]            (newest first, oldest dropped)
//     scale[t]   = fp8_max / max(max_l history[t][l], 1e-12)   (one IEEE fp32 division)
//     amax[t]    = 0                                           (the next step's max starts clean)
//
// One warp per tensor, all tensors of a model in one launch.  The maximum is taken on the
// integer view of the non-negative floats, so a NaN in the history wins and makes the scale
// NaN, as torch.max does.
#include "common.cuh"

namespace tnq {

constexpr int kDelayedMaxHistory = 1024;  // 32 values per lane

template <int OUT>
__global__ void __launch_bounds__(128)
    k_delayed_scale_update(float* __restrict__ history, float* __restrict__ amax, float* __restrict__ scale,
                           int tensors, int len) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tensors) return;
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  uint32_t* h = reinterpret_cast<uint32_t*>(history) + (int64_t)t * len;
  const uint32_t newest = __float_as_uint(amax[t]) & 0x7fffffffu;
  uint32_t keep[kDelayedMaxHistory / 32];
  uint32_t m = newest;
#pragma unroll
  for (int j = 0; j < kDelayedMaxHistory / 32; ++j) {
    const int l = j * 32 + lane;  // old position; moves to l + 1 unless it is the oldest
    keep[j] = (l < len - 1) ? (h[l] & 0x7fffffffu) : 0u;
    m = max(m, keep[j]);
  }
  m = warp_max_u32(m);
  __syncwarp();  // every old value is in registers before any slot is overwritten
#pragma unroll
  for (int j = 0; j < kDelayedMaxHistory / 32; ++j) {
    const int l = j * 32 + lane;
    if (l < len - 1) h[l + 1] = keep[j];
  }
  if (lane == 0) {
    h[0] = newest;
    scale[t] = scale_from_amax(__uint_as_float(m), Fp8Traits<OUT>::kMax);
    amax[t] = 0.0f;
  }
}

}  // namespace tnq

extern "C" int tnq_delayed_scale_update(float* amax_history, float* amax, float* scale, int64_t tensors,
                                        int history_len, int out_dtype, tnq_stream_t stream) {
  if (tensors < 0 || history_len < 1) return TNQ_EINVAL;
  if (out_dtype != TNQ_FP8_E4M3 && out_dtype != TNQ_FP8_E5M2) return TNQ_EINVAL;
  if (tensors == 0) return TNQ_OK;
  if (!amax_history || !amax || !scale) return TNQ_EINVAL;
  if (history_len > tnq::kDelayedMaxHistory || tensors > (1 << 30)) return TNQ_EUNSUPPORTED;
  const int warps = 4;
  const unsigned grid = (unsigned)((tensors + warps - 1) / warps);
  if (out_dtype == TNQ_FP8_E4M3)
    return tnq_host::launch_chained(tnq::k_delayed_scale_update<TNQ_FP8_E4M3>, dim3(grid), dim3(warps * 32), 0, stream, amax_history,
                                    amax, scale, (int)tensors, history_len);
  return tnq_host::launch_chained(tnq::k_delayed_scale_update<TNQ_FP8_E5M2>, dim3(grid), dim3(warps * 32), 0, stream, amax_history,
                                  amax, scale, (int)tensors, history_len);
}
