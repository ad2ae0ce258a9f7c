// Scale-matrix swizzle: row-major [H, W] one-byte scales -> the 128x4 layout that
// block-scaled tensor-core MMA reads (512-byte atoms: 32 rows x (4 row groups x 4
// columns)), zero padded to whole atoms.
//
// One CTA converts 128 rows x 32 columns (eight atoms, 4 KiB): byte loads with
// bounds checks gather the block into shared memory at the swizzled offsets, and
// the eight atoms, which are contiguous in the output, leave as 16-byte stores.
// The quantizer kernels write this layout directly; this kernel serves callers
// that hold raw scales.
#include "common.cuh"

namespace tnq {

__global__ void __launch_bounds__(256)
    k_to_blocked(const uint8_t* __restrict__ in, int64_t rows, int64_t cols, uint8_t* __restrict__ out, int64_t ncb) {
  __shared__ __align__(16) uint8_t s[4096];
  const int64_t rb = blockIdx.y;
  const int64_t cb0 = (int64_t)blockIdx.x * 8;
  pdl_wait();  // chained launch: nothing of the stream's previous kernel is read or overwritten before this
  pdl_launch_dependents();
  for (int idx = threadIdx.x; idx < 4096; idx += 256) {
    const int r = idx >> 5, c = idx & 31;
    const int64_t gr = rb * 128 + r, gc = cb0 * 4 + c;
    const uint8_t v = (gr < rows && gc < cols) ? in[gr * cols + gc] : (uint8_t)0;
    s[(c >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (c & 3)] = v;
  }
  __syncthreads();
  const int atom = threadIdx.x >> 5;
  if (cb0 + atom < ncb)
    stg128(out + (rb * ncb + cb0) * 512 + threadIdx.x * 16, *reinterpret_cast<const uint4*>(s + threadIdx.x * 16));
}

}  // namespace tnq

extern "C" int tnq_to_blocked(const void* in, int64_t rows, int64_t cols, void* out, tnq_stream_t stream) {
  if (rows < 0 || cols < 0) return TNQ_EINVAL;
  if (rows == 0 || cols == 0) return TNQ_OK;
  if (in == nullptr || out == nullptr) return TNQ_EINVAL;
  if (!tnq_host::aligned16(out)) return TNQ_EALIGN;
  const int64_t nrb = (rows + 127) / 128, ncb = (cols + 3) / 4;
  if (nrb > 65535) return TNQ_EUNSUPPORTED;
  dim3 grid((unsigned)((ncb + 7) / 8), (unsigned)nrb);
  return tnq_host::launch_chained(tnq::k_to_blocked, grid, dim3(256), 0, stream, static_cast<const uint8_t*>(in), rows, cols,
                                  static_cast<uint8_t*>(out), ncb);
}
