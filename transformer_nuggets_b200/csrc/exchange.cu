// Set-up side of the cross-GPU amax exchange: each rank allocates one small slot
// buffer with cudaMalloc, exports it as a CUDA IPC handle, and maps every peer's
// buffer (peer access over NVLink).  These are the only functions of the library
// that allocate or synchronise; they run once per process group, outside any timed
// or captured region.  The kernels that use the buffers are in fp8_tensor.cu.
#include <cstring>

#include "common.cuh"

using namespace tnq_host;

constexpr size_t kExchangeBytes = 4096;

extern "C" int tnq_exchange_create(void** local_slots, unsigned char ipc_handle[64]) {
  if (local_slots == nullptr || ipc_handle == nullptr) return TNQ_EINVAL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, kExchangeBytes);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemset(p, 0, kExchangeBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e);
  }
  std::memcpy(ipc_handle, &h, 64);
  *local_slots = p;
  return TNQ_OK;
}

extern "C" int tnq_exchange_open(const unsigned char ipc_handle[64], void** peer_slots) {
  if (ipc_handle == nullptr || peer_slots == nullptr) return TNQ_EINVAL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, ipc_handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e);
  *peer_slots = p;
  return TNQ_OK;
}

extern "C" int tnq_exchange_close(void* peer_slots) {
  if (peer_slots == nullptr) return TNQ_OK;
  cudaError_t e = cudaIpcCloseMemHandle(peer_slots);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

extern "C" int tnq_exchange_destroy(void* local_slots) {
  if (local_slots == nullptr) return TNQ_OK;
  cudaError_t e = cudaFree(local_slots);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}

// Synchronising read of the status word of this rank's slot buffer (0 = no bounded
// wait has expired since creation); *host_status is host memory.
extern "C" int tnq_exchange_status(const void* local_slots, uint32_t* host_status) {
  if (local_slots == nullptr || host_status == nullptr) return TNQ_EINVAL;
  cudaError_t e = cudaMemcpy(host_status, static_cast<const uint8_t*>(local_slots) + 2048, sizeof(uint32_t),
                             cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? TNQ_OK : cuda_fail(e);
}
