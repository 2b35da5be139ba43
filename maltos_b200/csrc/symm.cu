// Symmetric memory for one node: device buffers that every rank of a process group maps into its own address
// space through CUDA IPC, plus a small signal pad per rank. The fused compute+collective kernels read and write peer
// memory with plain loads/stores over NVLink through these mappings (no TMA multicast anywhere).
//
// Allocation is done once per (group, size) at set-up time; nothing here runs inside a training step.
#include <cstring>

#include "host.h"

MB_API int mb_symm_alloc(size_t bytes, void** ptr_out, unsigned char* handle_out64) {
  mb::bind_context();
  void* p = nullptr;
  MB_CHECK_CUDA(cudaMalloc(&p, bytes));
  MB_CHECK_CUDA(cudaMemset(p, 0, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    mb::set_last_error(cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  std::memcpy(handle_out64, &h, 64);
  *ptr_out = p;
  MB_CHECK_CUDA(cudaDeviceSynchronize());
  return 0;
}

MB_API int mb_symm_open(const unsigned char* handle64, void** ptr_out) {
  mb::bind_context();
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  MB_CHECK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = p;
  return 0;
}

MB_API int mb_symm_close(void* ptr) {
  MB_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

MB_API int mb_symm_free(void* ptr) {
  MB_CHECK_CUDA(cudaFree(ptr));
  return 0;
}

// 1 when `dev` can map memory of `peer` (NVLink / PCIe peer access).
MB_API int mb_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}
