// Raw device allocations and CUDA IPC handles. Transport and Fabric arenas are
// plain cudaMalloc regions whose 64-byte IPC handle travels as hex through the
// control plane (the reference does the same for Transport arenas,
// src/cext/transport/arena.cpp:40, and uses the NVSHMEM heap for the Fabric);
// every peer opens the handle once and keeps the mapped pointer.
#include <cuda_runtime.h>
#include <string.h>

#include "xpool/api.h"

extern "C" int xp_dev_alloc(void** ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return -static_cast<int>(e);
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? 0 : -1;
}
extern "C" int xp_dev_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

extern "C" int xp_ipc_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return -static_cast<int>(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
extern "C" int xp_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
extern "C" int xp_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }

extern "C" int xp_memset_async(void* ptr, int value, size_t bytes, void* stream) {
  return cudaMemsetAsync(ptr, value, bytes, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -1;
}

// For pointers of another device of the SAME process (tests, single-process deployments).
extern "C" int xp_enable_peer_access(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
