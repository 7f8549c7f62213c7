// Symmetric heap over CUDA IPC.
//
// Every rank allocates one region with cudaMalloc, exports it as a
// cudaIpcMemHandle_t (64 opaque bytes that travel through the process group's
// store) and maps every peer's region with cudaIpcOpenMemHandle.  On an
// NVSwitch machine the mapping is served by NVLink peer access; the kernels in
// this directory then address `heap[r] + offset` for any rank r.
// The reference has no counterpart: its ranks only ever meet inside NCCL,
// Gloo or Horovod library calls.
#include "runtime.h"

#include <cstring>

namespace grace {

static_assert(sizeof(cudaIpcMemHandle_t) == kIpcHandleBytes, "unexpected IPC handle size");

cudaError_t symm_alloc(void** ptr, size_t bytes) {
  cudaError_t err = cudaMalloc(ptr, bytes);
  if (err != cudaSuccess) return err;
  err = cudaMemset(*ptr, 0, bytes);
  if (err != cudaSuccess) return err;
  return cudaDeviceSynchronize();
}

cudaError_t symm_free(void* ptr) { return cudaFree(ptr); }

cudaError_t symm_export(void* ptr, char* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t err = cudaIpcGetMemHandle(&h, ptr);
  if (err != cudaSuccess) return err;
  std::memcpy(handle_out, &h, kIpcHandleBytes);
  return cudaSuccess;
}

cudaError_t symm_import(const char* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, kIpcHandleBytes);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

cudaError_t symm_release(void* ptr) { return cudaIpcCloseMemHandle(ptr); }

cudaError_t symm_enable_peer(int peer_device) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (peer_device == dev) return cudaSuccess;
  int can = 0;
  err = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (err != cudaSuccess) return err;
  if (!can) return cudaErrorPeerAccessUnsupported;
  err = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (err == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return cudaSuccess;
  }
  return err;
}

}  // namespace grace
