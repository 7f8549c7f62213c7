// Symmetric-heap runtime: one device allocation per rank that every peer of
// the NVSwitch domain maps into its own address space, so kernels can load
// from and store to any rank's buffers directly.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>

namespace grace {

constexpr size_t kIpcHandleBytes = 64;

cudaError_t symm_alloc(void** ptr, size_t bytes);          // zero-initialised
cudaError_t symm_free(void* ptr);
cudaError_t symm_export(void* ptr, char* handle_out);       // kIpcHandleBytes
cudaError_t symm_import(const char* handle, void** ptr);    // map a peer's heap
cudaError_t symm_release(void* ptr);                        // unmap a peer's heap
cudaError_t symm_enable_peer(int peer_device);

}  // namespace grace
