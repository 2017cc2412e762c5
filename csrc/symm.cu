// Peer-visible device buffers for the fused compute+collective kernels.
//
// One process drives one GPU.  A buffer allocated here with cudaMalloc is exported as a CUDA
// IPC handle, the handles are exchanged through the host-side process group, and every rank
// maps every peer's buffer into its own address space.  Kernels then read and write peer
// memory with ordinary loads and stores over NVLink (no bulk-tensor copy ever reads a peer's
// memory, and no library kernel is ever handed a peer pointer).
#include "common.cuh"

#include <string.h>

extern "C" {

// Allocates `bytes` of zeroed device memory on the current device.  Returns null on failure.
void* js_symm_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    return nullptr;
  }
  return p;
}

int js_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }

// Writes the 64-byte IPC handle of an allocation made by js_symm_alloc.
int js_symm_export(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

// Maps a peer's allocation from its IPC handle; returns the local address or null.
void* js_symm_import(const unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}

int js_symm_unmap(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

int js_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

}  // extern "C"
