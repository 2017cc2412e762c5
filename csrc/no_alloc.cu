// Allocation-free LM-head argmax: see no_alloc.h for who needs it and for the contract.
#include "no_alloc.h"

#include <stdint.h>

extern "C" int js_gemm_bf16(const void* A, const void* W, void* C, const void* residual, int M, int N, int K, int lda,
                            int ldw, int ldc, int epi, int bn, int split, int deep, float* part_val, int* part_idx,
                            float* part_lse, int* status, unsigned long long* trace, int pdl, cudaStream_t stream);
extern "C" int js_argmax_merge(const float* part_val, const int* part_idx, int n_tiles, int M, int* out_idx,
                               float* out_val, int pdl, cudaStream_t stream);

namespace {

constexpr int kMaxTiles = JS_STATIC_ARGMAX_MAX_VOCAB / 128;
constexpr size_t kValBytes = sizeof(float) * JS_STATIC_ARGMAX_MAX_ROWS * kMaxTiles;
constexpr size_t kIdxBytes = sizeof(int) * JS_STATIC_ARGMAX_MAX_ROWS * kMaxTiles;
constexpr size_t kStatusOffset = kValBytes + kIdxBytes;
constexpr size_t kScratchBytes = kStatusOffset + 256;

// [per-tile maxima fp32][per-tile argmax int32][status word].  In host code this NAME is only a
// stand-in for the symbol; the device address is obtained below with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};

// Once per device, with that device current.  Host threads may race to fill a slot: the lookup is
// idempotent (every thread gets the same address), and the slot is published with release/acquire
// atomics so no thread ever reads a half-written pointer.
unsigned char* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  void* p = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || p == nullptr) return nullptr;
    __atomic_store_n(&g_scratch_addr[dev], p, __ATOMIC_RELEASE);
  }
  return static_cast<unsigned char*>(p);
}

}  // namespace

extern "C" int js_lm_head_argmax_static(const void* h, const void* w, int M, int N, int K, int lda, int ldw,
                                        int* out_idx, float* out_val, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > JS_STATIC_ARGMAX_MAX_ROWS || N > JS_STATIC_ARGMAX_MAX_VOCAB) return -30;
  unsigned char* s = scratch_for_current_device();
  if (s == nullptr) return -31;
  float* part_val = reinterpret_cast<float*>(s);
  int* part_idx = reinterpret_cast<int*>(s + kValBytes);
  int* status = reinterpret_cast<int*>(s + kStatusOffset);
  // the status word must start at zero; the partials are fully overwritten by the GEMM epilogue
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return -32;
  const int n_tiles = (N + 127) / 128;
  int rc = js_gemm_bf16(h, w, nullptr, nullptr, M, N, K, lda, ldw, 0, /*epi argmax*/ 2, 128, 1, 0, part_val, part_idx,
                        nullptr, status, nullptr, 0, stream);
  if (rc != 0) return rc;
  return js_argmax_merge(part_val, part_idx, n_tiles, M, out_idx, out_val, 0, stream);
}

extern "C" int js_lm_head_argmax_static_status(int* host_status, cudaStream_t stream) {
  if (host_status == nullptr) return -33;
  unsigned char* s = scratch_for_current_device();
  if (s == nullptr) return -31;
  if (cudaMemcpyAsync(host_status, s + kStatusOffset, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -32;
  return cudaStreamSynchronize(stream) == cudaSuccess ? 0 : -32;
}
