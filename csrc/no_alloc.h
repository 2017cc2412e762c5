// Entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference implementation; it exists for hosts of
// this library that must not call cudaMalloc (or any allocating routine) on the decode path:
// code that runs while a CUDA graph is being captured on another stream of the same process,
// real-time serving loops with a frozen memory budget, and embedders (C, Rust, Go FFI) that
// hand us raw pointers and own every byte themselves.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch area covers.
#define JS_STATIC_ARGMAX_MAX_ROWS 128
#define JS_STATIC_ARGMAX_MAX_VOCAB 163840

// Greedy token per row of  h (M, K) x w (N, K)^T  (bf16 in, fp32 accumulate): out_idx[m] = argmax_n,
// out_val[m] = the winning logit (out_val may be null).  Same kernels and same results as the
// allocating entry points (js_gemm_bf16 with the argmax epilogue + js_argmax_merge); the per-tile
// partial maxima they exchange live in a file-scope __device__ array of about 1.3 MB that every
// GPU which loads this library holds until the process exits.
//
// Allocates nothing: no cudaMalloc / cudaFree / allocating library call.  The first call on each
// device looks up the array's device address (cudaGetSymbolAddress); make that first call before
// any stream capture begins.  Every call shares the one scratch array and the array keeps the
// previous call's contents, so two calls that overlap on the GPU (different streams) race: issue
// them on one stream or order them with events.
//
// Returns 0, -30 if M or N exceed the limits above, -31 if the scratch address lookup failed,
// or the negative code of the underlying launch.
int js_lm_head_argmax_static(const void* h, const void* w, int M, int N, int K, int lda, int ldw, int* out_idx,
                             float* out_val, cudaStream_t stream);

// The kernels behind js_lm_head_argmax_static never spin forever: a wait that runs out records a code in a
// status word inside the same scratch array and the call still returns 0 (the launch succeeded), with
// undefined tokens.  This accessor copies that word to *host_status (0 = the last call on this device ran
// clean; 1..3 = a bounded wait inside the GEMM gave up) and synchronises `stream`, so call it on the stream
// the argmax ran on, after it.  Allocates nothing.  Returns 0, -31 (address lookup failed), -32 (copy or
// synchronisation failed) or -33 (null pointer).
int js_lm_head_argmax_static_status(int* host_status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
