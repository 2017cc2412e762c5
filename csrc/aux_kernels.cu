// Two helpers off the steady decode path:
//
//  * sample_temperature: one CTA per row draws a token from softmax(logits / T) by inverse-CDF over the
//    vocabulary with a caller-supplied uniform number per row (the caller's Philox stream, e.g.
//    torch.rand with its generator), so a run is reproducible from the seed.  Counterpart of the reference
//    sampler (jetspec/core/sampler.py:10-17: softmax(logits / T) + multinomial).
//  * kv_compact: moves the accepted tree positions of a contiguous (Hkv, capacity, 128) cache directly
//    behind the prefix (the reference engine's physical compaction, jetspec/core/llm.py:86-112).  Rows are
//    staged in shared memory first, so overlapping source and destination ranges are safe.
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int kSampleThreads = 1024;

template <typename T>
JS_DEVICE float to_f(T v);
template <>
JS_DEVICE float to_f<float>(float v) { return v; }
template <>
JS_DEVICE float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, int ld, int V, float inv_temp, const float* __restrict__ uniform,
              long long* __restrict__ out) {
  __shared__ float red[32];
  __shared__ float chunk_sum[kSampleThreads];
  __shared__ int pick;
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + static_cast<size_t>(row) * ld;
  // every thread owns one contiguous slice of the vocabulary, so the scan order is the index order
  const int per = (V + kSampleThreads - 1) / kSampleThreads;
  const int lo = min(V, tid * per), hi = min(V, lo + per);
  float mx = -INFINITY;
  for (int i = lo; i < hi; ++i) mx = fmaxf(mx, to_f(x[i]) * inv_temp);
  mx = warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < kSampleThreads / 32; ++i) mx = fmaxf(mx, red[i]);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) s += expf(to_f(x[i]) * inv_temp - mx);
  chunk_sum[tid] = s;
  if (tid == 0) pick = V - 1;
  __syncthreads();
  if (tid == 0) {   // serial scan over 1024 slice sums: exact, order-independent of the launch
    float total = 0.f;
    for (int i = 0; i < kSampleThreads; ++i) total += chunk_sum[i];
    const float target = uniform[row] * total;
    float run = 0.f;
    int owner = kSampleThreads - 1;
    for (int i = 0; i < kSampleThreads; ++i) {
      if (run + chunk_sum[i] > target) { owner = i; break; }
      run += chunk_sum[i];
    }
    red[0] = run;            // mass before the owning slice
    red[1] = target;
    pick = -owner - 1;       // negative: slice index, resolved below
  }
  __syncthreads();
  const int owner = -pick - 1;
  __syncthreads();
  if (tid == owner) {
    float run = red[0];
    const float target = red[1];
    int choice = hi > lo ? hi - 1 : V - 1;
    for (int i = lo; i < hi; ++i) {
      run += expf(to_f(x[i]) * inv_temp - mx);
      if (run > target) { choice = i; break; }
    }
    out[row] = choice;
  }
}

// cache (Hkv, capacity, 128) bf16: position past + i <- position past + keep[i], i < n (n <= 64)
__global__ void kv_compact_kernel(__nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v, int capacity, int past,
                                  const int* __restrict__ keep, int n) {
  extern __shared__ uint4 stage[];     // n rows x 16 chunks of K, then the same of V
  const int h = blockIdx.x;
  __nv_bfloat16* kh = k + static_cast<size_t>(h) * capacity * 128;
  __nv_bfloat16* vh = v + static_cast<size_t>(h) * capacity * 128;
  for (int c = threadIdx.x; c < n * 16; c += blockDim.x) {
    const int r = c >> 4, ch = c & 15;
    const size_t src = static_cast<size_t>(past + keep[r]) * 128 + ch * 8;
    stage[c] = *reinterpret_cast<const uint4*>(kh + src);
    stage[n * 16 + c] = *reinterpret_cast<const uint4*>(vh + src);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < n * 16; c += blockDim.x) {
    const int r = c >> 4, ch = c & 15;
    const size_t dst = static_cast<size_t>(past + r) * 128 + ch * 8;
    *reinterpret_cast<uint4*>(kh + dst) = stage[c];
    *reinterpret_cast<uint4*>(vh + dst) = stage[n * 16 + c];
  }
}

}  // namespace js

// logits (N, V) fp32 (is_bf16 == 0) or bf16; uniform (N) in [0,1); out (N) int64.
extern "C" int js_sample_temperature(const void* logits, int is_bf16, int N, int V, int ld, float temperature,
                                     const float* uniform, long long* out, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (V <= 0 || temperature <= 0.f) return -10;
  const float inv = 1.f / temperature;
  if (is_bf16)
    js::sample_kernel<__nv_bfloat16><<<N, js::kSampleThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, V, inv, uniform, out);
  else
    js::sample_kernel<float><<<N, js::kSampleThreads, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, V, inv, uniform, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int js_kv_compact(void* k, void* v, int Hkv, int capacity, int past, const int* keep, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > 64 || past + n > capacity) return -10;
  const int smem = n * 16 * 16 * 2;
  js::kv_compact_kernel<<<Hkv, 256, smem, stream>>>(reinterpret_cast<__nv_bfloat16*>(k), reinterpret_cast<__nv_bfloat16*>(v),
                                                   capacity, past, keep, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------------------- weight prefetch into L2
// Decode rounds leave HBM idle while attention, norms and the GEMM prologues/epilogues run.  This kernel,
// launched on a side stream, asks the memory system to pull the NEXT GEMM's weights into L2
// (cp.async.bulk.prefetch.L2) so that GEMM finds them there; it only issues requests and exits.
namespace js {
__global__ void l2_prefetch_kernel(const uint8_t* base, size_t bytes, uint32_t chunk) {
  const size_t n = (bytes + chunk - 1) / chunk;
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t off = i * chunk;
    const uint32_t sz = static_cast<uint32_t>(bytes - off < chunk ? bytes - off : chunk) & ~15u;
    if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(sz) : "memory");
  }
}
}  // namespace js

// Prefetch `bytes` (rounded down to 16) starting at the 16-byte aligned `ptr` into L2.
extern "C" int js_l2_prefetch(const void* ptr, size_t bytes, int ctas, cudaStream_t stream) {
  if (bytes < 16) return 0;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return -11;
  if (ctas < 1) ctas = 8;
  js::l2_prefetch_kernel<<<ctas, 128, 0, stream>>>(reinterpret_cast<const uint8_t*>(ptr), bytes, 8192u);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
