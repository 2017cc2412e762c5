// MoE routing on the device: softmax over the experts + top-k (+ renormalisation), then the stable
// permutation of the (token, choice) pairs by local expert that the grouped GEMMs consume.
//
// Counterpart of the reference's router path (jetspec/models/moe_fused.py:16-51: softmax, topk, renorm,
// argsort by expert); here two kernels, no host synchronisation, static output shapes (graph-capturable):
//   route:  one warp per token, k rounds of a warp-wide argmax over the token's probabilities
//   sort:   one CTA; shared-memory histogram (integer atomics: counts are exact), scan, and a stable
//           placement where each key's pairs are ranked with warp ballots in pair order
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int kMaxExpertsPerLane = 8;     // experts <= 256
constexpr int kSortThreads = 1024;
constexpr int kSortMaxPairs = 16384;

__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int k, int renorm,
                                 float* __restrict__ wts, int* __restrict__ idx) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[kMaxExpertsPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[static_cast<size_t>(t) * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    v[i] = (lane + 32 * i) < E ? expf(v[i] - mx) : -1.f;    // -1 marks "not an expert"
    sum += fmaxf(v[i], 0.f);
  }
  sum = warp_sum(sum);
  float kept = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    // warp argmax; ties go to the lower expert index
    float best = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) { best = v[i]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    if ((be & 31) == lane) v[be >> 5] = -1.f;      // remove the winner
    kept += best;
    if (lane == j) { my_w = best; my_e = be; }
  }
  if (lane < k) {
    const float p = my_w / sum;
    wts[static_cast<size_t>(t) * k + lane] = renorm ? p / (kept / sum) : p;
    idx[static_cast<size_t>(t) * k + lane] = my_e;
  }
}

// pairs p = t*k + j with expert idx[p]; key = local expert (idx - first) or n_local for other ranks' experts
__global__ void __launch_bounds__(kSortThreads)
moe_sort_kernel(const int* __restrict__ idx, const float* __restrict__ wts, int P, int E, int first, int n_local,
                int* __restrict__ order, float* __restrict__ row_weight, int* __restrict__ group_off,
                int* __restrict__ counts_all, int k, int* __restrict__ token_of_row) {
  extern __shared__ int sh[];
  int* key = sh;                       // P
  int* cnt = key + P;                  // n_local + 1
  int* off = cnt + n_local + 1;        // n_local + 2
  int* call = off + n_local + 2;       // E
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i <= n_local; i += blockDim.x) cnt[i] = 0;
  for (int i = threadIdx.x; i < E; i += blockDim.x) call[i] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = idx[p];
    const int l = e - first;
    const int kk = (l >= 0 && l < n_local) ? l : n_local;
    key[p] = kk;
    atomicAdd(&cnt[kk], 1);
    if (e >= 0 && e < E) atomicAdd(&call[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {   // exclusive scan of the n_local + 1 counts by one warp, 32 entries per step
    const int ln = threadIdx.x;
    int run = 0;
    for (int i0 = 0; i0 <= n_local; i0 += 32) {
      const int i = i0 + ln;
      const int c = i <= n_local ? cnt[i] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (ln >= o) inc += v;
      }
      if (i <= n_local) off[i] = run + inc - c;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (ln == 0) off[n_local + 1] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= n_local; i += blockDim.x) group_off[i] = off[i];
  for (int i = threadIdx.x; i < E; i += blockDim.x) counts_all[i] = call[i];
  // stable placement: warp w ranks the pairs of keys w, w + warps, ...
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int kk = warp; kk <= n_local; kk += warps) {
    int base = off[kk];
    for (int p0 = 0; p0 < P; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < P && key[p] == kk;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int pos = base + __popc(m & ((1u << lane) - 1u));
        order[pos] = p;
        row_weight[pos] = wts[p];
        if (token_of_row != nullptr) token_of_row[pos] = p / k;
      }
      base += __popc(m);
    }
  }
}

// inverse of the sort: inv[pair] = row of that pair in the expert-sorted order
__global__ void moe_invert_kernel(const int* __restrict__ order, int P, int* __restrict__ inv) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < P) {
    const int p = order[i];
    if (p >= 0 && p < P) inv[p] = i;
  }
}

// out[t] = sum_j row_weight[r] * ys[r], r = inv[t*k + j], summed in choice order j = 0..k-1 in fp32
// (no atomics: a token's result does not depend on how the other tokens were routed or scheduled).
// With `residual` (same shape and leading dimension as out, may be out itself) the result is
// residual + bf16(sum): the rounding of a separate bf16 add after the combine, without its launch.
__global__ void __launch_bounds__(128)
moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, int ld, const int* __restrict__ inv,
                   const float* __restrict__ row_weight, int T, int k, int H, const __nv_bfloat16* residual,
                   __nv_bfloat16* out, int ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int r = inv[t * k + j];
      const float w = row_weight[r];
      const uint4 raw = *reinterpret_cast<const uint4*>(ys + static_cast<size_t>(r) * ld + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        acc[2 * e] += w * f.x;
        acc[2 * e + 1] += w * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    if (residual != nullptr) {
      const uint4 rr = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * ldo + c);
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(o2[e]), b = __bfloat1622float2(r2[e]);
        o2[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ldo + c) = o;
  }
}

}  // namespace js

// logits (T, E) fp32 -> wts (T, k) fp32, idx (T, k) int32.  E <= 256, k <= 32.
extern "C" int js_moe_route(const float* logits, int T, int E, int k, int renorm, float* wts, int* idx, int pdl,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 32 * js::kMaxExpertsPerLane || k < 1 || k > 32 || k > E) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3((T + 7) / 8);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::moe_route_kernel, logits, T, E, k, renorm, wts, idx) == cudaSuccess ? 0 : -4;
}

// idx / wts (P = T*k) -> order (P), row_weight (P), group_off (n_local + 1), counts_all (E) and, when
// token_of_row is given, the source token order[r] / k of every sorted row (the gather index of the dispatch).
extern "C" int js_moe_sort(const int* idx, const float* wts, int P, int E, int first, int n_local, int* order,
                           float* row_weight, int* group_off, int* counts_all, int k, int* token_of_row, int pdl,
                           cudaStream_t stream) {
  if (P <= 0) return 0;
  if (k < 1) return -10;
  if (P > js::kSortMaxPairs || n_local < 1 || E < 1) return -10;
  const int smem = (P + 2 * n_local + 3 + E) * 4;
  static int configured[js::kMaxDevicesCached] = {};
  if (js::ensure_dyn_smem(js::moe_sort_kernel, smem, configured) != 0) return -3;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(js::kSortThreads);
  c.dynamicSmemBytes = smem;
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::moe_sort_kernel, idx, wts, P, E, first, n_local, order, row_weight, group_off,
                            counts_all, k, token_of_row) == cudaSuccess ? 0 : -4;
}

// ys (T*k, H) bf16 in expert-sorted row order -> out (T, H) bf16: each token's k expert outputs weighted and
// summed in choice order.  `inv` is a (T*k) int32 scratch.  H a multiple of 8, rows 16-byte aligned.
// residual (optional, (T, H) with leading dimension ldo, may be `out`): out = residual + bf16(sum).
extern "C" int js_moe_combine(const void* ys, int ld, const int* order, const float* row_weight, int T, int k, int H,
                              int* inv, const void* residual, void* out, int ldo, int pdl, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (k < 1 || H % 8 || ld % 8 || ldo % 8) return -10;
  const int P = T * k;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3((P + 255) / 256);
  c.blockDim = dim3(256);
  c.stream = stream;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&c, js::moe_invert_kernel, order, P, inv) != cudaSuccess) return -4;
  c.gridDim = dim3(T);
  c.blockDim = dim3(128);
  return cudaLaunchKernelEx(&c, js::moe_combine_kernel, static_cast<const __nv_bfloat16*>(ys), ld,
                            static_cast<const int*>(inv), row_weight, T, k, H,
                            static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), ldo) == cudaSuccess ? 0 : -4;
}
