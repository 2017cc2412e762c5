// Small tensor-parallel collectives done with peer stores inside the kernel.
//
// tp_argmax_combine: the LM head is sharded over the vocabulary; each rank has merged its own
// tiles into a per-row (value, token) pair.  Every rank stores its pairs into every rank's
// gather buffer, bumps a flag there, waits (bounded) for all ranks' pairs and takes the
// maximum, lowest token id winning ties, so all ranks hold the same greedy tokens.
#include "common.cuh"

#include <math.h>
#include <cuda_bf16.h>

namespace js {

__global__ void __launch_bounds__(256, 1)
tp_argmax_combine_kernel(const float* part_val, const int* part_idx, int n_tiles, int M, int vocab_offset,
                         float2* const* peer_buf, int* const* peer_flags, int rank, int world, int m_cap,
                         int* out_idx, float* out_val, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  for (int row = tid; row < M; row += blockDim.x) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = 0; i < n_tiles; ++i) {
      const float v = part_val[static_cast<size_t>(row) * n_tiles + i];
      const int ix = part_idx[static_cast<size_t>(row) * n_tiles + i];
      if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
    }
    const float2 pk = make_float2(best, __int_as_float(bi == 0x7fffffff ? bi : bi + vocab_offset));
    for (int r = 0; r < world; ++r) peer_buf[r][static_cast<size_t>(rank) * m_cap + row] = pk;
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    for (int r = 0; r < world; ++r)
      asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(peer_flags[r]), "r"(1) : "memory");
    int ok = 0;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(peer_flags[rank]) : "memory");
      if (v >= world) { ok = 1; break; }
      __nanosleep(64);
    }
    if (!ok) report(status, kTimeoutPeer);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    for (int row = tid; row < M; row += blockDim.x) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int src = 0; src < world; ++src) {
        const float2 pk = __ldcg(peer_buf[rank] + static_cast<size_t>(src) * m_cap + row);
        const int ix = __float_as_int(pk.y);
        if (pk.x > best || (pk.x == best && ix < bi)) { best = pk.x; bi = ix; }
      }
      out_idx[row] = bi;
      if (out_val != nullptr) out_val[row] = best;
    }
  }
  __syncthreads();
  if (tid == 0 && s_ok) *peer_flags[rank] = 0;
}

// Expert-parallel combine, second half: wait (bounded) until every expert CTA of every rank has
// delivered its weighted rows into this rank's pair buffer, then out[t] = residual[t] + sum over the
// k choices of token t, in choice order (the same order on every rank: replicas stay identical).
// The last CTA to finish re-arms the counters for the buffer's next use.
__global__ void __launch_bounds__(256)
ep_combine_finish_kernel(const __nv_bfloat16* pairs, int* cnt, const int* expected, int* done,
                         const __nv_bfloat16* residual, __nv_bfloat16* out, int T, int k, int H, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const int want = *expected;
    int ok = 0;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
      if (v >= want) { ok = 1; break; }
      __nanosleep(64);
    }
    if (!ok) report(status, kTimeoutPeer);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const int vec = H / 8;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < T * vec; i += gridDim.x * blockDim.x) {
      const int t = i / vec, c = i % vec;
      float acc[8];
      {
        const uint4 rv = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c * 8);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(r2[u]); acc[2 * u] = f.x; acc[2 * u + 1] = f.y; }
      }
      for (int j = 0; j < k; ++j) {
        const uint4 pv = __ldcg(reinterpret_cast<const uint4*>(pairs + (static_cast<size_t>(t) * k + j) * H + c * 8));
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
        for (int u = 0; u < 4; ++u) { const float2 f = __bfloat1622float2(p2[u]); acc[2 * u] += f.x; acc[2 * u + 1] += f.y; }
      }
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(acc[2 * u], acc[2 * u + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c * 8) = ov;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done, 1) == static_cast<int>(gridDim.x) - 1) {   // last CTA: re-arm
      *cnt = 0;
      *done = 0;
    }
  }
}

}  // namespace js

extern "C" int js_ep_combine_finish(const void* pairs, int* cnt, const int* expected, int* done, const void* residual,
                                    void* out, int T, int k, int H, int* status, int pdl, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  cudaLaunchConfig_t c = {};
  int blocks = (T * (H / 8) + 255) / 256;
  if (blocks > 148) blocks = 148;      // all CTAs are resident while they wait on the counter
  c.gridDim = dim3(blocks);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::ep_combine_finish_kernel, reinterpret_cast<const __nv_bfloat16*>(pairs), cnt,
                            expected, done, reinterpret_cast<const __nv_bfloat16*>(residual),
                            reinterpret_cast<__nv_bfloat16*>(out), T, k, H, status) == cudaSuccess ? 0 : -4;
}

extern "C" int js_tp_argmax_combine(const float* part_val, const int* part_idx, int n_tiles, int M, int vocab_offset,
                                    void* const* peer_buf, int* const* peer_flags, int rank, int world, int m_cap,
                                    int* out_idx, float* out_val, int* status, int pdl, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > m_cap) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_argmax_combine_kernel, part_val, part_idx, n_tiles, M, vocab_offset,
                            reinterpret_cast<float2* const*>(peer_buf), peer_flags, rank, world, m_cap, out_idx,
                            out_val, status) == cudaSuccess ? 0 : -4;
}
