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

// Second half of the tensor-parallel row-parallel GEMM: the GEMM kernels of all ranks PUSH their bf16 partial
// tiles into every rank's receive buffer (world, m_cap, N) and bump one flag per CTA; this kernel (one CTA per
// 128 x 128 output tile) waits until the `split` flags of its tile have been bumped by all `world` ranks, sums
// the partials in rank order together with the residual, writes the output and re-arms the flags.  The GEMM
// never waits for a peer, so its tiles keep streaming while earlier tiles cross NVLink.
__global__ void __launch_bounds__(256)
tp_allreduce_finish_kernel(const __nv_bfloat16* recv, int* flags, const __nv_bfloat16* residual, __nv_bfloat16* out,
                           int M, int N, int ldc, int m_cap, int world, int split, int* status) {
  pdl_launch_dependents();
  pdl_wait();                       // this GPU's own GEMM has completed; only other GPUs are waited for below
  __shared__ int s_bad;
  const int nt = blockIdx.x, mt = blockIdx.y;
  int* f = flags + (mt * gridDim.x + nt) * split;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if (threadIdx.x < split) {
    int ok = 0;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f + threadIdx.x) : "memory");
      if (v >= world) { ok = 1; break; }
      __nanosleep(32);
    }
    if (!ok) {
      report(status, kTimeoutPeer);
      s_bad = 1;
    }
  }
  __syncthreads();
  const bool s_ok = s_bad == 0;
  if (s_ok) {
    for (int i = threadIdx.x; i < 128 * 16; i += blockDim.x) {
      const int r = mt * 128 + (i >> 4), c = nt * 128 + (i & 15) * 8;
      if (r >= M || c >= N) continue;
      float acc[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) acc[u] = 0.f;
      for (int src = 0; src < world; ++src) {
        const uint4 pv = __ldcg(reinterpret_cast<const uint4*>(recv + (static_cast<size_t>(src) * m_cap + r) * N + c));
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
        for (int u = 0; u < 4; ++u) { const float2 v2 = __bfloat1622float2(p2[u]); acc[2 * u] += v2.x; acc[2 * u + 1] += v2.y; }
      }
      if (residual != nullptr) {
        const uint4 rv = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(r) * ldc + c);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int u = 0; u < 4; ++u) { const float2 v2 = __bfloat1622float2(r2[u]); acc[2 * u] += v2.x; acc[2 * u + 1] += v2.y; }
      }
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(acc[2 * u], acc[2 * u + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * ldc + c) = ov;
    }
  }
  __syncthreads();
  if (threadIdx.x < split && s_ok) f[threadIdx.x] = 0;      // ready for this buffer's next turn
}

// Low-latency variant: the receive buffer holds 8-byte cells {two bf16 outputs, flag}; a cell is valid once its
// flag word is 1.  Every thread polls the cells it needs (bounded), sums the ranks' values in rank order, adds the
// residual, writes 8 outputs and zeroes the cells for the buffer's next turn.  No counters, no fences.
__global__ void __launch_bounds__(256)
tp_allreduce_finish_ll_kernel(unsigned long long* recv, const __nv_bfloat16* residual, __nv_bfloat16* out, int M, int N,
                              int ldc, int m_cap, int world, int* status) {
  pdl_launch_dependents();
  pdl_wait();                       // this GPU's own GEMM has completed; only other GPUs are waited for below
  const int groups_per_row = N >> 3;                       // one thread = 8 consecutive outputs of one row
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= M * groups_per_row) return;
  const int r = g / groups_per_row, c = (g - r * groups_per_row) << 3;
  float acc[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) acc[u] = 0.f;
  bool ok = true;
  for (int src = 0; src < world && ok; ++src) {
    unsigned long long* cells = recv + (((static_cast<size_t>(src) * m_cap + r) * N + c) >> 1);    // 4 cells = 32 bytes
    uint4 a, b;
    ok = false;
    for (uint32_t it = 0; it < (1u << 21); ++it) {
      // both 16-byte loads are in flight together; every 8-byte cell carries its own flag
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(cells) : "memory");
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(cells + 2) : "memory");
      if (a.y == 1u && a.w == 1u && b.y == 1u && b.w == 1u) { ok = true; break; }
      if (it > 8) __nanosleep(20);
    }
    if (!ok) break;
    const unsigned int d[4] = {a.x, a.z, b.x, b.z};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d[u]));
      acc[2 * u] += v2.x;
      acc[2 * u + 1] += v2.y;
    }
    // consumed: ready for this buffer's next turn
    *reinterpret_cast<uint4*>(cells) = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(cells + 2) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (!ok) {
    report(status, kTimeoutPeer);
    return;
  }
  if (residual != nullptr) {
    const uint4 rv = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(r) * ldc + c);
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
    for (int u = 0; u < 4; ++u) { const float2 v2 = __bfloat1622float2(r2[u]); acc[2 * u] += v2.x; acc[2 * u + 1] += v2.y; }
  }
  uint4 ov;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(acc[2 * u], acc[2 * u + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * ldc + c) = ov;
}

}  // namespace js

// recv: THIS rank's receive buffer of 8-byte cells (world, m_cap, N/2).
extern "C" int js_tp_allreduce_finish_ll(void* recv, const void* residual, void* out, int M, int N, int ldc, int m_cap,
                                         int world, int* status, int pdl, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((N % 8) || (ldc % 8)) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3((static_cast<unsigned>(M) * (N / 8) + 255) / 256);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_allreduce_finish_ll_kernel, reinterpret_cast<unsigned long long*>(recv),
                            reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<__nv_bfloat16*>(out), M, N,
                            ldc, m_cap, world, status) == cudaSuccess ? 0 : -4;
}

// recv: THIS rank's receive buffer (world, m_cap, N); flags: this rank's flag array (one per GEMM CTA).
extern "C" int js_tp_allreduce_finish(const void* recv, int* flags, const void* residual, void* out, int M, int N, int ldc,
                                      int m_cap, int world, int split, int* status, int pdl, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((N % 8) || (ldc % 8) || split < 1 || split > 32) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3((N + 127) / 128, (M + 127) / 128);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_allreduce_finish_kernel, reinterpret_cast<const __nv_bfloat16*>(recv), flags,
                            reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<__nv_bfloat16*>(out), M, N,
                            ldc, m_cap, world, split, status) == cudaSuccess ? 0 : -4;
}

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
