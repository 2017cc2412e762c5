// Small tensor-parallel collectives done with peer stores inside the kernel.
// (No counterpart in the reference: its only collectives are the benchmark's NCCL reductions, bench/engine/tps_walltime.py:111-139.)
//
// tp_argmax_combine: the LM head is sharded over the vocabulary; each rank has merged its own
// tiles into a per-row (value, token) pair.  Every rank stores its pairs into every rank's
// gather buffer, bumps a flag there, waits (bounded) for all ranks' pairs and takes the
// maximum, lowest token id winning ties, so all ranks hold the same greedy tokens.
#include "common.cuh"
#include "topk_merge.cuh"

#include <math.h>
#include <cuda_bf16.h>

namespace js {

__global__ void __launch_bounds__(256, 1)
tp_argmax_combine_kernel(const float* part_val, const int* part_idx, int n_tiles, int M, int vocab_offset,
                         float2* const* peer_buf, int* const* peer_flags, int rank, int world, int m_cap,
                         int* out_idx, float* out_val, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  // one CTA per 256 rows, each with its own counter on every rank (all CTAs are resident: at most 16)
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  const int row = blockIdx.x * blockDim.x + tid;
  if (row < M) {
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
      asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(peer_flags[r] + blockIdx.x), "r"(1) : "memory");
    int ok = 0;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(peer_flags[rank] + blockIdx.x) : "memory");
      if (v >= world) { ok = 1; break; }
      __nanosleep(64);
    }
    if (!ok) report(status, kTimeoutPeer);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok && row < M) {
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
  __syncthreads();
  if (tid == 0 && s_ok) peer_flags[rank][blockIdx.x] = 0;
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

// ---------------------------------------------------------------------------------------------------------
// All-reduce tail fused with the NEXT RMSNorm.
//
// A row-parallel GEMM of the decoder (o_proj, down_proj) pushes its bf16 partial tiles over NVLink as 8-byte
// cells {two bf16 values, flag word 1} (EPI_ALLREDUCE of the GEMM kernel, low-latency modes).  This kernel is
// everything that follows until the next GEMM's input exists:
//
//   one shot  (small worlds): every rank received every rank's whole partial (world, m_cap, N); a thread polls
//             the `world` cells of its 8 outputs, sums them in rank order, adds the residual;
//   two shot  (reduce-scatter + all-gather; bytes per rank stay flat as the world grows): rank r received only
//             its N/world column slice from everybody (world, m_cap, N/world).  Phase 1 sums that slice in rank
//             order, adds the residual, rounds to bf16 and stores the result, again as flagged cells, into every
//             rank's gather buffer (m_cap, N); phase 2 polls the gather buffer for the whole row.
//
// Either way each rank then holds the identical new residual row (same numbers added in the same order, or one
// owner's rounded result), writes it, and - when a norm weight is given - applies RMSNorm to it in the same pass
// (the row is still in registers), which is the input of the next column-parallel GEMM.  Consumed cells are
// zeroed for the buffer's next turn.  Every poll is bounded; a poll that runs out reports kTimeoutPeer and the
// kernel finishes with whatever it has (no hang, the host reads the status word).
//
// Deadlock freedom of the two-shot form: phase 1 depends only on GEMM pushes, which the stream order of every
// rank has already issued; phase 2 depends on the peers' phase 1.  Every CTA runs ALL its phase-1 units before
// its first phase-2 poll, and the grid is sized to be fully resident, so no phase-1 unit anywhere waits behind a
// phase-2 poll.
constexpr int kFinishThreads = 256;
constexpr int kFinishMaxGroups = 4;      // 8-column groups per thread and row: N <= 8192
constexpr int kFinishMaxWorld = 8;
constexpr uint32_t kCellPolls = 1u << 21;

struct FinishNormParams {
  unsigned long long* rs_recv;               // this rank's first-phase cells
  unsigned long long* const* ag_peers;       // [world] every rank's gather buffer (two shot), else null
  const __nv_bfloat16* residual;             // (M, N) or null
  __nv_bfloat16* x_out;                      // (M, N) new residual stream (may alias residual)
  const __nv_bfloat16* norm_w;               // (N) or null: no norm
  __nv_bfloat16* h_out;                      // (M, N) normalised rows
  int ldx, ldh;
  float eps;
  int M, N, m_cap, world, rank, two_shot;
  // one shot: the `world` sources of the 8 values at (row, c) sit at rs_recv + row * row_stride + c / 2 +
  // src * src_stride (cells).  Tensor parallelism: (world, m_cap, N) -> row_stride N/2, src_stride m_cap*N/2.
  // Expert-parallel combine: the "sources" are a token's k expert outputs, (T, k, H) -> row_stride k*H/2,
  // src_stride H/2, summed in choice order.
  size_t row_stride, src_stride;
  int* status;
};

JS_DEVICE void ld_cells4(const unsigned long long* p, uint4& a, uint4& b) {
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p) : "memory");
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + 2) : "memory");
}
JS_DEVICE bool cells4_ready(const uint4& a, const uint4& b) { return a.y == 1u && a.w == 1u && b.y == 1u && b.w == 1u; }
JS_DEVICE void st_cells4(unsigned long long* p, const uint4& d) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d.x), "r"(1u), "r"(d.y), "r"(1u) : "memory");
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p + 2), "r"(d.z), "r"(1u), "r"(d.w), "r"(1u) : "memory");
}
JS_DEVICE void zero_cells4(unsigned long long* p) {
  *reinterpret_cast<uint4*>(p) = make_uint4(0u, 0u, 0u, 0u);
  *reinterpret_cast<uint4*>(p + 2) = make_uint4(0u, 0u, 0u, 0u);
}
JS_DEVICE void add_bf16x8(const uint4& a, const uint4& b, float* acc) {   // the 8 payload values of 4 cells
  const unsigned int d[4] = {a.x, a.z, b.x, b.z};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d[u]));
    acc[2 * u] += v2.x;
    acc[2 * u + 1] += v2.y;
  }
}
JS_DEVICE void add_bf16x8_plain(const uint4& v, float* acc) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float2 f = __bfloat1622float2(h[u]);
    acc[2 * u] += f.x;
    acc[2 * u + 1] += f.y;
  }
}
JS_DEVICE uint4 pack_bf16x8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// Sum over `world` sources of the 8 values at `cells + src * src_stride` (cells of 8 bytes), in rank order.
// All sources' loads are in flight together; only the ones not yet flagged are loaded again.  Zeroes the cells.
JS_DEVICE bool gather_sources(unsigned long long* cells, size_t src_stride, int world, float* acc) {
  uint4 a[kFinishMaxWorld], b[kFinishMaxWorld];
  unsigned pending = (1u << world) - 1u;
  for (uint32_t it = 0; it < kCellPolls && pending; ++it) {
#pragma unroll
    for (int s = 0; s < kFinishMaxWorld; ++s)
      if (s < world && (pending >> s & 1u)) ld_cells4(cells + s * src_stride, a[s], b[s]);
#pragma unroll
    for (int s = 0; s < kFinishMaxWorld; ++s)
      if (s < world && (pending >> s & 1u) && cells4_ready(a[s], b[s])) pending &= ~(1u << s);
    if (pending && it > 8) __nanosleep(20);
  }
  if (pending) return false;
#pragma unroll
  for (int s = 0; s < kFinishMaxWorld; ++s)
    if (s < world) {
      add_bf16x8(a[s], b[s], acc);
      zero_cells4(cells + s * src_stride);
    }
  return true;
}

__global__ void __launch_bounds__(kFinishThreads, 2)
tp_finish_norm_kernel(FinishNormParams p) {
  pdl_launch_dependents();
  pdl_wait();                       // this GPU's own GEMM has completed; only other GPUs are waited for below
  __shared__ float red[kFinishThreads / 32];
  __shared__ float s_inv;
  const int tid = threadIdx.x;
  const int N = p.N;
  bool ok = true, ok2 = true;

  if (p.two_shot) {
    // ---- phase 1: reduce this rank's column slice, broadcast the rounded result
    const int Nw = N / p.world;
    const int gpr = Nw >> 3;                                   // 8-column groups of the slice per row
    const int total = p.M * gpr;
    const size_t src_stride = (static_cast<size_t>(p.m_cap) * Nw) >> 1;
    for (int u = blockIdx.x * kFinishThreads + tid; u < total; u += gridDim.x * kFinishThreads) {
      const int r = u / gpr, cl = (u - r * gpr) << 3, c = p.rank * Nw + cl;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      unsigned long long* cells = p.rs_recv + ((static_cast<size_t>(r) * Nw + cl) >> 1);
      if (!gather_sources(cells, src_stride, p.world, acc)) { ok = false; continue; }
      if (p.residual != nullptr)
        add_bf16x8_plain(*reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(r) * p.ldx + c), acc);
      const uint4 ov = pack_bf16x8(acc);
      const size_t cell = (static_cast<size_t>(r) * N + c) >> 1;
      for (int q = 0; q < p.world; ++q) st_cells4(p.ag_peers[q] + cell, ov);     // own gather buffer included
    }
  }

  // ---- phase 2 (or the whole job, one shot): one row per CTA turn
  unsigned long long* ag_mine = p.two_shot ? p.ag_peers[p.rank] : nullptr;
  const int groups = N >> 3;
  for (int row = blockIdx.x; row < p.M; row += gridDim.x) {
    uint4 keep[kFinishMaxGroups];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kFinishMaxGroups; ++i) {
      const int g = tid + i * kFinishThreads;
      if (g >= groups) continue;
      const int c = g << 3;
      uint4 ov = make_uint4(0u, 0u, 0u, 0u);
      if (p.two_shot) {
        unsigned long long* cells = ag_mine + ((static_cast<size_t>(row) * N + c) >> 1);
        uint4 a, b;
        bool got = false;
        for (uint32_t it = 0; it < kCellPolls; ++it) {
          ld_cells4(cells, a, b);
          if (cells4_ready(a, b)) { got = true; break; }
          if (it > 8) __nanosleep(20);
        }
        if (got) {
          ov = make_uint4(a.x, a.z, b.x, b.z);
          zero_cells4(cells);
        } else {
          ok2 = false;
        }
      } else {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        unsigned long long* cells = p.rs_recv + static_cast<size_t>(row) * p.row_stride + (c >> 1);
        if (gather_sources(cells, p.src_stride, p.world, acc)) {
          if (p.residual != nullptr)
            add_bf16x8_plain(*reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.ldx + c), acc);
          ov = pack_bf16x8(acc);
        } else {
          ok = false;
        }
      }
      keep[i] = ov;
      *reinterpret_cast<uint4*>(p.x_out + static_cast<size_t>(row) * p.ldx + c) = ov;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
      add_bf16x8_plain(ov, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    if (p.norm_w != nullptr) {          // uniform for the CTA: every thread reaches the barriers
      ss = warp_sum(ss);
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      if (tid < 32) {
        float v = tid < kFinishThreads / 32 ? red[tid] : 0.f;
        v = warp_sum(v);
        if (tid == 0) s_inv = rsqrtf(v / N + p.eps);
      }
      __syncthreads();
      const float inv = s_inv;
#pragma unroll
      for (int i = 0; i < kFinishMaxGroups; ++i) {
        const int g = tid + i * kFinishThreads;
        if (g >= groups) continue;
        const int c = g << 3;
        float f[8], w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { f[j] = 0.f; w[j] = 0.f; }
        add_bf16x8_plain(keep[i], f);
        add_bf16x8_plain(*reinterpret_cast<const uint4*>(p.norm_w + c), w);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * inv * w[j];
        *reinterpret_cast<uint4*>(p.h_out + static_cast<size_t>(row) * p.ldh + c) = pack_bf16x8(f);
      }
      __syncthreads();                  // red / s_inv are reused by the next row
    }
  }
  if (!ok) report(p.status, kTimeoutCellsReduce);
  if (!ok2) report(p.status, kTimeoutCellsGather);
}

// ---------------------------------------------------------------------------------------------------------
// Vocabulary-parallel top-k with full-vocabulary log-probabilities (the draft head's logits under tensor
// parallelism): every rank ran the top-k epilogue over ITS vocabulary shard.  One CTA per row merges the local
// tiles (topk_merge_row), stores the row's record {8 values, 8 global token ids, running max, sum of exp} as
// flagged 8-byte cells into every rank's exchange buffer, polls (bounded) its own buffer for all ranks' records,
// and merges them: larger value first, lower token id among equals, log-sum-exp folded in rank order - the same
// arithmetic on every rank, so the replicas' draft trees stay identical.  Consumed cells are zeroed.
constexpr int kTopkRecWords = 18;

__global__ void __launch_bounds__(256)
tp_topk_combine_kernel(const float* part_val, const int* part_idx, const float* part_lse, int n_tiles, int M, int K,
                       int vocab_offset, unsigned long long* const* peer_buf, int rank, int world, int m_cap,
                       int* out_tok, float* out_lp, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= M) return;
  __shared__ float win_v[8];
  __shared__ int win_i[8];
  __shared__ float row_m, row_s;
  __shared__ unsigned int rec[kFinishMaxWorld][kTopkRecWords];
  __shared__ int s_bad;
  const int tid = threadIdx.x;
  if (tid == 0) s_bad = 0;
  topk_merge_row(part_val, part_idx, part_lse, n_tiles, row, 8, win_v, win_i, &row_m, &row_s);
  if (tid < kTopkRecWords) {
    unsigned int w;
    if (tid < 8) w = __float_as_uint(win_v[tid]);
    else if (tid < 16) w = static_cast<unsigned int>(win_i[tid - 8] == 0x7fffffff ? 0x7fffffff : win_i[tid - 8] + vocab_offset);
    else w = __float_as_uint(tid == 16 ? row_m : row_s);
    const size_t cell = (static_cast<size_t>(rank) * m_cap + row) * kTopkRecWords + tid;
    for (int q = 0; q < world; ++q)
      asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(peer_buf[q] + cell), "r"(w), "r"(1u) : "memory");
  }
  if (tid < kTopkRecWords * world) {
    const int src = tid / kTopkRecWords, w = tid - src * kTopkRecWords;
    unsigned long long* cell = peer_buf[rank] + (static_cast<size_t>(src) * m_cap + row) * kTopkRecWords + w;
    unsigned int lo = 0, hi = 0;
    bool got = false;
    for (uint32_t it = 0; it < kCellPolls; ++it) {
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "l"(cell) : "memory");
      if (hi == 1u) { got = true; break; }
      if (it > 8) __nanosleep(20);
    }
    if (got) {
      rec[src][w] = lo;
      *cell = 0ull;
    } else {
      s_bad = 1;
    }
  }
  __syncthreads();
  if (s_bad) {
    if (tid == 0) report(status, kTimeoutTopk);
    return;
  }
  if (tid == 0) {
    float gm = -INFINITY, gs = 0.f;
    for (int s = 0; s < world; ++s) {
      const float m2 = __uint_as_float(rec[s][16]), s2 = __uint_as_float(rec[s][17]);
      const float m = fmaxf(gm, m2);
      if (m != -INFINITY) { gs = gs * __expf(gm - m) + s2 * __expf(m2 - m); gm = m; }
    }
    const float lse = gm + logf(gs);
    int head[kFinishMaxWorld];
    for (int s = 0; s < world; ++s) head[s] = 0;
    for (int k = 0; k < K; ++k) {      // K-way merge of sorted lists; vocabulary shards are disjoint
      float bv = -INFINITY;
      int bi = 0x7fffffff, bs = -1;
      for (int s = 0; s < world; ++s) {
        if (head[s] >= 8) continue;
        const float v = __uint_as_float(rec[s][head[s]]);
        const int ix = static_cast<int>(rec[s][8 + head[s]]);
        if (bs < 0 || cand_better(v, ix, bv, bi)) { bv = v; bi = ix; bs = s; }
      }
      if (bs >= 0) ++head[bs];
      out_tok[row * K + k] = bi;
      out_lp[row * K + k] = bv - lse;
    }
  }
}

}  // namespace js

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
  if (M > m_cap || M > 16 * 256) return -10;       // 16 counters per flag buffer
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3((M + 255) / 256);
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

// Tail of a row-parallel GEMM's all-reduce fused with the following RMSNorm (see tp_finish_norm_kernel).
// rs_recv: THIS rank's first-phase cell buffer; ag_peers: device array of `world` gather-buffer addresses (two
// shot) or null (one shot).  norm_w / h_out may be null (no norm).  x_out may alias residual.
extern "C" int js_tp_finish_norm(void* rs_recv, void* const* ag_peers, const void* residual, void* x_out, int ldx,
                                 const void* norm_w, void* h_out, int ldh, float eps, int M, int N, int m_cap,
                                 int world, int rank, int two_shot, int* status, int pdl, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((N % 8) || (ldx % 8) || (norm_w != nullptr && (ldh % 8))) return -10;
  if (N > js::kFinishMaxGroups * js::kFinishThreads * 8) return -11;
  if (world < 1 || world > js::kFinishMaxWorld || M > m_cap) return -12;
  if (two_shot && (ag_peers == nullptr || (N % (8 * world)) != 0)) return -13;
  js::FinishNormParams p;
  p.rs_recv = reinterpret_cast<unsigned long long*>(rs_recv);
  p.ag_peers = reinterpret_cast<unsigned long long* const*>(ag_peers);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.x_out = reinterpret_cast<__nv_bfloat16*>(x_out);
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.h_out = reinterpret_cast<__nv_bfloat16*>(h_out);
  p.ldx = ldx; p.ldh = ldh; p.eps = eps;
  p.M = M; p.N = N; p.m_cap = m_cap; p.world = world; p.rank = rank; p.two_shot = two_shot;
  p.row_stride = static_cast<size_t>(N) >> 1;
  p.src_stride = (static_cast<size_t>(m_cap) * N) >> 1;
  p.status = status;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(M < 2 * 148 ? M : 2 * 148);      // all CTAs resident (two per SM): see the deadlock note
  c.blockDim = dim3(js::kFinishThreads);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_finish_norm_kernel, p) == cudaSuccess ? 0 : -4;
}

// Vocabulary-parallel top-K: part_* are this rank's per-tile partials of the top-k GEMM epilogue over its shard;
// peer_buf: device array of `world` exchange buffers of (world, m_cap, 18) 8-byte cells.
extern "C" int js_tp_topk_combine(const float* part_val, const int* part_idx, const float* part_lse, int n_tiles, int M,
                                  int K, int vocab_offset, void* const* peer_buf, int rank, int world, int m_cap,
                                  int* out_tok, float* out_lp, int* status, int pdl, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K < 1 || K > 8 || M > m_cap || world < 1 || world > js::kFinishMaxWorld || M > 148) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(M);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_topk_combine_kernel, part_val, part_idx, part_lse, n_tiles, M, K, vocab_offset,
                            reinterpret_cast<unsigned long long* const*>(peer_buf), rank, world, m_cap, out_tok,
                            out_lp, status) == cudaSuccess ? 0 : -4;
}

// Owner side of the expert-parallel combine: pairs is THIS rank's (T, k, H) buffer of flagged cells that the
// experts' down-projection epilogues of all ranks fill; out[t] = residual[t] + sum over the k choices of token t
// in choice order, and (norm_w given) h_out = RMSNorm(out) * norm_w in the same pass.
extern "C" int js_ep_combine_finish_norm(void* pairs, const void* residual, void* x_out, int ldx, const void* norm_w,
                                         void* h_out, int ldh, float eps, int T, int H, int k, int* status, int pdl,
                                         cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H % 8) || (ldx % 8) || (norm_w != nullptr && (ldh % 8))) return -10;
  if (H > js::kFinishMaxGroups * js::kFinishThreads * 8 || k < 1 || k > js::kFinishMaxWorld) return -11;
  js::FinishNormParams p;
  p.rs_recv = reinterpret_cast<unsigned long long*>(pairs);
  p.ag_peers = nullptr;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.x_out = reinterpret_cast<__nv_bfloat16*>(x_out);
  p.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  p.h_out = reinterpret_cast<__nv_bfloat16*>(h_out);
  p.ldx = ldx; p.ldh = ldh; p.eps = eps;
  p.M = T; p.N = H; p.m_cap = T; p.world = k; p.rank = 0; p.two_shot = 0;
  p.row_stride = (static_cast<size_t>(k) * H) >> 1;
  p.src_stride = static_cast<size_t>(H) >> 1;
  p.status = status;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(T < 2 * 148 ? T : 2 * 148);
  c.blockDim = dim3(js::kFinishThreads);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tp_finish_norm_kernel, p) == cudaSuccess ? 0 : -4;
}
