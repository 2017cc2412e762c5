// Expert-parallel dispatch for sparse-MoE layers whose tokens are SHARDED over the ranks.
// (The reference's MoE is single-GPU, jetspec/models/moe_fused.py:16-116; this exchange has no counterpart there.)
//
// Every rank owns some tokens (its requests' tree nodes) and some experts (E / world consecutive ones).  A
// layer moves each (token, choice) row to the rank that owns the chosen expert, runs the experts there as
// grouped tcgen05 GEMMs, and returns each weighted output row to the token's owner only:
//
//   ep_route_count   softmax / top-k / renormalisation of the local tokens' router logits (one warp per
//                    token), a per-expert histogram of the local (token, choice) pairs, and the histogram
//                    pushed to every rank as flagged 8-byte cells: after this kernel every rank can know the
//                    whole (source rank x expert) count matrix.
//   ep_dispatch      waits (bounded) for all ranks' counts, derives where each source's rows of each expert
//                    start in the owning rank's receive slab (expert-major, then source rank), and stores
//                    every local pair's token row, routing weight and return address straight into that
//                    slab over NVLink with plain 16-byte peer stores.  Rows of one expert are therefore
//                    contiguous on the receiver, which is what the grouped GEMM's row ranges (group_off,
//                    written here) and its local TMA loads need.  One release per (source, destination) tells
//                    the receiver that a source's rows have landed; the last CTA of this kernel waits
//                    (bounded) for all sources before the kernel ends, so the grouped GEMM that follows in
//                    the stream reads a complete slab.
//
// The way back is the epilogue of the experts' down projection (EPI_EP_COMBINE of the GEMM kernel, cell
// mode): each output row, scaled by its routing weight, goes as flagged cells to the (token, choice) slot of
// the token's owner, and the owner's finishing kernel sums a token's k rows in choice order, adds the
// residual and applies the next RMSNorm (tp_finish_norm_kernel with the pair-buffer strides).
//
// Row placement inside an expert's group uses an integer atomic counter, so the ORDER of rows within a group
// can differ from run to run; every output row depends on its own input row only and a token's k rows are
// summed in choice order, so the results do not depend on that order.
//
// Everything re-arms itself: consumed count cells, arrival counters and placement counters are zeroed by
// the last CTA, so the same buffers serve the next layer (a layer cannot start on any rank before every rank
// has consumed the previous layer's cells: its own combine needs all ranks' expert outputs first).
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int kEpMaxExperts = 256;
constexpr int kEpMaxWorld = 8;
constexpr int kEpExpertsPerLane = 8;
constexpr uint32_t kEpPolls = 1u << 21;

struct EpRouteParams {
  const float* logits;     // (T, E) fp32 router logits of the local tokens
  int T, E, k, renorm;
  float* wts;              // (T, k)
  int* idx;                // (T, k) global expert ids
  int* hist;               // (E) zero on entry, zero again on exit
  int* done;               // CTA counter, zero on entry and exit
  unsigned long long* const* cnt_peers;   // [world] -> (world, E) cells on that rank
  int rank, world;
};

__global__ void __launch_bounds__(256)
ep_route_count_kernel(EpRouteParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp_in_cta = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp_in_cta;
  if (t < p.T) {
    float v[kEpExpertsPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kEpExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < p.E ? p.logits[static_cast<size_t>(t) * p.E + e] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kEpExpertsPerLane; ++i) {
      v[i] = (lane + 32 * i) < p.E ? expf(v[i] - mx) : -1.f;    // -1 marks "not an expert"
      sum += fmaxf(v[i], 0.f);
    }
    sum = warp_sum(sum);
    float kept = 0.f, my_w = 0.f;
    int my_e = 0;
    for (int j = 0; j < p.k; ++j) {          // warp argmax; ties go to the lower expert index
      float best = -1.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kEpExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        if (v[i] > best) { best = v[i]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
      }
      if ((be & 31) == lane) v[be >> 5] = -1.f;
      kept += best;
      if (lane == j) { my_w = best; my_e = be; }
    }
    if (lane < p.k) {
      const float pr = my_w / sum;
      p.wts[static_cast<size_t>(t) * p.k + lane] = p.renorm ? pr / (kept / sum) : pr;
      p.idx[static_cast<size_t>(t) * p.k + lane] = my_e;
      atomicAdd(&p.hist[my_e], 1);
    }
  }
  // the last CTA to finish publishes the histogram to every rank and clears it
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(p.done, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const unsigned int c = static_cast<unsigned int>(atomicExch(&p.hist[e], 0));
    const size_t cell = static_cast<size_t>(p.rank) * p.E + e;
    for (int q = 0; q < p.world; ++q)
      asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p.cnt_peers[q] + cell), "r"(c), "r"(1u) : "memory");
  }
  if (threadIdx.x == 0) *p.done = 0;
}

struct EpDispatchParams {
  const __nv_bfloat16* x;      // (T, H) local tokens (the normalised MoE input)
  int ldx;
  const float* wts;            // (T, k)
  const int* idx;              // (T, k)
  int T, H, k, E, n_local, rank, world;
  int slab_rows;               // capacity of every rank's slab
  int max_rows_per_expert;     // rows of one expert the grouped GEMM launch covers
  unsigned long long* cnt_mine;           // (world, E) cells on this rank
  __nv_bfloat16* const* slab_peers;       // [world] -> (slab_rows, H)
  int2* const* meta_peers;                // [world] -> (slab_rows) {source rank, pair index at the source}
  float* const* w_peers;                  // [world] -> (slab_rows) routing weights
  int* const* arrive_peers;               // [world] -> (world) arrival counters
  int* fill;                   // (E) placement counters, zero on entry and exit
  int* done;                   // CTA counter, zero on entry and exit
  int* group_off;              // out: (n_local + 1) row ranges of this rank's experts in its slab
  int* status;
};

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpDispatchParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_cnt[kEpMaxWorld][kEpMaxExperts];   // count matrix (source, expert)
  __shared__ int s_base[kEpMaxExperts];               // first slab row of MY rows of expert e on its owner
  __shared__ int s_ok, s_last;
  const int tid = threadIdx.x;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  for (int i = tid; i < p.world * p.E; i += blockDim.x) {
    unsigned int lo = 0, hi = 0;
    bool got = false;
    for (uint32_t it = 0; it < kEpPolls; ++it) {
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "l"(p.cnt_mine + i) : "memory");
      if (hi == 1u) { got = true; break; }
      if (it > 8) __nanosleep(20);
    }
    if (!got) s_ok = 0;
    s_cnt[i / p.E][i % p.E] = got ? static_cast<int>(lo) : 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  // rows of expert e on its owner: experts in order, inside an expert the sources in rank order
  for (int e = tid; e < p.E; e += blockDim.x) {
    const int first = (e / p.n_local) * p.n_local;
    int base = 0, total_e = 0;
    for (int e2 = first; e2 < e; ++e2)
      for (int s = 0; s < p.world; ++s) base += s_cnt[s][e2];
    for (int s = 0; s < p.world; ++s) {
      if (s < p.rank) base += s_cnt[s][e];
      total_e += s_cnt[s][e];
    }
    s_base[e] = base;
    (void)total_e;      // any number of rows per expert is fine: the grouped GEMM walks on through an expert's row tiles
  }
  if (blockIdx.x == 0 && tid == 0) {     // this rank's own experts: the grouped GEMM's row ranges
    int run = 0;
    for (int le = 0; le < p.n_local; ++le) {
      p.group_off[le] = run;
      for (int s = 0; s < p.world; ++s) run += s_cnt[s][p.rank * p.n_local + le];
    }
    p.group_off[p.n_local] = run;
    if (run > p.slab_rows) report(p.status, kEpOverflow);
  }
  __syncthreads();
  if (ok) {
    const int warp = (blockIdx.x * blockDim.x + tid) >> 5, lane = tid & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int vec = p.H >> 3;
    for (int pr = warp; pr < p.T * p.k; pr += warps) {
      const int e = p.idx[pr];
      if (e < 0 || e >= p.E) continue;
      const int o = e / p.n_local;
      int row = 0;
      if (lane == 0) row = s_base[e] + atomicAdd(&p.fill[e], 1);
      row = __shfl_sync(0xffffffffu, row, 0);
      if (row >= p.slab_rows) continue;                        // reported above
      const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(pr / p.k) * p.ldx);
      uint4* dst = reinterpret_cast<uint4*>(p.slab_peers[o] + static_cast<size_t>(row) * p.H);
      for (int i = lane; i < vec; i += 32) dst[i] = src[i];
      if (lane == 0) {
        p.meta_peers[o][row] = make_int2(p.rank, pr);
        p.w_peers[o][row] = p.wts[pr];
      }
    }
  }
  // publish: every thread's peer stores, then one release per destination from the last CTA
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(p.done, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (tid < p.world)
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p.arrive_peers[tid] + p.rank), "r"(1) : "memory");
  // wait for every source's rows, then re-arm everything this layer used
  if (tid < p.world) {
    int* mine = p.arrive_peers[p.rank] + tid;
    bool got = false;
    for (uint32_t it = 0; it < kEpPolls; ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v >= 1) { got = true; break; }
      __nanosleep(40);
    }
    if (!got) report(p.status, kTimeoutEpArrive);
    *mine = 0;
  }
  for (int i = tid; i < p.world * p.E; i += blockDim.x) p.cnt_mine[i] = 0ull;
  for (int e = tid; e < p.E; e += blockDim.x) p.fill[e] = 0;
  if (!ok && tid == 0) report(p.status, kTimeoutEpCounts);
  if (tid == 0) *p.done = 0;
}

}  // namespace js

// Router + histogram + count exchange for the local tokens.  hist (E ints) and done (1 int) are scratch words
// that must be zero before the first call (the kernel leaves them zero).  T may be 0 (a rank without tokens
// still publishes its zero counts).
extern "C" int js_ep_route_count(const float* logits, int T, int E, int k, int renorm, float* wts, int* idx, int* hist,
                                 int* done, void* const* cnt_peers, int rank, int world, int pdl, cudaStream_t stream) {
  if (E > js::kEpMaxExperts || E > 32 * js::kEpExpertsPerLane || k < 1 || k > 32 || k > E) return -10;
  if (world < 1 || world > js::kEpMaxWorld || T < 0) return -11;
  js::EpRouteParams p{logits, T, E, k, renorm, wts, idx, hist, done,
                      reinterpret_cast<unsigned long long* const*>(cnt_peers), rank, world};
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(T > 0 ? (T + 7) / 8 : 1);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::ep_route_count_kernel, p) == cudaSuccess ? 0 : -4;
}

// Dispatch of the local (token, choice) rows to the owners of their experts (see the file comment).
extern "C" int js_ep_dispatch(const void* x, int ldx, const float* wts, const int* idx, int T, int H, int k, int E,
                              int n_local, int rank, int world, int slab_rows, int max_rows_per_expert, void* cnt_mine,
                              void* const* slab_peers, void* const* meta_peers, void* const* w_peers,
                              int* const* arrive_peers, int* fill, int* done, int* group_off, int* status, int pdl,
                              cudaStream_t stream) {
  if ((H % 8) || (ldx % 8) || E > js::kEpMaxExperts || world < 1 || world > js::kEpMaxWorld || n_local * world != E)
    return -10;
  js::EpDispatchParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx; p.wts = wts; p.idx = idx;
  p.T = T; p.H = H; p.k = k; p.E = E; p.n_local = n_local; p.rank = rank; p.world = world;
  p.slab_rows = slab_rows; p.max_rows_per_expert = max_rows_per_expert;
  p.cnt_mine = reinterpret_cast<unsigned long long*>(cnt_mine);
  p.slab_peers = reinterpret_cast<__nv_bfloat16* const*>(slab_peers);
  p.meta_peers = reinterpret_cast<int2* const*>(meta_peers);
  p.w_peers = reinterpret_cast<float* const*>(w_peers);
  p.arrive_peers = arrive_peers;
  p.fill = fill; p.done = done; p.group_off = group_off; p.status = status;
  const int pairs = T * k;
  int ctas = (pairs + 7) / 8;          // one warp per pair, 8 warps per CTA
  if (ctas < 1) ctas = 1;
  if (ctas > 148) ctas = 148;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(ctas);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::ep_dispatch_kernel, p) == cudaSuccess ? 0 : -4;
}
