// Device-side tree construction and acceptance/commit, so that a whole decode round
// (draft -> build -> verify -> accept -> commit) replays from one CUDA graph with a single
// host read at the end.
//
// tree_build: best-first expansion under a node budget, bit-identical to the host builder
// (largest cumulative log-probability first, held in double, ties broken by insertion order;
// per-depth fan-out caps; the budget counts the root).  Also emits what the verify forward
// needs: rotary positions (past + depth), KV slots of the tree window, packed ancestor bits,
// and pad rows up to the graph's bucket size (token 0, last real position, self-only mask).
//
// tree_accept_commit: greedy acceptance (token == target argmax at the parent, the later of
// two equal siblings wins, deepest fully matching path), then the commit: permute the
// window's slot-map entries so the accepted nodes' slots become positions past..past+acc,
// append accepted tokens + correction to the committed-token buffer, advance the sequence
// state, check EOS, and write a small result record for the host.
//
// Reference behaviour: jetspec/tree/_core/fanout_cap_builder.py:18-75, accept.py:73-141,
// and the no-gather commit at jetspec/inference_engine/engine.py:1114-1125.
#include "common.cuh"

namespace js {

constexpr int kMaxNodes = 256;
constexpr int kMaxWords = kMaxNodes / 32;
constexpr int kMaxCand = 512;       // depth x width entries of the candidate table staged in shared memory
constexpr int kMaxCapDepth = 64;

// sequence state (int32 words) shared by the round's kernels
enum : int { ST_PAST = 0, ST_CTX = 1, ST_NEW = 2, ST_DONE = 3, ST_GEN = 4, ST_NNODES = 5, ST_ROUNDS = 6 };

__global__ void __launch_bounds__(256, 1)
tree_build_kernel(const int* topk_tok, const float* topk_lp, const int* caps, int D, int K, int budget, int NB, int W,
                  const int* committed, int* state, const int* slot_map, const int* seq_row, int max_len,
                  int* tokens, int* parents, int* depth, int* positions, int* slots, int* mask_bits, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int* slot_row = slot_map + static_cast<size_t>(*seq_row) * max_len;
  __shared__ int s_tok[kMaxNodes], s_par[kMaxNodes], s_dep[kMaxNodes];
  __shared__ int s_bits[kMaxNodes][kMaxWords];
  __shared__ int s_n;
  // the candidate table, staged once by the whole block: the serial expansion below then never waits on
  // global memory (one dependent global load per pushed node was most of this kernel's time)
  __shared__ float c_lp[kMaxCand];
  __shared__ int c_tok[kMaxCand], c_cap[kMaxCapDepth];
  const int tid = threadIdx.x;
  const int past = state[ST_PAST];
  if (budget > NB) budget = NB;
  const bool staged = D * K <= kMaxCand && D <= kMaxCapDepth;
  if (staged) {
    for (int i = tid; i < D * K; i += blockDim.x) {
      c_lp[i] = topk_lp[i];
      c_tok[i] = topk_tok[i];
    }
    for (int i = tid; i < D; i += blockDim.x) c_cap[i] = (caps != nullptr) ? caps[i] : K;
  }
  __syncthreads();
  const float* lp_tab = staged ? c_lp : topk_lp;
  const int* tok_tab = staged ? c_tok : topk_tok;

  // Best-first expansion without a heap.  Nodes are numbered in push order, so "insertion order" IS the node index
  // and the heap's pop (smallest (key, order)) is an argmin over the nodes that were pushed and not yet popped.
  // Thread i owns node i: its key lives in a register; one block-wide argmin (shuffles + one barrier) per pop
  // replaces the serial sift-down, and the children of the popped node are written by `take` threads at once.
  __shared__ double r_key[2][8];
  __shared__ int r_idx[2][8];
  const int lane = tid & 31, warp = tid >> 5;
  double my_key = 0.0;            // negated cumulative log-probability of node `tid`
  bool alive = (tid == 0);
  int n = 1, max_dep = 0;      // uniform across the block
  if (tid == 0) {
    s_tok[0] = committed[past];
    s_par[0] = -1;
    s_dep[0] = 0;
  }
  __syncthreads();
  for (int it = 0; it <= kMaxNodes && n < budget; ++it) {
    double k = alive ? my_key : INFINITY;
    int ix = alive ? tid : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ok = __shfl_xor_sync(0xffffffffu, k, o);
      const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
      if (ok < k || (ok == k && oi < ix)) { k = ok; ix = oi; }
    }
    const int buf = it & 1;
    if (lane == 0) { r_key[buf][warp] = k; r_idx[buf][warp] = ix; }
    __syncthreads();
    k = r_key[buf][0];
    ix = r_idx[buf][0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      const double ok = r_key[buf][w];
      const int oi = r_idx[buf][w];
      if (ok < k || (ok == k && oi < ix)) { k = ok; ix = oi; }
    }
    if (ix == 0x7fffffff) break;                 // nothing left to pop
    if (tid == ix) alive = false;
    const int d = s_dep[ix];
    if (d >= D) continue;
    int take = staged ? c_cap[d] : ((caps != nullptr) ? caps[d] : K);
    if (take > K) take = K;
    if (take > budget - n) take = budget - n;
    const int jc = tid - n;                      // thread n + j creates child j
    if (jc >= 0 && jc < take) {
      const double cum = -k + static_cast<double>(lp_tab[d * K + jc]);
      s_tok[tid] = tok_tab[d * K + jc];
      s_par[tid] = ix;
      s_dep[tid] = d + 1;
      my_key = -cum;
      alive = true;
    }
    if (take > 0 && d + 1 > max_dep) max_dep = d + 1;
    n += take;
  }
  if (tid == 0) {
    s_n = n;
    state[ST_NNODES] = n;
  }
  __syncthreads();
  // ancestor bits, one node per thread: walk the parent chain (parents precede children, depth <= D)
  for (int i = tid; i < s_n; i += blockDim.x) {
    int bits[kMaxWords];
#pragma unroll
    for (int w = 0; w < kMaxWords; ++w) bits[w] = 0;
    int c = i, steps = 0;
    while (c >= 0 && steps <= kMaxNodes) {
#pragma unroll
      for (int w = 0; w < kMaxWords; ++w)
        if (w == (c >> 5)) bits[w] |= (1 << (c & 31));
      c = s_par[c];
      ++steps;
    }
#pragma unroll
    for (int w = 0; w < kMaxWords; ++w) s_bits[i][w] = bits[w];
  }
  __syncthreads();
  const int last_pos = past + max_dep;
  for (int i = tid; i < NB; i += blockDim.x) {
    const bool real = i < n;
    tokens[i] = real ? s_tok[i] : 0;
    parents[i] = real ? s_par[i] : -1;
    depth[i] = real ? s_dep[i] : 0;
    positions[i] = real ? past + s_dep[i] : last_pos;
    const int pos = past + i;
    if (pos < max_len) {
      slots[i] = slot_row[pos];
    } else {
      slots[i] = 0;
      report(status, kBadSlot);
    }
    for (int w = 0; w < W; ++w) mask_bits[i * W + w] = real ? s_bits[i][w] : ((w == (i >> 5)) ? (1 << (i & 31)) : 0);
  }
}

__global__ void __launch_bounds__(256, 1)
tree_accept_commit_kernel(const int* tokens, const int* parents, const int* depth, const int* greedy, int NB,
                          int* state, int* slot_map, const int* seq_row, int max_len, int* committed,
                          int committed_cap, const int* eos_ids, int n_eos, int max_new, int* path_idx, int* result,
                          int* status) {
  pdl_launch_dependents();
  pdl_wait();
  int* slot_row = slot_map + static_cast<size_t>(*seq_row) * max_len;
  __shared__ int s_tok[kMaxNodes], s_par[kMaxNodes], s_dep[kMaxNodes], s_grd[kMaxNodes], s_ok[kMaxNodes];
  __shared__ int s_slot[kMaxNodes], s_inpath[kMaxNodes], s_path[kMaxNodes];
  __shared__ unsigned long long s_best;
  __shared__ int s_acc;
  const int tid = threadIdx.x;
  const int n = state[ST_NNODES];
  const int past = state[ST_PAST];
  if (tid == 0) s_best = 0ull;
  for (int i = tid; i < NB; i += blockDim.x) {
    s_tok[i] = tokens[i];
    s_par[i] = parents[i];
    s_dep[i] = depth[i];
    s_grd[i] = greedy[i];
    s_inpath[i] = 0;
    const int pos = past + i;
    s_slot[i] = pos < max_len ? slot_row[pos] : 0;
  }
  __syncthreads();
  // per-node match
  for (int i = tid; i < NB; i += blockDim.x) {
    int ok = 0;
    if (i == 0) {
      ok = 1;
    } else if (i < n) {
      const int pr = s_par[i];
      if (pr >= 0 && pr < n && s_tok[i] == s_grd[pr]) {
        ok = 1;
        for (int j = i + 1; j < n; ++j)
          if (s_par[j] == pr && s_tok[j] == s_tok[i]) { ok = 0; break; }   // a later equal sibling wins
      }
    }
    s_ok[i] = ok;
  }
  __syncthreads();
  // whole root path must match; pick the deepest such node (lowest index on equal depth)
  for (int i = tid; i < n; i += blockDim.x) {
    int c = i, good = 1, steps = 0;
    while (c > 0 && steps <= kMaxNodes) {
      if (!s_ok[c]) { good = 0; break; }
      c = s_par[c];
      if (c < 0 || c >= n) { good = 0; report(status, kBadNode); break; }
      ++steps;
    }
    if (good) {
      const unsigned long long key = (static_cast<unsigned long long>(s_dep[i] + 1) << 32) |
                                     static_cast<unsigned long long>(0x7fffffff - i);
      atomicMax(&s_best, key);
    }
  }
  __syncthreads();
  if (tid == 0) {
    const int best = 0x7fffffff - static_cast<int>(s_best & 0xffffffffull);
    const int acc = s_dep[best];
    s_acc = acc;
    int c = best;
    for (int d = acc; d >= 0; --d) {
      s_path[d] = c;
      s_inpath[c] = 1;
      c = s_par[c] < 0 ? 0 : s_par[c];
    }
    const int corr = s_grd[best];
    // committed tokens: root is committed[past]; accepted nodes then the correction follow
    int eos_at = -1;
    int gen = state[ST_GEN];
    int emitted = 0;
    for (int j = 0; j <= acc; ++j) {
      const int tok = j < acc ? s_tok[s_path[j + 1]] : corr;
      const int pos = past + 1 + j;
      if (pos < committed_cap) committed[pos] = tok;
      result[8 + j] = tok;
      ++emitted;
      bool is_eos = false;
      for (int e = 0; e < n_eos; ++e) is_eos |= (eos_ids[e] == tok);
      if (is_eos && eos_at < 0) eos_at = j;
    }
    gen += emitted;
    result[0] = acc;
    result[1] = corr;
    result[2] = eos_at;
    result[3] = n;
    result[4] = past + acc + 1;
    result[5] = gen;
    result[6] = atomicAdd(status, 0);
    for (int j = 0; j <= acc; ++j) path_idx[j] = s_path[j];
    state[ST_PAST] = past + acc + 1;
    state[ST_NEW] = acc + 1;
    state[ST_GEN] = gen;
    state[ST_ROUNDS] = state[ST_ROUNDS] + 1;
    if (eos_at >= 0 || gen >= max_new) state[ST_DONE] = 1;
  }
  __syncthreads();
  // slot-map permutation of the window: accepted path first (path order), the rest after
  const int acc = s_acc;
  for (int i = tid; i < NB; i += blockDim.x) {
    int dst;
    if (s_inpath[i]) {
      dst = s_dep[i];                 // a path node's order on the path is its depth
    } else {
      int before = 0;
      for (int j = 0; j < i; ++j) before += s_inpath[j] ? 0 : 1;
      dst = acc + 1 + before;
    }
    const int pos = past + dst;
    if (pos < max_len) slot_row[pos] = s_slot[i];
  }
}

// positions / slots / block token ids of one draft-head step.  The block is
// [anchor, mask, mask, ...]; its rows sit at positions ctx .. ctx+bs-1 where ctx is the
// context length AFTER this round's new rows (state[ST_CTX] + state[ST_NEW]).
// `fill` (optional): n_fill tokens, `fill_stride` ints apart, that replace the first mask tokens of the block - the
// path-conditioned form of the step (the block then reads [anchor, fill_0, fill_1, ..., mask, ...]).
__global__ void draft_prep_kernel(int* state, const int* committed, int mask_token, int bs, int rows_pad,
                                  int ctx_rows_pad, int* block_ids, int* block_pos, int* ctx_pos, int* n_new_out,
                                  const int* fill, int fill_stride, int n_fill) {
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int ctx_old = state[ST_CTX];
  const int n_new = state[ST_NEW];
  const int ctx = ctx_old + n_new;
  const int past = state[ST_PAST];
  for (int i = tid; i < rows_pad; i += blockDim.x) {
    block_ids[i] = (i == 0) ? committed[past]
                            : ((fill != nullptr && i - 1 < n_fill) ? fill[(i - 1) * fill_stride] : mask_token);
    block_pos[i] = ctx + i;
  }
  for (int i = tid; i < ctx_rows_pad; i += blockDim.x) ctx_pos[i] = ctx_old + i;
  __syncthreads();
  if (tid == 0) {
    *n_new_out = n_new;
    state[ST_CTX] = ctx;
    state[ST_NEW] = 0;
  }
}

// Gate of the tree extension ("ceiling raise"): fires when the drafter's rank-1 chain is fully present in the built
// tree and the mean top-1 / top-2 gap along it exceeds the threshold, and there is room for `ext` more nodes.
// out = {fire, leaf node of the chain, node count}.  One thread: the tree has at most a few hundred nodes.
__global__ void tree_ext_gate_kernel(const int* tokens, const int* parents, const int* state, const int* topk_tok,
                                     const float* topk_lp, int D, int K, float gap_threshold, int ext, int NB,
                                     int* out) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0) return;
  const int n = state[ST_NNODES];
  int node = 0, fire = (K >= 2 && D > 0 && n + ext <= NB) ? 1 : 0;
  float gap = 0.f;
  for (int d = 0; d < D && fire; ++d) {
    const int want = topk_tok[d * K];
    int child = -1;
    for (int i = node + 1; i < n; ++i)
      if (parents[i] == node && tokens[i] == want) { child = i; break; }
    if (child < 0) fire = 0;
    node = child;
    gap += topk_lp[d * K] - topk_lp[d * K + 1];
  }
  if (fire && !(gap / static_cast<float>(D) > gap_threshold)) fire = 0;
  out[0] = fire;
  out[1] = fire ? node : 0;
  out[2] = n;
}

// Chain extension: `ext` nodes, one under the other, below `leaf`; their tokens are the argmax of the first `ext`
// rows of the path-conditioned draft pass.  Rows n .. n+ext-1 of the round's tree arrays were pad rows (their KV
// slots are already assigned); they become real nodes here and the node count grows.
__global__ void tree_ext_splice_kernel(int* tokens, int* parents, int* depth, int* positions, int* mask_bits,
                                       int* state, const int* gate, const int* ext_tok, int ext, int NB, int W,
                                       int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0 || gate[0] == 0) return;
  const int leaf = gate[1], n = gate[2], past = state[ST_PAST];
  if (leaf < 0 || leaf >= n || n + ext > NB) {
    report(status, kBadNode);
    return;
  }
  for (int i = 0; i < ext; ++i) {
    const int idx = n + i, par = (i == 0) ? leaf : idx - 1;
    tokens[idx] = ext_tok[i];
    parents[idx] = par;
    depth[idx] = depth[par] + 1;
    positions[idx] = past + depth[idx];
    for (int w = 0; w < W; ++w) mask_bits[idx * W + w] = mask_bits[par * W + w] | ((w == (idx >> 5)) ? (1 << (idx & 31)) : 0);
  }
  state[ST_NNODES] = n + ext;
}

// Fan-out caps of one round from that round's per-depth top-k log-probs, on the device, so that algorithms other
// than full fan-out keep the whole round inside one graph.  `plan_i` = {mode}, `plan_f` = {a, b} (doubles),
// `templates` = 3 x D ints; the plan is per-request data in device memory, not a launch argument, so one captured
// graph serves every algorithm.
//   mode 0  caps[d] = templates[d]
//   mode 1  caps[d] = max(1, round_half_even(K * sigmoid(-a * ((lp[d][0] - lp[d][1]) - b))))
//   mode 2  g = mean over d of (lp[d][0] - lp[d][1]);  templates row 0 if g > a, row 1 if g < b, else row 2
// Arithmetic in double, summed in depth order: the same numbers the host evaluator produces.
__global__ void caps_from_topk_kernel(const float* topk_lp, int D, int K, const int* plan_i, const double* plan_f,
                                      const int* templates, int* caps) {
  pdl_launch_dependents();
  pdl_wait();
  const int mode = plan_i[0];
  const double a = plan_f[0], b = plan_f[1];
  if (mode == 1 && K >= 2) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const double gap = static_cast<double>(topk_lp[d * K]) - static_cast<double>(topk_lp[d * K + 1]);
      const double z = -a * (gap - b);
      const double s = z >= 0.0 ? 1.0 / (1.0 + exp(-z)) : exp(z) / (1.0 + exp(z));
      const int c = static_cast<int>(rint(static_cast<double>(K) * s));       // round half to even
      caps[d] = c < 1 ? 1 : c;
    }
    return;
  }
  int row = 0;
  if (mode == 2 && K >= 2) {
    double sum = 0.0;
    for (int d = 0; d < D; ++d) sum += static_cast<double>(topk_lp[d * K]) - static_cast<double>(topk_lp[d * K + 1]);
    const double g = sum / static_cast<double>(D);
    row = g > a ? 0 : (g < b ? 1 : 2);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) caps[d] = templates[row * D + d];
}

}  // namespace js

extern "C" int js_tree_ext_gate(const int* tokens, const int* parents, const int* state, const int* topk_tok,
                                const float* topk_lp, int D, int K, float gap_threshold, int ext, int NB, int* out,
                                int pdl, cudaStream_t stream) {
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(32);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tree_ext_gate_kernel, tokens, parents, state, topk_tok, topk_lp, D, K,
                            gap_threshold, ext, NB, out) == cudaSuccess ? 0 : -4;
}

extern "C" int js_tree_ext_splice(int* tokens, int* parents, int* depth, int* positions, int* mask_bits, int* state,
                                  const int* gate, const int* ext_tok, int ext, int NB, int W, int* status, int pdl,
                                  cudaStream_t stream) {
  if (ext < 1 || NB > js::kMaxNodes || W < 1 || W > js::kMaxWords) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(32);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tree_ext_splice_kernel, tokens, parents, depth, positions, mask_bits, state, gate,
                            ext_tok, ext, NB, W, status) == cudaSuccess ? 0 : -4;
}

extern "C" int js_caps_from_topk(const float* topk_lp, int D, int K, const int* plan_i, const double* plan_f,
                                 const int* templates, int* caps, int pdl, cudaStream_t stream) {
  if (D <= 0) return 0;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(64);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::caps_from_topk_kernel, topk_lp, D, K, plan_i, plan_f, templates, caps) == cudaSuccess ? 0 : -4;
}

extern "C" int js_tree_build(const int* topk_tok, const float* topk_lp, const int* caps, int D, int K, int budget,
                             int NB, int W, const int* committed, int* state, const int* slot_map,
                             const int* seq_row, int max_len, int* tokens, int* parents, int* depth, int* positions,
                             int* slots, int* mask_bits, int* status, int pdl, cudaStream_t stream) {
  if (NB < 1 || NB > js::kMaxNodes || W < 1 || W > js::kMaxWords || NB > W * 32) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tree_build_kernel, topk_tok, topk_lp, caps, D, K, budget, NB, W, committed, state,
                            slot_map, seq_row, max_len, tokens, parents, depth, positions, slots, mask_bits, status) == cudaSuccess ? 0 : -4;
}

extern "C" int js_tree_accept_commit(const int* tokens, const int* parents, const int* depth, const int* greedy,
                                     int NB, int* state, int* slot_map, const int* seq_row, int max_len,
                                     int* committed, int committed_cap, const int* eos_ids, int n_eos, int max_new,
                                     int* path_idx, int* result, int* status, int pdl, cudaStream_t stream) {
  if (NB < 1 || NB > js::kMaxNodes) return -10;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(256);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::tree_accept_commit_kernel, tokens, parents, depth, greedy, NB, state, slot_map,
                            seq_row, max_len, committed, committed_cap, eos_ids, n_eos, max_new, path_idx, result,
                            status) == cudaSuccess ? 0 : -4;
}

extern "C" int js_draft_prep_fill(int* state, const int* committed, int mask_token, int bs, int rows_pad,
                                  int ctx_rows_pad, int* block_ids, int* block_pos, int* ctx_pos, int* n_new_out,
                                  const int* fill, int fill_stride, int n_fill, int pdl, cudaStream_t stream);

extern "C" int js_draft_prep(int* state, const int* committed, int mask_token, int bs, int rows_pad, int ctx_rows_pad,
                             int* block_ids, int* block_pos, int* ctx_pos, int* n_new_out, int pdl,
                             cudaStream_t stream) {
  return js_draft_prep_fill(state, committed, mask_token, bs, rows_pad, ctx_rows_pad, block_ids, block_pos, ctx_pos,
                            n_new_out, nullptr, 0, 0, pdl, stream);
}

extern "C" int js_draft_prep_fill(int* state, const int* committed, int mask_token, int bs, int rows_pad,
                                  int ctx_rows_pad, int* block_ids, int* block_pos, int* ctx_pos, int* n_new_out,
                                  const int* fill, int fill_stride, int n_fill, int pdl, cudaStream_t stream) {
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(1);
  c.blockDim = dim3(64);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, js::draft_prep_kernel, state, committed, mask_token, bs, rows_pad, ctx_rows_pad,
                            block_ids, block_pos, ctx_pos, n_new_out, fill, fill_stride, n_fill) == cudaSuccess ? 0 : -4;
}
