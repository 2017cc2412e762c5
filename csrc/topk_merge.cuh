// Row-wise merge of the per-tile top-8 + (max, sum-exp) partials that the vocabulary GEMM's top-k epilogue emits.
// Shared by the single-GPU merge kernel and the vocabulary-parallel (tensor-parallel) combine.
#pragma once

#include "common.cuh"

#include <math.h>

namespace js {

// larger value first; among equal values the lower token id
JS_DEVICE bool cand_better(float v1, int i1, float v2, int i2) { return v1 > v2 || (v1 == v2 && i1 < i2); }

JS_DEVICE void topk_block_finish(float (&lv)[8], int (&li)[8], float mx, float se, int K, float* win_v, int* win_i,
                                 float* row_m, float* row_s);

// sorted insertion of one candidate into a private top-8 (larger value first, lower id first among equals)
JS_DEVICE void topk_insert(float (&lv)[8], int (&li)[8], float v, int ix) {
  if (!cand_better(v, ix, lv[7], li[7])) return;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (cand_better(v, ix, lv[q], li[q])) {
      const float fv = lv[q];
      const int fi = li[q];
      lv[q] = v; li[q] = ix;
      v = fv; ix = fi;
    }
  }
}

// Called by all 256 threads of a block for one row.  Each thread folds the sorted 8-entry lists of its tiles
// into a private sorted top-8 (registers, one pass over global memory, coalesced 32-byte reads), then K
// block-wide argmax rounds over the threads' list heads pick the row's top-K.  Vocabulary tiles are disjoint,
// so a token id appears in one list only and the winner of a round is identified by its id.
// Results: win_v[k], win_i[k] (shared memory, k < K) and the row's running (max, sum of exp) in *row_m, *row_s;
// valid for every thread after the function returns (it ends with a block barrier).
JS_DEVICE void topk_merge_row(const float* part_val, const int* part_idx, const float* part_lse, int n_tiles, int row,
                              int K, float* win_v, int* win_i, float* row_m, float* row_s) {
  const int tid = threadIdx.x;
  float lv[8];
  int li[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { lv[e] = -INFINITY; li[e] = 0x7fffffff; }
  float mx = -INFINITY, se = 0.f;
  for (int t = tid; t < n_tiles; t += blockDim.x) {
    const size_t o = static_cast<size_t>(row) * n_tiles + t;
    const float2 ms = *reinterpret_cast<const float2*>(part_lse + o * 2);
    if (ms.x != -INFINITY) {
      if (ms.x > mx) { se = se * __expf(mx - ms.x) + ms.y; mx = ms.x; } else { se += ms.y * __expf(ms.x - mx); }
    }
    const float4 va = *reinterpret_cast<const float4*>(part_val + o * 8);
    const float4 vb = *reinterpret_cast<const float4*>(part_val + o * 8 + 4);
    const int4 ia = *reinterpret_cast<const int4*>(part_idx + o * 8);
    const int4 ib = *reinterpret_cast<const int4*>(part_idx + o * 8 + 4);
    const float tv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
    const int ti[8] = {ia.x, ia.y, ia.z, ia.w, ib.x, ib.y, ib.z, ib.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = tv[e];
      int ix = ti[e];
      if (v < lv[7]) break;                                // the tile's list is sorted: nothing further can enter
      if (!cand_better(v, ix, lv[7], li[7])) continue;
#pragma unroll
      for (int q = 0; q < 8; ++q) {                        // insert, pushing the displaced entry down
        if (cand_better(v, ix, lv[q], li[q])) {
          const float fv = lv[q];
          const int fi = li[q];
          lv[q] = v; li[q] = ix;
          v = fv; ix = fi;
        }
      }
    }
  }
  topk_block_finish(lv, li, mx, se, K, win_v, win_i, row_m, row_s);
}

// Second half of the row merge, shared with the kernel that scans raw logits: every thread of the 256-thread block
// brings a private sorted top-8 (lv, li) and a running (max, sum of exp); the block's (max, sum) goes to *row_m,
// *row_s and K block-wide argmax rounds over the threads' list heads fill win_v / win_i.  Ends with a block barrier.
JS_DEVICE void topk_block_finish(float (&lv)[8], int (&li)[8], float mx, float se, int K, float* win_v, int* win_i,
                                 float* row_m, float* row_s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = 8;
  __shared__ float s_m[kWarps], s_s[kWarps];
  __shared__ float s_v[2][kWarps];
  __shared__ int s_i[2][kWarps];
  // log-sum-exp of the row: warp shuffle, then the 8 warp results
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, mx, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, se, o);
    const float m = fmaxf(mx, m2);
    if (m != -INFINITY) { se = se * __expf(mx - m) + s2 * __expf(m2 - m); mx = m; }
  }
  if (lane == 0) { s_m[warp] = mx; s_s[warp] = se; }
  __syncthreads();
  float gm = -INFINITY, gs = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const float m2 = s_m[w], s2 = s_s[w];
    const float m = fmaxf(gm, m2);
    if (m != -INFINITY) { gs = gs * __expf(gm - m) + s2 * __expf(m2 - m); gm = m; }
  }
  if (tid == 0) { *row_m = gm; *row_s = gs; }
  for (int k = 0; k < K && k < 8; ++k) {
    float bv = lv[0];
    int bi = li[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int buf = k & 1;
    if (lane == 0) { s_v[buf][warp] = bv; s_i[buf][warp] = bi; }
    __syncthreads();
    bv = s_v[buf][0];
    bi = s_i[buf][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w)
      if (cand_better(s_v[buf][w], s_i[buf][w], bv, bi)) { bv = s_v[buf][w]; bi = s_i[buf][w]; }
    if (li[0] == bi && lv[0] == bv && bi != 0x7fffffff) {     // this thread's head won: pop it
#pragma unroll
      for (int q = 0; q < 7; ++q) { lv[q] = lv[q + 1]; li[q] = li[q + 1]; }
      lv[7] = -INFINITY; li[7] = 0x7fffffff;
    }
    if (tid == 0) { win_v[k] = bv; win_i[k] = bi; }
  }
  __syncthreads();
}

}  // namespace js
