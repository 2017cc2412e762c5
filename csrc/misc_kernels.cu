// Memory-bound helper kernels of the decode round: embedding gather, RMSNorm, the fused
// Reference twins: the ATen ops between the GEMMs of jetspec/inference_engine/compiled_verify_stack.py:170-272 (norms, RoPE,
// KV write) and the drafter's log_softmax + topk, jetspec/tree/_core/topk_build.py:10-63 / jetspec/draft_head_adapter.py:129.
// QKV post-processing (per-head RMSNorm + RoPE + KV scatter into slots), SwiGLU, row
// gathers, and the merges of the per-tile argmax / top-k partials the LM-head GEMM emits.
// All math is fp32; tensors are bf16.  Each kernel joins programmatic dependent launch:
// it lets its successor start early and waits for its predecessor before reading.
#include "common.cuh"
#include "topk_merge.cuh"

#include <math.h>

namespace js {

JS_DEVICE void bf16x8_to_float(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
JS_DEVICE uint4 float_to_bf16x8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// out[t, :] = table[ids[t], :]     (H % 8 == 0)
__global__ void embed_kernel(const int* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= T) return;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// y = x * rsqrt(mean(x^2) + eps) * w ; one CTA per row
__global__ void rmsnorm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, int T, int H,
                               int ldx, int ldy, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float f[8];
    bf16x8_to_float(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / H + eps);
  }
  __syncthreads();
  const float inv = red[0];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * ldy);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float f[8], g[8];
    bf16x8_to_float(xr[i], f);
    bf16x8_to_float(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * inv * g[j];
    yr[i] = float_to_bf16x8(f);
  }
}

// Fused QKV post-processing, head_dim 128.  One warp per (token, head) of the fused row
// [q heads | k heads | v heads]: q and k heads get RMSNorm over the head then rotate-half RoPE
// at positions[t]; q goes to q_out (T, Hq, 128), k and v go to the pools (Hkv, S, 128) at
// slots[t].  norm weights may be null (no per-head norm).  q_out may be null (context rows of
// the draft head only produce K/V).
__global__ void qkv_post_kernel(const __nv_bfloat16* qkv, int ld, const __nv_bfloat16* qw, const __nv_bfloat16* kw,
                                const int* positions, const int* slots, const float* inv_freq,
                                __nv_bfloat16* q_out, __nv_bfloat16* k_pool, __nv_bfloat16* v_pool, int T, int Hq,
                                int Hkv, int S, float eps, const int* n_valid, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int heads = Hq + 2 * Hkv;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= T * heads) return;
  const int t = gw / heads, hd = gw % heads;
  if (n_valid != nullptr && t >= *n_valid) return;
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * ld + hd * 128;
  // lane holds elements (2*lane, 2*lane+1) of each half: x1 = [0,64), x2 = [64,128)
  float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2 * lane));
  float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 64 + 2 * lane));
  const bool is_q = hd < Hq, is_k = !is_q && hd < Hq + Hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? qw : kw;
    if (nw != nullptr) {
      float ss = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
      const float inv = rsqrtf(ss / 128.f + eps);
      const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + 2 * lane));
      const float2 w2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + 64 + 2 * lane));
      // round to bf16 after the norm, as an unfused norm kernel would
      a.x = __bfloat162float(__float2bfloat16_rn(a.x * inv * w1.x));
      a.y = __bfloat162float(__float2bfloat16_rn(a.y * inv * w1.y));
      b.x = __bfloat162float(__float2bfloat16_rn(b.x * inv * w2.x));
      b.y = __bfloat162float(__float2bfloat16_rn(b.y * inv * w2.y));
    }
    const float pos = static_cast<float>(positions[t]);
    float s0, c0, s1, c1;
    sincosf(pos * inv_freq[2 * lane], &s0, &c0);
    sincosf(pos * inv_freq[2 * lane + 1], &s1, &c1);
    const float2 ra = make_float2(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
    const float2 rb = make_float2(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    a = ra;
    b = rb;
  }
  __nv_bfloat16* dst;
  if (is_q) {
    if (q_out == nullptr) return;
    dst = q_out + (static_cast<size_t>(t) * Hq + hd) * 128;
  } else {
    int slot = slots[t];
    if (slot < 0 || slot >= S) {
      if (lane == 0) report(status, kBadSlot);
      return;
    }
    const int kvh = is_k ? hd - Hq : hd - Hq - Hkv;
    dst = (is_k ? k_pool : v_pool) + (static_cast<size_t>(kvh) * S + slot) * 128;
  }
  *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(a.x, a.y);
  *reinterpret_cast<__nv_bfloat162*>(dst + 64 + 2 * lane) = __floats2bfloat162_rn(b.x, b.y);
}

// out[t, j] = silu(in[t, j]) * in[t, I + j]
__global__ void silu_mul_kernel(const __nv_bfloat16* in, __nv_bfloat16* out, int T, int I) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = static_cast<size_t>(T) * I / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / (I / 8), c = i % (I / 8);
    float g[8], u[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(in + t * 2 * I + c * 8), g);
    bf16x8_to_float(*reinterpret_cast<const uint4*>(in + t * 2 * I + I + c * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(out + t * I + c * 8) = float_to_bf16x8(g);
  }
}

// dst[i, dst_col0 : dst_col0 + H] = src[idx ? idx[i] : i, :]   (row gather / column-block copy)
__global__ void gather_rows_kernel(const __nv_bfloat16* src, int lds, const int* idx, const int* n_valid,
                                   __nv_bfloat16* dst, int ldd, int dst_col0, int rows, int H, int src_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= rows) return;
  int r = idx != nullptr ? idx[i] : i;
  const bool valid = (n_valid == nullptr || i < *n_valid) && r >= 0 && r < src_rows;
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<size_t>(valid ? r : 0) * lds);
  uint4* d = reinterpret_cast<uint4*>(dst + static_cast<size_t>(i) * ldd + dst_col0);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) d[c] = valid ? s[c] : zero;
}

// argmax over the per-tile partials of the LM-head GEMM: one warp per row; lowest index wins ties
__global__ void argmax_merge_kernel(const float* part_val, const int* part_idx, int n_tiles, int M, int* out_idx,
                                    float* out_val) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lane; i < n_tiles; i += 32) {
    const float v = part_val[static_cast<size_t>(row) * n_tiles + i];
    const int ix = part_idx[static_cast<size_t>(row) * n_tiles + i];
    if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) {
    out_idx[row] = bi;
    if (out_val != nullptr) out_val[row] = best;
  }
}

// Merge per-tile top-8 and (max, sum-exp) partials into per-row top-K tokens and full-vocabulary
// log-probabilities.  One block per row (see topk_merge.cuh).
__global__ void __launch_bounds__(256)
topk_merge_kernel(const float* part_val, const int* part_idx, const float* part_lse, int n_tiles,
                  int M, int K, int* out_tok, float* out_lp) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= M) return;
  __shared__ float win_v[8];
  __shared__ int win_i[8];
  __shared__ float row_m, row_s;
  topk_merge_row(part_val, part_idx, part_lse, n_tiles, row, K, win_v, win_i, &row_m, &row_s);
  if (threadIdx.x < K && threadIdx.x < 8) {
    const float lse = row_m + logf(row_s);
    out_tok[row * K + threadIdx.x] = win_i[threadIdx.x];
    out_lp[row * K + threadIdx.x] = win_v[threadIdx.x] - lse;
  }
}

// First pass of a two-pass top-k over materialised fp32 logits (the few-rows vocabulary pass of a draft block: the
// GEMM stores its logits with the plain fp32 epilogue, which streams the weights at the argmax epilogue's rate).
// Block (slice, row) scans columns [slice * slice_cols, ...) of one row and emits that slice's sorted top-8 and
// (max, sum of exp) in the layout of the GEMM's per-tile partials, so topk_merge_kernel finishes the row.
__global__ void __launch_bounds__(256)
logits_topk_slice_kernel(const float* logits, long long ld, int N, int M, int slice_cols, float* part_val, int* part_idx,
                         float* part_lse) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y, sl = blockIdx.x, n_slices = gridDim.x;
  if (row >= M) return;
  __shared__ float win_v[8];
  __shared__ int win_i[8];
  __shared__ float row_m, row_s;
  const int c0 = sl * slice_cols, c1 = min(N, c0 + slice_cols);
  float lv[8];
  int li[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { lv[e] = -INFINITY; li[e] = 0x7fffffff; }
  float mx = -INFINITY, se = 0.f;
  const float* src = logits + static_cast<size_t>(row) * ld;
  for (int c = c0 + 4 * static_cast<int>(threadIdx.x); c < c1; c += 4 * 256) {     // N, slice_cols, ld: multiples of 4
    const float4 q = *reinterpret_cast<const float4*>(src + c);
    const float v[4] = {q.x, q.y, q.z, q.w};
    const float cm = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    if (cm != -INFINITY) {
      const float nm = fmaxf(mx, cm);
      se = (mx == -INFINITY ? 0.f : se * __expf(mx - nm)) + __expf(v[0] - nm) + __expf(v[1] - nm) + __expf(v[2] - nm) +
           __expf(v[3] - nm);
      mx = nm;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) topk_insert(lv, li, v[j], c + j);
  }
  topk_block_finish(lv, li, mx, se, 8, win_v, win_i, &row_m, &row_s);
  const size_t o = static_cast<size_t>(row) * n_slices + sl;
  if (threadIdx.x < 8) {
    part_val[o * 8 + threadIdx.x] = win_v[threadIdx.x];
    part_idx[o * 8 + threadIdx.x] = win_i[threadIdx.x];
  }
  if (threadIdx.x == 0) {
    part_lse[o * 2] = row_m;
    part_lse[o * 2 + 1] = row_s;
  }
}

static cudaLaunchAttribute g_pdl_attr;
static void launch_cfg(cudaLaunchConfig_t& c, dim3 grid, dim3 block, cudaStream_t stream, int pdl) {
  c = cudaLaunchConfig_t{};
  c.gridDim = grid;
  c.blockDim = block;
  c.stream = stream;
  g_pdl_attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  g_pdl_attr.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &g_pdl_attr;
  c.numAttrs = pdl ? 1 : 0;
}

}  // namespace js

#define JS_LAUNCH(kern, grid, block, ...)                                             \
  do {                                                                                \
    cudaLaunchConfig_t c;                                                             \
    js::launch_cfg(c, grid, block, stream, pdl);                                      \
    return cudaLaunchKernelEx(&c, kern, __VA_ARGS__) == cudaSuccess ? 0 : -4;         \
  } while (0)

extern "C" int js_embed(const int* ids, const void* table, void* out, int T, int H, int V, int pdl, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  JS_LAUNCH(js::embed_kernel, dim3(T), dim3(128), ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V);
}

extern "C" int js_rmsnorm(const void* x, const void* w, void* y, int T, int H, int ldx, int ldy, float eps, int pdl,
                          cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H % 8) || (ldx % 8) || (ldy % 8)) return -10;
  const int threads = H >= 2048 ? 256 : 128;
  JS_LAUNCH(js::rmsnorm_kernel, dim3(T), dim3(threads), (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
            (__nv_bfloat16*)y, T, H, ldx, ldy, eps);
}

extern "C" int js_qkv_post(const void* qkv, int ld, const void* qw, const void* kw, const int* positions,
                           const int* slots, const float* inv_freq, void* q_out, void* k_pool, void* v_pool, int T,
                           int Hq, int Hkv, int S, float eps, const int* n_valid, int* status, int pdl,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  const int warps = T * (Hq + 2 * Hkv);
  JS_LAUNCH(js::qkv_post_kernel, dim3((warps + 7) / 8), dim3(256), (const __nv_bfloat16*)qkv, ld,
            (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, positions, slots, inv_freq, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, T, Hq, Hkv, S, eps, n_valid, status);
}

extern "C" int js_silu_mul(const void* in, void* out, int T, int I, int pdl, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 8) return -10;
  const size_t n = static_cast<size_t>(T) * I / 8;
  const int blocks = static_cast<int>((n + 255) / 256 > 1184 ? 1184 : (n + 255) / 256);
  JS_LAUNCH(js::silu_mul_kernel, dim3(blocks), dim3(256), (const __nv_bfloat16*)in, (__nv_bfloat16*)out, T, I);
}

extern "C" int js_gather_rows(const void* src, int lds, const int* idx, const int* n_valid, void* dst, int ldd,
                              int dst_col0, int rows, int H, int src_rows, int pdl, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((H % 8) || (lds % 8) || (ldd % 8) || (dst_col0 % 8)) return -10;
  JS_LAUNCH(js::gather_rows_kernel, dim3(rows), dim3(128), (const __nv_bfloat16*)src, lds, idx, n_valid,
            (__nv_bfloat16*)dst, ldd, dst_col0, rows, H, src_rows);
}

extern "C" int js_argmax_merge(const float* part_val, const int* part_idx, int n_tiles, int M, int* out_idx,
                               float* out_val, int pdl, cudaStream_t stream) {
  if (M <= 0) return 0;
  JS_LAUNCH(js::argmax_merge_kernel, dim3((M + 7) / 8), dim3(256), part_val, part_idx, n_tiles, M, out_idx, out_val);
}

// Slice partials of materialised logits (M, N) fp32 with leading dimension ld: part_val / part_idx (M, n_slices, 8),
// part_lse (M, n_slices, 2); finish with js_topk_merge(..., n_tiles = n_slices, ...).
extern "C" int js_logits_topk_slices(const float* logits, long long ld, int M, int N, int n_slices, float* part_val,
                                     int* part_idx, float* part_lse, int pdl, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (n_slices < 1 || (N % 4) || (ld % 4) || (reinterpret_cast<uintptr_t>(logits) & 15)) return -10;
  const int slice_cols = (((N + n_slices - 1) / n_slices) + 3) / 4 * 4;
  JS_LAUNCH(js::logits_topk_slice_kernel, dim3(n_slices, M), dim3(256), logits, ld, N, M, slice_cols, part_val, part_idx,
            part_lse);
}

extern "C" int js_topk_merge(const float* part_val, const int* part_idx, const float* part_lse, int n_tiles, int M,
                             int K, int* out_tok, float* out_lp, int pdl, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K < 1 || K > 8) return -10;
  JS_LAUNCH(js::topk_merge_kernel, dim3(M), dim3(256), part_val, part_idx, part_lse, n_tiles, M, K, out_tok, out_lp);
}
