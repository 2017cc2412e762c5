// Paged tree-masked attention (verify, prefill and decode share this kernel), head_dim 128.
//
// A sequence's keys are its logical positions 0 .. past+n-1; position p lives in KV slot
// slot_map[row][p] of a (Hkv, S, 128) pool, so the accepted-path commit never moves KV.
// Positions below `past` are visible to every query of the sequence; position past+j is
// visible to query node i when bit j of mask_bits[i] is set (tree) or j <= i (causal).
//
// One CTA = (q tile, kv head, key split).  The GQA group is packed into the row dimension:
// 64 rows = (64/G) nodes x G query heads, so K/V tiles are read once per group.  4 warps,
// each 16 rows; K/V tiles of 64 keys are gathered row by row with cp.async into swizzled
// shared memory (double buffered), S = QK^T and O += PV run on mma.sync m16n8k16 with fp32
// online softmax.  With more than one key split, partial (m, l, O) go to a workspace and a
// second kernel merges them.
//
// Counterpart of the reference's Triton kernel (jetspec/inference_engine/paged_tree_attn.py:54-272):
// ragged batch, binary search of the sequence, causal tile pruning, all-masked-row guard.
// The tree mask is packed bits (W words per query) instead of an fp32 (total_q, total_q) bias.
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int AD = 128;        // head dim
constexpr int AROWS = 64;      // query rows per CTA
constexpr int AKEYS = 64;      // keys per tile
constexpr int ATHREADS = 128;

struct AttnParams {
  const __nv_bfloat16* q;      // (T, Hq, 128)
  const __nv_bfloat16* k_pool; // (Hkv, S, 128)
  const __nv_bfloat16* v_pool;
  const int* slot_map;         // (max_seqs, max_len)
  const int* seq_rows;         // (B)
  const int* cu_q;             // (B+1)
  const int* past_lens;        // (B)
  const int* mask_bits;        // (T, W) or null when causal
  __nv_bfloat16* out;          // (T, Hq*128)
  float* ws_o;                 // (splits, T, Hq, 128) partial outputs
  float* ws_ml;                // (splits, T, Hq, 2)   partial (max, sum)
  int* status;
  int B, T, Hq, Hkv, S, max_len, W, causal, splits;
  float scale_log2;            // softmax scale * log2(e)
};

JS_DEVICE void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = smem_u32(smem);
  const int n = valid ? 16 : 0;   // src-size 0 -> zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
JS_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
JS_DEVICE void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

JS_DEVICE void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
JS_DEVICE void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
JS_DEVICE void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
JS_DEVICE uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk `c` (0..15) of row `r` in a [rows][128] bf16 tile, XOR-swizzled
JS_DEVICE uint32_t swz(int r, int c) { return static_cast<uint32_t>(r * 256 + ((c ^ (r & 7)) << 4)); }

template <int G>
__global__ void __launch_bounds__(ATHREADS, 2) paged_tree_attn_kernel(AttnParams p) {
  constexpr int NPT = AROWS / G;   // nodes per q tile
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;                       // 64 x 256 B
  uint8_t* sK = sQ + AROWS * 256;           // 2 x 64 x 256 B
  uint8_t* sV = sK + 2 * AKEYS * 256;       // 2 x 64 x 256 B
  int* sMask = reinterpret_cast<int*>(sV + 2 * AKEYS * 256);   // NPT x W

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, split = blockIdx.z;

  pdl_launch_dependents();
  pdl_wait();

  // ---- which sequence does this q tile belong to?  tiles are numbered so that sequence b
  // starts at tile cu_q[b]/NPT + b (an upper bound on the tiles of the sequences before it).
  int lo = 0, hi = p.B - 1;
  const int tile = blockIdx.x;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (p.cu_q[mid] / NPT + mid <= tile) lo = mid; else hi = mid - 1;
  }
  const int b = lo;
  const int q_begin = p.cu_q[b], n_b = p.cu_q[b + 1] - q_begin;
  const int node0 = (tile - (q_begin / NPT + b)) * NPT;
  if (node0 >= n_b) return;
  const int past = p.past_lens[b];
  const int row_sm = p.seq_rows[b];
  const int* slots = p.slot_map + static_cast<size_t>(row_sm) * p.max_len;
  int L = past + n_b;
  if (p.causal) L = min(L, past + node0 + NPT);   // later keys are invisible to this tile
  const int n_tiles = (L + AKEYS - 1) / AKEYS;
  const int t_begin = (n_tiles * split) / p.splits;
  const int t_end = (n_tiles * (split + 1)) / p.splits;

  // ---- stage Q (rows = node-major, group member minor) and the tile's mask words
  for (int c = tid; c < AROWS * 16; c += ATHREADS) {
    const int r = c >> 4, ch = c & 15;
    const int node = node0 + r / G, head = h * G + r % G;
    const bool valid = node < n_b;
    const __nv_bfloat16* src = p.q + (static_cast<size_t>(q_begin + (valid ? node : 0)) * p.Hq + head) * AD + ch * 8;
    cp_async16(sQ + swz(r, ch), src, valid);
  }
  if (!p.causal) {
    for (int c = tid; c < NPT * p.W; c += ATHREADS) {
      const int node = node0 + c / p.W;
      sMask[c] = node < n_b ? p.mask_bits[static_cast<size_t>(q_begin + node) * p.W + c % p.W] : 0;
    }
  }
  cp_async_commit();

  auto load_kv = [&](int t, int buf) {
    const int k0 = t * AKEYS;
    for (int c = tid; c < AKEYS * 16; c += ATHREADS) {
      const int r = c >> 4, ch = c & 15;
      const int kp = k0 + r;
      const bool valid = kp < L;
      int slot = valid ? __ldg(slots + kp) : 0;
      if (slot < 0 || slot >= p.S) { report(p.status, kBadSlot); slot = 0; }
      const size_t off = (static_cast<size_t>(h) * p.S + slot) * AD + ch * 8;
      cp_async16(sK + buf * AKEYS * 256 + swz(r, ch), p.k_pool + off, valid);
      cp_async16(sV + buf * AKEYS * 256 + swz(r, ch), p.v_pool + off, valid);
    }
    cp_async_commit();
  };

  if (t_begin < t_end) load_kv(t_begin, 0);
  cp_async_wait<0>();   // (Q and the first tile; the loop below re-syncs per tile)
  __syncthreads();

  // ---- Q fragments: 8 k-steps x 4 regs
  uint32_t qf[8][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int ch = ks * 2 + (lane >> 4);
      ldsm_x4(smem_u32(sQ + swz(r, ch)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int r_lo = warp * 16 + (lane >> 2);       // this thread's two rows within the tile
  const int node_lo = r_lo / G, node_hi = (r_lo + 8) / G;   // tile-local node of each row

  for (int t = t_begin; t < t_end; ++t) {
    const int buf = (t - t_begin) & 1;
    if (t + 1 < t_end) load_kv(t + 1, buf ^ 1);
    if (t + 1 < t_end) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const uint8_t* kT = sK + buf * AKEYS * 256;
    const uint8_t* vT = sV + buf * AKEYS * 256;

    // S = Q K^T  (16 rows x 64 keys per warp)
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {   // pairs of 8-key n-tiles
        const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int ch = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(kT + swz(key, ch)), b0, b1, b2, b3);
        mma_bf16(s[np * 2], qf[ks], b0, b1);
        mma_bf16(s[np * 2 + 1], qf[ks], b2, b3);
      }
    }

    // mask + online softmax
    const int k0 = t * AKEYS;
    const bool window = (k0 + AKEYS > past);   // tile touches the tree / causal window
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kp = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const int nl = (e < 2) ? node_lo : node_hi;
        bool vis = kp < L && (node0 + nl) < n_b;
        if (vis && window && kp >= past) {
          const int j = kp - past;
          vis = p.causal ? (j <= node0 + nl) : ((sMask[nl * p.W + (j >> 5)] >> (j & 31)) & 1);
        }
        const float x = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    }
    // The running maximum is kept as an INTEGER (in the log2 domain).  Probabilities are then
    // 2^(s - m) with m integral, so choosing a different m (another tile order, another key
    // split) only moves them by an exact power of two: the bf16 rounding of P and every
    // rescale are bit-identical whatever the KV layout.  A node's attention output therefore
    // does not depend, beyond fp32 summation order, on where its ancestors sit in the window.
    float alpha[2], m_new[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      m_new[i] = fmaxf(m_run[i], ceilf(mx[i]));
      const float m_safe = (m_new[i] == -INFINITY) ? 0.f : m_new[i];   // all-masked row guard
      alpha[i] = exp2f(m_run[i] - m_safe);
      m_run[i] = m_new[i];
      m_new[i] = m_safe;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4][4];   // P as A fragments for the 4 k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - m_new[0]), p1 = exp2f(s[nt][1] - m_new[0]);
      const float p2 = exp2f(s[nt][2] - m_new[1]), p3 = exp2f(s[nt][3] - m_new[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      const int ks = nt >> 1, half = nt & 1;
      pf[ks][half * 2] = pack_bf16(p0, p1);
      pf[ks][half * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + rs[i];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }

    // O += P V  (k = keys, n = head dim)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int np = 0; np < 8; ++np) {   // pairs of 8-wide d tiles
        const int key = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int ch = np * 2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(vT + swz(key, ch)), b0, b1, b2, b3);
        mma_bf16(o[np * 2], pf[ks], b0, b1);
        mma_bf16(o[np * 2 + 1], pf[ks], b2, b3);
      }
    }
    __syncthreads();   // everyone is done with `buf` before the next prefetch overwrites it
  }

  // ---- finish: row sums across the 4 lanes of a quad
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r_lo + half * 8;
    const int node = node0 + r / G, head = h * G + r % G;
    if (node >= n_b) continue;
    const size_t row = static_cast<size_t>(q_begin + node) * p.Hq + head;
    if (p.splits == 1) {
      const float inv = l_run[half] > 0.f ? 1.f / l_run[half] : 0.f;
      __nv_bfloat16* dst = p.out + row * AD;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
      }
    } else {
      float* dst = p.ws_o + (static_cast<size_t>(split) * p.T * p.Hq + row) * AD;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const int d = nt * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(dst + d) = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
      }
      if ((lane & 3) == 0) {
        float* ml = p.ws_ml + (static_cast<size_t>(split) * p.T * p.Hq + row) * 2;
        ml[0] = m_run[half];
        ml[1] = l_run[half];
      }
    }
  }
}

// merge key splits: one warp per (token, head)
__global__ void attn_merge_kernel(AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= p.T * p.Hq) return;
  const size_t stride = static_cast<size_t>(p.T) * p.Hq;
  float m = -INFINITY;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, p.ws_ml[(s * stride + row) * 2]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = p.ws_ml[(s * stride + row) * 2], ls = p.ws_ml[(s * stride + row) * 2 + 1];
    if (ms == -INFINITY) continue;   // this split saw no visible key (its O may be unwritten)
    const float w = exp2f(ms - m);
    l += ls * w;
    const float4 v = *reinterpret_cast<const float4*>(p.ws_o + (s * stride + row) * AD + lane * 4);
    acc[0] += v.x * w; acc[1] += v.y * w; acc[2] += v.z * w; acc[3] += v.w * w;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * AD + lane * 4;
  *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
}

template <int G>
static int launch_attn(const AttnParams& p, int q_tiles, bool pdl, cudaStream_t stream) {
  constexpr int NPT = AROWS / G;
  const int smem = AROWS * 256 + 4 * AKEYS * 256 + NPT * p.W * 4 + 16;
  static int configured[kMaxDevicesCached] = {};
  auto kern = paged_tree_attn_kernel<G>;
  if (ensure_dyn_smem(kern, 100 * 1024, configured) != 0) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(q_tiles, p.Hkv, p.splits);
  cfg.blockDim = dim3(ATHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return -4;
  if (p.splits > 1) {
    cudaLaunchConfig_t c2 = {};
    c2.gridDim = dim3((p.T * p.Hq + 7) / 8);
    c2.blockDim = dim3(256);
    c2.stream = stream;
    c2.attrs = attr;
    c2.numAttrs = pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&c2, attn_merge_kernel, p) != cudaSuccess) return -5;
  }
  return 0;
}

}  // namespace js

// q (T,Hq,128) bf16; pools (Hkv,S,128); out (T,Hq*128).  max_q = largest per-sequence query count
// (bounds the grid); splits = key splits (workspace needed when > 1).  Returns 0 or a negative code.
extern "C" int js_paged_tree_attention(const void* q, const void* k_pool, const void* v_pool, const int* slot_map,
                                       const int* seq_rows, const int* cu_q, const int* past_lens, const int* mask_bits,
                                       void* out, float* ws_o, float* ws_ml, int* status, int B, int T, int Hq, int Hkv,
                                       int S, int max_len, int W, int causal, int splits, float scale, int pdl,
                                       cudaStream_t stream) {
  using namespace js;
  if (T <= 0 || B <= 0) return 0;
  if (Hq % Hkv) return -10;
  const int G = Hq / Hkv;
  if (splits < 1) return -11;
  if (splits > 1 && (ws_o == nullptr || ws_ml == nullptr)) return -12;
  if (!causal && (mask_bits == nullptr || W < 1 || W > 64)) return -13;
  AttnParams p{reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k_pool),
               reinterpret_cast<const __nv_bfloat16*>(v_pool), slot_map, seq_rows, cu_q, past_lens, mask_bits,
               reinterpret_cast<__nv_bfloat16*>(out), ws_o, ws_ml, status, B, T, Hq, Hkv, S, max_len, W, causal,
               splits, scale * 1.4426950408889634f};
  switch (G) {
    case 1: return launch_attn<1>(p, T + B, pdl != 0, stream);
    case 2: return launch_attn<2>(p, (T + 31) / 32 + B, pdl != 0, stream);
    case 4: return launch_attn<4>(p, (T + 15) / 16 + B, pdl != 0, stream);
    case 8: return launch_attn<8>(p, (T + 7) / 8 + B, pdl != 0, stream);
    case 16: return launch_attn<16>(p, (T + 3) / 4 + B, pdl != 0, stream);
    default: return -14;
  }
}

// Merge the key splits of a (splits, T, Hq, 128) fp32 workspace with its (max, sum) pairs into out (T, Hq*128).
extern "C" int js_attn_merge(float* ws_o, float* ws_ml, void* out, int T, int Hq, int splits, int pdl, cudaStream_t stream) {
  using namespace js;
  AttnParams p{};
  p.ws_o = ws_o; p.ws_ml = ws_ml; p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.T = T; p.Hq = Hq; p.splits = splits;
  cudaLaunchConfig_t c2 = {};
  c2.gridDim = dim3((T * Hq + 7) / 8);
  c2.blockDim = dim3(256);
  c2.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  c2.attrs = attr;
  c2.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c2, attn_merge_kernel, p) == cudaSuccess ? 0 : -5;
}
