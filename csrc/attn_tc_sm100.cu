// Paged tree-masked attention on the 5th-generation tensor cores (tcgen05 + tensor memory), head_dim 128.
// Reference twins: the Triton paged kernel jetspec/inference_engine/paged_tree_attn.py:55-367 (fp32 qq_bias, block tables)
// and the dense tree-attention kernel of the Hugging Face path, jetspec/core/tree_attention_kernel.py:63-216.
//
// Same contract as the mma.sync kernel in attn_sm100.cu (logical positions through a slot map, packed
// ancestor bits or causal window, GQA group packed into rows, optional key splits merged by
// attn_merge_kernel), different engine:
//
//   * one CTA = 128 query rows (128/G tree nodes x G query heads of one KV head) x one key split;
//   * S = Q K^T and O += P V are tcgen05.mma with M = 128; S (2 x 64 columns) and O (128 columns)
//     live in tensor memory, so the softmax threads own one ROW each (no shuffles): they read S with
//     tcgen05.ld, write P as bf16 into a swizzled shared-memory tile that feeds the second MMA, and
//     rescale O in tensor memory only when a row's integer running maximum grows;
//   * K/V rows are gathered by slot with cp.async into 128-byte-swizzled tiles (three stages) by four
//     loader warps; V is consumed as an MN-major operand, so no transpose is ever made;
//   * warp 4 issues all MMAs: QK(t+1) is issued before PV(t), so the tensor pipe works on the next
//     scores while the softmax of the current tile runs.
//
// Roles (416 threads): warps 0-3 softmax + epilogue (tensor-memory lane quadrant = warp id),
// warp 4 MMA issuer / TMEM owner, warps 5-12 loaders.  Every wait is bounded (status word).
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int TD = 128;          // head dim
constexpr int TROWS = 128;       // query rows per CTA
constexpr int TKEYS = 64;        // keys per tile
constexpr int TSTAGES = 3;
constexpr int TLOADERS = 256;       // loader threads (gather throughput grows with the copies in flight)
constexpr int TTHREADS = 160 + TLOADERS;
constexpr int kStageKV = 2 * TKEYS * 256;      // K then V, each 2 halves x 64 keys x 128 B
constexpr int kSmemQ = TROWS * 256;            // 2 halves x 128 rows x 128 B
constexpr int kSmemP = TROWS * 128;            // 128 rows x 64 keys bf16
constexpr int kAttnTcSmem = kSmemQ + TSTAGES * kStageKV + 2 * kSmemP + 256 + 1024;
// Key splits that merge inside a cluster (portable cluster size); the chunk receive area must fit the dead
// K/V stages + P buffers, the (max, sum) pairs the dead Q tile.
constexpr int kMaxClusterSplits = 8;
static_assert(kMaxClusterSplits * 16384 <= TSTAGES * kStageKV + 2 * kSmemP, "chunk receive area");
static_assert(3 * 2 * 16384 <= TSTAGES * kStageKV + 2 * kSmemP, "chunk receive area, 3 splits own 2 chunks each");
static_assert(kMaxClusterSplits * TROWS * 8 <= kSmemQ, "(max, sum) receive area");

struct AttnTcParams {
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
  float scale_log2;
  int cluster_merge;           // the key splits of a tile form a cluster and merge through distributed shared memory
};

JS_DEVICE void cp_async16_tc(uint32_t smem_addr, const void* gmem, bool valid) {
  const int n = valid ? 16 : 0;   // src-size 0 -> zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gmem), "r"(n) : "memory");
}
JS_DEVICE void cp_async_commit_tc() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
JS_DEVICE void cp_async_wait_tc() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

JS_DEVICE void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// Bounded wait that backs off between polls: the waiting roles share the SM's load/store path with the
// loaders' cp.async traffic, so they must not spin on it.
JS_DEVICE bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, int* status, int code) {
  for (uint32_t i = 0; i < (kSpinLimit >> 2); ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    __nanosleep(20);
  }
  report(status, code);
  return false;
}
JS_DEVICE float fast_exp2(float x) {     // 2^x, flushing denormal results to zero; exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
JS_DEVICE void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand tile stored as two 64-element halves of 128-byte rows (8-row groups 1024 B apart,
// halves `half_stride` bytes apart), 128-byte swizzle.
JS_DEVICE uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t half_stride) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(half_stride >> 4) << 16;      // leading byte offset: next 64 elements along MN
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset: next 8 rows along K
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
JS_DEVICE constexpr uint32_t umma_idesc_bf16_bmn(int M, int N) {   // B operand MN-major
  return umma_idesc_bf16(M, N) | (1u << 16);
}

// Optional phase trace (nanosecond timestamps written by CTA (0,0,0)); null unless a profiling script sets it.
__device__ unsigned long long* g_attn_trace = nullptr;
JS_DEVICE void attn_trace(int slot) {
  if (g_attn_trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_attn_trace[slot] = t;
  }
}

template <int G>
__global__ void __launch_bounds__(TTHREADS, 1) paged_tree_attn_tc_kernel(AttnTcParams p) {
  constexpr int NPT = TROWS / G;   // nodes per q tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + kSmemQ;
  uint8_t* sP = sKV + TSTAGES * kStageKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kSmemP);
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // TSTAGES
  uint64_t* kv_empty = kv_full + TSTAGES;  // TSTAGES
  uint64_t* s_full = kv_empty + TSTAGES;   // 2
  uint64_t* p_full = s_full + 2;           // 2
  uint64_t* pv_done = p_full + 2;          // 2
  uint64_t* o_done = pv_done + 2;          // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, split = blockIdx.z;

  pdl_launch_dependents();
  pdl_wait();
  if (tid == 0) attn_trace(0);

  // ---- which sequence does this q tile belong to (same numbering as the mma.sync kernel)
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
  const int* slots = p.slot_map + static_cast<size_t>(p.seq_rows[b]) * p.max_len;
  int L = past + n_b;
  if (p.causal) L = min(L, past + node0 + NPT);
  const int n_tiles = (L + TKEYS - 1) / TKEYS;
  const int t_begin = (n_tiles * split) / p.splits;
  const int t_end = (n_tiles * (split + 1)) / p.splits;
  const int nt = t_end - t_begin;

  // softmax thread's row
  const int row = (warp & 3) * 32 + lane;
  const int node = node0 + row / G, head = h * G + row % G;
  const bool row_valid = node < n_b;
  const size_t out_row = static_cast<size_t>(q_begin + (row_valid ? node : 0)) * p.Hq + head;

  const bool cmerge = p.cluster_merge != 0;
  float m_run = -INFINITY, l_run = 0.f;     // softmax threads: running (integer) maximum and sum of their row
  bool sm_ok = true;
  if (nt <= 0 && !cmerge) {   // more splits than key tiles: this split contributes nothing
    if (warp < 4 && row_valid && p.splits > 1) {
      float* ml = p.ws_ml + (static_cast<size_t>(split) * p.T * p.Hq + out_row) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    return;
  }

  if (tid == 0 && nt > 0) {
    mbar_init(q_full, TLOADERS);
    for (int s = 0; s < TSTAGES; ++s) { mbar_init(&kv_full[s], TLOADERS); mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128); mbar_init(&pv_done[i], 1); }
    mbar_init(o_done, 1);
    fence_barrier_init();
  }
  if (warp == 4 && nt > 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = nt > 0 ? *tmem_slot : 0u;
  if (tid == 0) attn_trace(1);      // setup done
  const uint32_t tmem_o = tmem_base + 128;      // S buffers at columns [0,64) and [64,128)

  const uint32_t t_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
  if (nt <= 0) {
    // (cluster merge) nothing to compute: this CTA only takes part in the exchange below
  } else if (warp >= 5) {
    // ================================================================ loaders
    const int lt = tid - 160;
    const uint32_t q_addr = smem_u32(sQ);
    for (int c = lt; c < TROWS * 16; c += TLOADERS) {
      const int r = c >> 4, ch = c & 15;
      const int nd = node0 + r / G;
      const bool valid = nd < n_b;
      const __nv_bfloat16* src = p.q + (static_cast<size_t>(q_begin + (valid ? nd : 0)) * p.Hq + h * G + r % G) * TD + ch * 8;
      cp_async16_tc(q_addr + (ch >> 3) * (TROWS * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4), src, valid);
    }
    cp_async_commit_tc();
    constexpr int RSTEP = TLOADERS / 16;        // key rows covered by one pass of all loader threads
    const int ch = lt & 15, r0 = lt >> 4;       // this thread copies chunk `ch` of keys r0, r0+RSTEP, ...
    // slots of the first tile; the next tile's are fetched while the current tile's copies are issued
    int slot_next[TKEYS / RSTEP];
#pragma unroll
    for (int j = 0; j < TKEYS / RSTEP; ++j) {
      const int kp = t_begin * TKEYS + r0 + RSTEP * j;
      slot_next[j] = kp < L ? __ldg(slots + kp) : 0;
    }
    bool ok = true;
    // copies complete in issue order (Q, tile 0, tile 1, ...); `next_sig` is the next one to publish (-1 = Q)
    int next_sig = -1;
    auto publish_before = [&](int upto) {
      if (next_sig < upto) fence_proxy_async();
      for (; next_sig < upto; ++next_sig) {
        if (next_sig < 0) mbar_arrive(q_full); else mbar_arrive(&kv_full[next_sig % TSTAGES]);
        if (lt == 0 && next_sig >= 0 && next_sig < 8) attn_trace(40 + next_sig);   // tile published by loader thread 0
      }
    };
    for (int i = 0; i < nt && ok; ++i) {
      const int s = i % TSTAGES;
      if (i >= TSTAGES) {
        const uint32_t par = ((i / TSTAGES) & 1) ^ 1;
        if (!mbar_test_wait(&kv_empty[s], par)) {
          // about to block on the consumer: it may itself be waiting for tiles not yet published
          cp_async_wait_tc<0>();
          publish_before(i);
          ok = mbar_wait_backoff(&kv_empty[s], par, p.status, kTimeoutEmpty);
        }
      }
      if (!ok) break;
      const int k0 = (t_begin + i) * TKEYS;
      const uint32_t k_addr = smem_u32(sKV + s * kStageKV);
      int slot_cur[TKEYS / RSTEP];
#pragma unroll
      for (int j = 0; j < TKEYS / RSTEP; ++j) {
        slot_cur[j] = slot_next[j];
        const int kpn = k0 + TKEYS + r0 + RSTEP * j;
        slot_next[j] = (i + 1 < nt && kpn < L) ? __ldg(slots + kpn) : 0;
      }
#pragma unroll
      for (int j = 0; j < TKEYS / RSTEP; ++j) {
        const int r = r0 + RSTEP * j;
        const int kp = k0 + r;
        const bool valid = kp < L;
        int slot = slot_cur[j];
        if (slot < 0 || slot >= p.S) { report(p.status, kBadSlot); slot = 0; }
        const size_t off = (static_cast<size_t>(h) * p.S + slot) * TD + ch * 8;
        const uint32_t dst = (ch >> 3) * (TKEYS * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
        cp_async16_tc(k_addr + dst, p.k_pool + off, valid);
        cp_async16_tc(k_addr + TKEYS * 256 + dst, p.v_pool + off, valid);
      }
      cp_async_commit_tc();
      if (lt == 0 && i < 8) attn_trace(32 + i);    // copies of tile i issued
      cp_async_wait_tc<2>();          // everything but the two newest groups has landed
      publish_before(i - 1);
    }
    if (ok) {
      cp_async_wait_tc<0>();
      publish_before(nt);
    }
  } else if (warp == 4) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(TROWS, TKEYS);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_bmn(TROWS, TD);
      bool ok = mbar_wait_backoff(q_full, 0, p.status, kTimeoutFull);
      attn_trace(2);                // Q landed
      auto issue_pv = [&](int j) {
        const int s = j % TSTAGES, pb = j & 1;
        const uint32_t v_addr = smem_u32(sKV + s * kStageKV + TKEYS * 256);
        const uint64_t a_desc = umma_desc_sw128(smem_u32(sP + pb * kSmemP));
#pragma unroll
        for (int k = 0; k < TKEYS / 16; ++k)
          umma_f16(tmem_o, a_desc + 2 * k, umma_desc_sw128_mn(v_addr + k * 2048, TKEYS * 128), idesc_pv, (j | k) != 0 ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(&pv_done[pb]);
      };
      for (int i = 0; i < nt && ok; ++i) {
        const int s = i % TSTAGES, sb = i & 1;
        ok = mbar_wait_backoff(&kv_full[s], (i / TSTAGES) & 1, p.status, kTimeoutFull);
        if (!ok) break;
        if (i < 8) attn_trace(8 + i);   // K/V tile i landed
        // S buffer sb was consumed when P of tile i-2 was published (waited for below, before PV(i-2))
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKV + s * kStageKV);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t hoff = (k >> 2), kk = k & 3;
          umma_f16(tmem_base + sb * TKEYS, umma_desc_sw128(smem_u32(sQ) + hoff * (TROWS * 128)) + 2 * kk,
                   umma_desc_sw128(k_addr + hoff * (TKEYS * 128)) + 2 * kk, idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        if (i >= 1) {
          ok = mbar_wait_backoff(&p_full[(i - 1) & 1], ((i - 1) >> 1) & 1, p.status, kTimeoutAccum);
          if (!ok) break;
          tc_fence_after();
          issue_pv(i - 1);
        }
      }
      if (ok) {
        ok = mbar_wait_backoff(&p_full[(nt - 1) & 1], ((nt - 1) >> 1) & 1, p.status, kTimeoutAccum);
        if (ok) {
          tc_fence_after();
          issue_pv(nt - 1);
        }
      }
      umma_commit(o_done);     // also releases the epilogue on an error path
    }
  } else {
    // ================================================================ softmax + epilogue (one row per thread)
    int mw[8];
#pragma unroll
    for (int w = 0; w < 8; ++w)
      mw[w] = (!p.causal && row_valid && w < p.W) ? p.mask_bits[static_cast<size_t>(q_begin + node) * p.W + w] : 0;
    bool ok = true;
    for (int i = 0; i < nt && ok; ++i) {
      const int sb = i & 1;
      ok = mbar_wait_backoff(&s_full[sb], (i >> 1) & 1, p.status, kTimeoutAccum);
      if (!ok) break;
      tc_fence_after();
      if (tid == 0 && i < 8) attn_trace(16 + i);   // scores of tile i ready
      uint32_t sr[64];
      tmem_ld_32x32(tmem_base + t_lane + sb * TKEYS, sr);
      tmem_ld_32x32(tmem_base + t_lane + sb * TKEYS + 32, sr + 32);
      tmem_ld_wait();
      // visibility of the tile's 64 keys for this row, as one 64-bit word (bit c = key k0 + c)
      const int k0 = (t_begin + i) * TKEYS;
      const int jlo = k0 - past;                         // window index of the tile's first key (may be < 0)
      unsigned long long vm = 0ull;
      if (row_valid) {
        if (jlo <= -TKEYS) {
          vm = ~0ull;                                    // the whole tile is prefix
        } else {
          if (jlo < 0) vm = (1ull << (-jlo)) - 1ull;     // prefix part of a mixed tile
          if (p.causal) {
            const int cmax = node - jlo;                 // window key j = jlo + c is visible when j <= node
            if (cmax >= 63) vm = ~0ull; else if (cmax >= 0) vm |= (1ull << (cmax + 1)) - 1ull;
          } else {
#pragma unroll
            for (int w = 0; w < 8; ++w) {
              const int sh = 32 * w - jlo;               // where bit 0 of mask word w falls in the tile
              const unsigned long long word = static_cast<unsigned int>(mw[w]);
              if (sh >= 0 && sh < 64) vm |= word << sh;
              else if (sh < 0 && sh > -32) vm |= word >> (-sh);
            }
          }
        }
        const int left = L - k0;                         // keys at or past L do not exist
        if (left < 64) vm &= (left <= 0) ? 0ull : ((1ull << left) - 1ull);
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one 64-deep
      if (vm == ~0ull) {              // the common case: every key of the tile is visible to this row
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = __uint_as_float(sr[c]) * p.scale_log2;
          sr[c] = __float_as_uint(x);
          mx4[c & 3] = fmaxf(mx4[c & 3], x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const bool vis = (vm >> c) & 1ull;
          const float x = vis ? __uint_as_float(sr[c]) * p.scale_log2 : -INFINITY;
          sr[c] = __float_as_uint(x);
          mx4[c & 3] = fmaxf(mx4[c & 3], x);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // integer running maximum in the log2 domain (probabilities are then exact powers of two apart
      // whatever the tile order or key split; see the mma.sync kernel)
      const float m_new = fmaxf(m_run, ceilf(mx));
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_safe);          // 0 when nothing was visible before
      m_run = m_new;
      // P buffer sb is free once PV of tile i-2 has completed
      if (i >= 2) ok = mbar_wait_backoff(&pv_done[sb], ((i - 2) >> 1) & 1, p.status, kTimeoutAccum);
      if (!ok) break;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t p_row = smem_u32(sP + sb * kSmemP) + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = fast_exp2(__uint_as_float(sr[c8 * 8 + 2 * e]) - m_safe);
          const float p1 = fast_exp2(__uint_as_float(sr[c8 * 8 + 2 * e + 1]) - m_safe);
          rs4[e] += p0 + p1;
          __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
          w4[e] = *reinterpret_cast<uint32_t*>(&v);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + ((c8 ^ (row & 7)) << 4)), "r"(w4[0]),
                     "r"(w4[1]), "r"(w4[2]), "r"(w4[3]) : "memory");
      }
      l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
      // rescale O when some row of this warp raised its maximum (tcgen05.ld/st are warp-wide)
      const bool need = i > 0 && alpha != 1.f;
      if (__any_sync(0xffffffffu, need)) {
        ok = mbar_wait_backoff(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, p.status, kTimeoutAccum);   // every earlier PV is in O
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < TD; c0 += 32) {
          uint32_t orr[32];
          tmem_ld_32x32(tmem_o + t_lane + c0, orr);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
          tmem_st_32x32(tmem_o + t_lane + c0, orr);
        }
        tmem_st_wait();
      }
      fence_proxy_async();          // P (generic-proxy stores) -> visible to the MMA's async-proxy reads
      tc_fence_before();
      mbar_arrive(&p_full[sb]);
      if (tid == 0 && i < 8) attn_trace(24 + i);   // P of tile i published
    }
    // ---- epilogue
    if (ok) ok = mbar_wait_backoff(o_done, 0, p.status, kTimeoutAccum);
    tc_fence_after();
    if (tid == 0) attn_trace(3);    // output accumulator complete
    sm_ok = ok;
    if (ok && !cmerge) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < TD; c0 += 32) {
        uint32_t orr[32];
        tmem_ld_32x32(tmem_o + t_lane + c0, orr);
        tmem_ld_wait();
        if (!row_valid) continue;
        if (p.splits == 1) {
          uint4 pk[4];
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(pk);
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o2[j] = __floats2bfloat162_rn(__uint_as_float(orr[2 * j]) * inv, __uint_as_float(orr[2 * j + 1]) * inv);
          uint4* dst = reinterpret_cast<uint4*>(p.out + out_row * TD + c0);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = pk[j];
        } else {
          float4* dst = reinterpret_cast<float4*>(p.ws_o + (static_cast<size_t>(split) * p.T * p.Hq + out_row) * TD + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j] = make_float4(__uint_as_float(orr[4 * j]), __uint_as_float(orr[4 * j + 1]),
                                 __uint_as_float(orr[4 * j + 2]), __uint_as_float(orr[4 * j + 3]));
        }
      }
      if (p.splits > 1 && row_valid) {
        float* ml = p.ws_ml + (static_cast<size_t>(split) * p.T * p.Hq + out_row) * 2;
        ml[0] = m_run;
        ml[1] = l_run;
      }
    }
  }

  if (cmerge) {
    // ---------------------------------------------------------------- merge of the key splits inside the cluster
    // Column chunk c (32 of the 128 output columns) is finished by CTA c % splits.  Every CTA pushes its
    // unnormalised chunk (column-major, 16 KB) into the owner's shared memory and its rows' (max, sum) to
    // all CTAs; the receive areas reuse the K/V stages + P buffers (chunks, at most 8 x 16 KB = 128 KB) and the
    // Q tile ((max, sum) pairs, at most 8 KB), all dead once every CTA of the cluster has left its main loop.
    const int per_owner = (4 + p.splits - 1) / p.splits;
    float* recv_o = reinterpret_cast<float*>(sKV);
    float* recv_ml = reinterpret_cast<float*>(sQ);
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (tid == 0) attn_trace(5);    // every CTA of the cluster left its main loop
    if (warp < 4) {
      const bool have = nt > 0 && sm_ok;
      const float m_pub = have ? m_run : -INFINITY;
      const uint32_t ml_addr = smem_u32(recv_ml) + static_cast<uint32_t>((split * TROWS + row) * 8);
      for (int d = 0; d < p.splits; ++d) {
        const uint32_t a = map_to_cta(ml_addr, d);
        st_dsmem_f32(a, m_pub);
        st_dsmem_f32(a + 4, have ? l_run : 0.f);
      }
      if (have) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t orr[32];
          tmem_ld_32x32(tmem_o + t_lane + c * 32, orr);
          tmem_ld_wait();
          const uint32_t dst = map_to_cta(smem_u32(recv_o), c % p.splits) +
                               static_cast<uint32_t>(((split * per_owner + c / p.splits) * 4096 + row) * 4);
#pragma unroll
          for (int j = 0; j < 32; ++j) st_dsmem_f32(dst + j * (TROWS * 4), __uint_as_float(orr[j]));
        }
      }
    }
    if (tid == 0) attn_trace(6);    // partials pushed
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (tid == 0) attn_trace(7);    // partials of all splits landed
    if (warp < 4 && row_valid) {
      float m = -INFINITY;
      for (int s2 = 0; s2 < p.splits; ++s2) m = fmaxf(m, recv_ml[(s2 * TROWS + row) * 2]);
      float wsrc[8], lsum = 0.f;
      for (int s2 = 0; s2 < p.splits; ++s2) {
        const float ms = recv_ml[(s2 * TROWS + row) * 2];
        wsrc[s2] = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
        lsum += recv_ml[(s2 * TROWS + row) * 2 + 1] * wsrc[s2];
      }
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      for (int c = split; c < 4; c += p.splits) {
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0.f;
        for (int s2 = 0; s2 < p.splits; ++s2) {
          if (wsrc[s2] == 0.f) continue;       // that split saw no visible key (its chunk was never pushed)
          const float* src = recv_o + (s2 * per_owner + c / p.splits) * 4096 + row;
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] += src[j * TROWS] * wsrc[s2];
        }
        uint4 pk[4];
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(pk);
#pragma unroll
        for (int j = 0; j < 16; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j] * inv, acc[2 * j + 1] * inv);
        uint4* dst = reinterpret_cast<uint4*>(p.out + out_row * TD + c * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = pk[j];
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (tid == 0) attn_trace(4);      // epilogue stores issued
  tc_fence_before();
  __syncthreads();
  if (warp == 4 && nt > 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int G>
static int launch_attn_tc(const AttnTcParams& p, int q_tiles, bool pdl, cudaStream_t stream) {
  static int configured[kMaxDevicesCached] = {};
  auto kern = paged_tree_attn_tc_kernel<G>;
  if (ensure_dyn_smem(kern, kAttnTcSmem, configured) != 0) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(q_tiles, p.Hkv, p.splits);
  cfg.blockDim = dim3(TTHREADS);
  cfg.dynamicSmemBytes = kAttnTcSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.cluster_merge) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = p.splits;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kern, p) == cudaSuccess ? 0 : -4;
}

}  // namespace js

// Profiling hook: 32 timestamps of CTA (0,0,0) go to `buf` (device memory) on every launch; nullptr switches it off.
extern "C" int js_attn_tc_set_trace(unsigned long long* buf) {
  return cudaMemcpyToSymbol(js::g_attn_trace, &buf, sizeof(buf)) == cudaSuccess ? 0 : -1;
}

extern "C" int js_attn_merge(float* ws_o, float* ws_ml, void* out, int T, int Hq, int splits, int pdl, cudaStream_t stream);

// How many clusters of `splits` CTAs of the kernel for GQA group size G can be resident at once on the current
// device (a cluster lives inside one GPC, so this is less than SMs / splits); 0 or negative = cannot say.  The host
// picks the number of key splits from it so that a launch is one wave.
extern "C" int js_attn_tc_max_active_clusters(int G, int splits) {
  using namespace js;
  if (splits < 1 || splits > kMaxClusterSplits) return -1;
  const void* kern = nullptr;
  switch (G) {
    case 1: kern = reinterpret_cast<const void*>(paged_tree_attn_tc_kernel<1>); break;
    case 2: kern = reinterpret_cast<const void*>(paged_tree_attn_tc_kernel<2>); break;
    case 4: kern = reinterpret_cast<const void*>(paged_tree_attn_tc_kernel<4>); break;
    case 8: kern = reinterpret_cast<const void*>(paged_tree_attn_tc_kernel<8>); break;
    case 16: kern = reinterpret_cast<const void*>(paged_tree_attn_tc_kernel<16>); break;
    default: return -2;
  }
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnTcSmem) != cudaSuccess) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, splits);
  cfg.blockDim = dim3(TTHREADS);
  cfg.dynamicSmemBytes = kAttnTcSmem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return -4; }
  return n;
}

// Same arguments as js_paged_tree_attention.  Needs 128 % (Hq / Hkv) == 0 and W <= 8 (windows of up to 256 nodes).
extern "C" int js_paged_tree_attention_tc(const void* q, const void* k_pool, const void* v_pool, const int* slot_map,
                                          const int* seq_rows, const int* cu_q, const int* past_lens,
                                          const int* mask_bits, void* out, float* ws_o, float* ws_ml, int* status, int B,
                                          int T, int Hq, int Hkv, int S, int max_len, int W, int causal, int splits,
                                          float scale, int pdl, cudaStream_t stream) {
  using namespace js;
  if (T <= 0 || B <= 0) return 0;
  if (Hq % Hkv) return -10;
  const int G = Hq / Hkv;
  if (splits < 1) return -11;
  if (splits > 1 && (ws_o == nullptr || ws_ml == nullptr)) return -12;
  if (!causal && (mask_bits == nullptr || W < 1 || W > 8)) return -13;
  // The key splits merge inside a cluster only while every cluster of the launch is resident at once (a second
  // wave would double the kernel's time); otherwise partials go through the workspace and the merge kernel.
  bool in_cluster = splits >= 2 && splits <= kMaxClusterSplits;
  if (in_cluster) {
    static int room[kMaxDevicesCached][5][kMaxClusterSplits + 1] = {};     // 0 = not asked yet
    int dev = 0;
    cudaGetDevice(&dev);
    const int gi = G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : G == 8 ? 3 : 4;
    int r = 0;
    if (dev >= 0 && dev < kMaxDevicesCached) r = room[dev][gi][splits];
    if (r == 0) {
      r = js_attn_tc_max_active_clusters(G, splits);
      if (r <= 0) r = -1;
      if (dev >= 0 && dev < kMaxDevicesCached) room[dev][gi][splits] = r;
    }
    const int npt = 128 / G;
    in_cluster = r > 0 && ((T + npt - 1) / npt) * Hkv <= r;
  }
  AttnTcParams p{reinterpret_cast<const __nv_bfloat16*>(q), reinterpret_cast<const __nv_bfloat16*>(k_pool),
                 reinterpret_cast<const __nv_bfloat16*>(v_pool), slot_map, seq_rows, cu_q, past_lens, mask_bits,
                 reinterpret_cast<__nv_bfloat16*>(out), ws_o, ws_ml, status, B, T, Hq, Hkv, S, max_len, W, causal,
                 splits, scale * 1.4426950408889634f, in_cluster ? 1 : 0};
  int rc;
  switch (G) {
    case 1: rc = launch_attn_tc<1>(p, (T + 127) / 128 + B, pdl != 0, stream); break;
    case 2: rc = launch_attn_tc<2>(p, (T + 63) / 64 + B, pdl != 0, stream); break;
    case 4: rc = launch_attn_tc<4>(p, (T + 31) / 32 + B, pdl != 0, stream); break;
    case 8: rc = launch_attn_tc<8>(p, (T + 15) / 16 + B, pdl != 0, stream); break;
    case 16: rc = launch_attn_tc<16>(p, (T + 7) / 8 + B, pdl != 0, stream); break;
    default: return -14;
  }
  if (rc != 0 || splits == 1 || p.cluster_merge) return rc;
  return js_attn_merge(ws_o, ws_ml, out, T, Hq, splits, pdl, stream);
}
