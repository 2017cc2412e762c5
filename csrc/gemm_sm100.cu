// bf16 GEMM for sm_100a:  C[M,N] = A[M,K] * W[N,K]^T  with fused epilogues.
// Reference twins (library GEMMs + ATen glue of the fused verify stack): jetspec/inference_engine/compiled_verify_stack.py:170-272
// (fused QKV, o_proj, gate/up + activation, down + residual, LM head); grouped mode: jetspec/models/moe_fused.py:16-116.
//
// Both operands are K-major (activations row-major, weights in nn.Linear layout), so a tile
// is a stack of 128-byte rows that TMA drops into shared memory with the 128-byte swizzle and
// tcgen05.mma consumes through shared-memory descriptors.  One CTA owns a 128 x BN output
// tile; the fp32 accumulator lives in tensor memory (BN columns x 128 lanes).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer (one
// elected lane issues tcgen05.mma), warps 2..5 = epilogue, each reading the TMEM lane
// quadrant (warp_id % 4) it is allowed to touch.
//
// The decode-time shapes are skinny (M <= 128 rows against 4096..151936 weight rows), i.e.
// bound by streaming the weights from HBM.  To put all 148 SMs to work on the narrow
// projections the K dimension can be split across a thread-block cluster (1,1,SPLIT): each
// CTA accumulates its K range, parks the partial tile in its own shared memory, and after a
// cluster barrier every CTA reduces and finishes a column slice of the tile by reading its
// peers' partials through distributed shared memory — no global round trip, no atomics,
// deterministic summation order.  (Partials are PUSHED: each CTA stores its chunks into the
// owning peer's receive area with st.shared::cluster, so the reduce reads local memory only.)
//
// NVFP4 mode (template flag FP4): both operands are packed e2m1 (256 elements per 128-byte
// swizzle row, so one stage carries four K=64 MMAs), the e4m3 block scales arrive with plain
// bulk copies in 512-byte tiles (128 rows x 4 blocks), are copied to tensor memory with
// tcgen05.cp and consumed by tcgen05.mma.kind::mxf4nvf4.block_scale; the epilogue applies the
// per-row activation scale times the per-tensor weight scale.
//
// Epilogues: plain store (+ residual), SwiGLU (the tile holds BN/2 gate and BN/2 up columns
// of the same outputs), per-tile argmax partials (LM head), per-tile top-8 + log-sum-exp
// partials (draft head logits).
#include "common.cuh"

#include <math.h>

namespace js {

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int kTopK = 8;

enum GemmEpi : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ARGMAX = 2, EPI_TOPK = 3, EPI_STORE_F32 = 4, EPI_ALLREDUCE = 5, EPI_EP_COMBINE = 6 };

struct GemmParams {
  int M, N, K;
  int ldc;                      // elements
  void* C;                      // bf16 (or fp32 for EPI_STORE_F32) output
  const __nv_bfloat16* residual;  // optional, same shape/ld as C (may alias C)
  float* part_val;              // ARGMAX: [M, n_tiles] ; TOPK: [M, n_tiles, 8] values
  int* part_idx;                // ARGMAX: [M, n_tiles] ; TOPK: [M, n_tiles, 8] indices
  float* part_lse;              // TOPK: [M, n_tiles, 2] (running max, sum of exp)
  int* status;
  unsigned long long* trace;    // optional: 8 phase timestamps (ns) written by CTA (0,0,0)
  // EPI_ALLREDUCE (tensor-parallel row-parallel GEMM): every rank's receive buffer and flag array
  __nv_bfloat16* const* peer_recv;  // [world] -> (world, m_cap, N) bf16 on that rank
  int* const* peer_flags;           // [world] -> one counter per CTA of this grid on that rank
  int rank, world, m_cap;
  // grouped mode (MoE experts): blockIdx.z is the expert; its rows are group_off[e] .. group_off[e+1]
  // of A and C, its weights are rows e*N .. (e+1)*N of W.  No K split in this mode.
  const int* group_off;
  // EPI_EP_COMBINE (expert-parallel down projection): row r of the sorted rows belongs to
  // (token, choice) pair row_pair[r] with routing weight row_weight[r]; the weighted output row is
  // stored into every rank's pair buffer (n_pairs, N) and a per-rank counter is bumped per CTA.
  const int* row_pair;
  const float* row_weight;
  __nv_bfloat16* const* peer_pairs;
  int* const* peer_cnt;
  // EPI_EP_COMBINE with token-sharded dispatch: row r of this rank's receive slab came from rank row_meta[r].x
  // as that rank's (token, choice) pair row_meta[r].y; the weighted output row returns to that rank only, as
  // flagged 8-byte cells {two bf16 values, 1} that the owner's finishing kernel polls (no counters)
  const int2* row_meta;
  // NVFP4 mode: block scales of A and W in 512-byte tiles, per-row scale of A, per-tensor scale of W
  const uint8_t* sfa;
  const uint8_t* sfw;
  const float* row_scale;
  float w_scale;
  // EPI_ALLREDUCE: only push the partial tile and bump the flags; a finishing kernel reduces (no wait in this kernel)
  int ar_push_only;
  // Tile order: 0 = column tiles fastest (consecutive CTAs share the activation tile), 1 = row tiles fastest
  // (consecutive CTAs share the WEIGHT tile: for a vocabulary matrix larger than L2 and many row tiles, each
  // weight tile then comes from HBM once instead of once per row tile)
  int m_fast;
  // Grouped mode: a row tile with at most this many rows left loads its activations through the second tensor map,
  // whose box holds only that many rows (0 = always the 128-row box).  With ~8 rows per expert (MoE decode) a
  // 128-row box would make the activations half of every stage's bytes although almost none of its rows are used;
  // the accumulator rows beyond the box read stale shared memory and are never stored.
  int a_small_rows;
};

JS_DEVICE void red_release_sys_add(int* addr, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
JS_DEVICE int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
JS_DEVICE void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the 4 epilogue warps

JS_DEVICE unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define JS_TRACE(slot)                                                                     \
  do {                                                                                     \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.trace[slot] = gtime(); \
  } while (0)

// BUDGET_KB bounds the pipeline's shared memory: ~96 KB lets two CTAs share an SM (more tiles
// in flight, natural load balance when the tile count is not a multiple of 148), ~192 KB gives
// one CTA per SM a deeper pipeline.
// MT = row tiles per CTA (1 or 2): with 2, one CTA computes a 256 x BN tile as two 128-row accumulators that share
// every weight stage, so a k-block brings 1.5x the FLOPs per byte through the L2-to-SM path (many-row GEMMs).
template <int BN, int BUDGET_KB, bool FP4 = false, int MT = 1>
struct GemmSmem {
  static constexpr int kStageA = MT * BM * BK * 2; // 128-byte rows in both modes
  static constexpr int kStageW = BN * BK * 2;
  static constexpr int kStageSF = FP4 ? 2048 + (BN / 128) * 2048 : 0;   // 4 scale tiles of A + 4 per 128 rows of W
  static constexpr int kStage = kStageA + kStageW + kStageSF;
  static constexpr int kBudget = BUDGET_KB * 1024;
  static constexpr int kMaxStages = FP4 ? 4 : 8;   // FP4: every stage also owns 32 tensor-memory columns of scales
  static constexpr int kStages = (kBudget / kStage) > kMaxStages ? kMaxStages : ((kBudget / kStage) < 2 ? 2 : (kBudget / kStage));
  static constexpr int kMinBlocks = BUDGET_KB <= 100 ? 2 : 1;
  static constexpr int kTiles = kStages * kStage;
};

// Split-K receive area: every CTA of the cluster owns some 32-column chunks of the tile and gets,
// from each source CTA, one 16 KB slot (32 columns x 128 rows fp32, column-major) per owned chunk.
__host__ __device__ inline int recv_slots_per_src(int split, int bn, bool swiglu) {
  const int hc = (swiglu ? bn / 2 : bn) / 32;
  const int per = (hc + split - 1) / split;
  return swiglu ? 2 * per : per;
}
__host__ __device__ inline int recv_bytes(int split, int bn, bool swiglu) {
  return split > 1 ? split * recv_slots_per_src(split, bn, swiglu) * 16384 : 0;
}

// The receive area shares the stages' memory only when the two do not fit side by side.
__host__ __device__ inline bool recv_aliases_stages(int tiles_bytes, int recv_total) {
  return recv_total > 0 && tiles_bytes + recv_total + 1280 > 227 * 1024;
}

template <int BN, int EPI, int BUDGET_KB, bool FP4 = false, int MT = 1>
__global__ void __launch_bounds__(kGemmThreads, GemmSmem<BN, BUDGET_KB, FP4, MT>::kMinBlocks)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                 const __grid_constant__ CUtensorMap tmA2, GemmParams p) {
  using S = GemmSmem<BN, BUDGET_KB, FP4, MT>;
  constexpr int kStages = S::kStages;
  static_assert(!FP4 || BN == 128, "the NVFP4 path is built for 128-column tiles");
  static_assert(MT == 1 || (MT == 2 && !FP4 && BN == 256), "two row tiles per CTA: bf16, 256-column tiles, no K split");
  // FP4: accumulator in columns [0,128), block scales of stage s in [128 + 32 s, 128 + 32 s + 32)
  // MT == 2: the second row tile's accumulator sits in columns [BN, 2 BN)
  constexpr uint32_t kTmemCols = MT == 2 ? 512 : FP4 ? 256 : (BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256);   // power of two
  constexpr int kXStep = FP4 ? 128 : BK;              // TMA x advance per k-block (bytes resp. bf16 elements)
  constexpr int kKPerBlock = FP4 ? 256 : BK;          // K elements per pipeline stage

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [pipeline stages][split-K receive area][barriers].  Peers push into the receive area while
  // this CTA may still be streaming, so it normally sits behind the stages; only when both do
  // not fit (deep pipeline) it ALIASES them, guarded by one more cluster barrier after the main loop.
  const bool grouped = p.group_off != nullptr;
  const int recv_total = recv_bytes(grouped ? 1 : gridDim.z, BN, EPI == EPI_SWIGLU);
  const bool alias = recv_aliases_stages(S::kTiles, recv_total);
  const int data_bytes = alias ? (S::kTiles > recv_total ? S::kTiles : recv_total) : S::kTiles + recv_total;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + data_bytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* accum_bar = empty_bar + kStages;
  uint64_t* tmem_free = accum_bar + 1;       // grouped mode: the epilogue has drained the accumulator of a row tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int split = grouped ? 1 : gridDim.z;
  const int z = grouped ? 0 : blockIdx.z;    // == rank in the (1,1,split) cluster
  const int expert = grouped ? blockIdx.z : 0;
  int bx = blockIdx.x, by = blockIdx.y;        // column tile, row tile
  if (!grouped && p.m_fast) {
    const int lin = blockIdx.y * gridDim.x + blockIdx.x;
    by = lin % static_cast<int>(gridDim.y);
    bx = lin / static_cast<int>(gridDim.y);
  }
  const int n0 = bx * BN;
  const int m_first = grouped ? p.group_off[expert] + by * BM : by * BM * MT;
  const int m_end = grouped ? p.group_off[expert + 1] : p.M;
  const int wn0 = expert * p.N + n0;         // row of this tile in the (stacked) weight matrix
  if (m_first >= m_end) return;              // this expert has fewer row tiles (uniform for the CTA)
  // Grouped mode: the launch covers gridDim.y row tiles per expert; an expert with more rows than that is still
  // finished, because this CTA goes on to row tiles by + gridDim.y, by + 2 gridDim.y, ... of its expert (same
  // weight tile, the pipeline simply keeps running; the accumulator is handed back and forth between the MMA
  // issuer and the epilogue through `tmem_free`).  Every other mode processes exactly one tile.
  const int tile_step = grouped ? static_cast<int>(gridDim.y) * BM : BM;
  const int n_tiles_cta = grouped ? (m_end - m_first + tile_step - 1) / tile_step : 1;
  int m0 = m_first;
  const int kb_total = (p.K + kKPerBlock - 1) / kKPerBlock;
  const int kb_begin = (kb_total * z) / split;
  const int kb_end = (kb_total * (z + 1)) / split;
  const int nkb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    JS_TRACE(0);   // kernel start
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmW);
    if (p.a_small_rows > 0) tma_prefetch_desc(&tmA2);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    mbar_init(tmem_free, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Let the next kernel in the stream start its own prologue; it still waits for this grid
  // to finish before touching our output.
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      JS_TRACE(1);   // setup done, first TMA about to issue
      // Weights do not depend on the previous kernel: start streaming them before waiting on it.
      const int pre = nkb < kStages ? nkb : kStages;
      // FP4: scale tiles of k-block kb are 4 consecutive 512-byte tiles of this operand's row tile
      const size_t sf_row = static_cast<size_t>(p.K / 64) * 512;
      auto load_sfw = [&](int s, int kb) {
        if constexpr (FP4)
          bulk_load_1d(smem + s * S::kStage + S::kStageA + S::kStageW + 2048,
                       p.sfw + static_cast<size_t>(wn0 / 128) * sf_row + static_cast<size_t>(kb) * 2048, 2048, &full_bar[s]);
      };
      auto load_sfa = [&](int s, int kb) {
        if constexpr (FP4)
          bulk_load_1d(smem + s * S::kStage + S::kStageA + S::kStageW,
                       p.sfa + static_cast<size_t>(m0 / 128) * sf_row + static_cast<size_t>(kb) * 2048, 2048, &full_bar[s]);
      };
      // bytes a stage receives: the activation box shrinks for a row tile with few rows left (grouped mode)
      auto small_tile = [&](int m_tile) { return p.a_small_rows > 0 && m_end - m_tile <= p.a_small_rows; };
      auto stage_bytes = [&](bool small) {
        return static_cast<uint32_t>(small ? S::kStage - S::kStageA + p.a_small_rows * BK * 2 : S::kStage);
      };
      const bool small0 = small_tile(m0);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], stage_bytes(small0));
        tma_load_2d(smem + i * S::kStage + S::kStageA, &tmW, &full_bar[i], (kb_begin + i) * kXStep, wn0);
        load_sfw(i, kb_begin + i);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        if (small0) {
          tma_load_2d(smem + i * S::kStage, &tmA2, &full_bar[i], (kb_begin + i) * kXStep, m0);
        } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d(smem + i * S::kStage + mt * (BM * BK * 2), &tmA, &full_bar[i], (kb_begin + i) * kXStep, m0 + mt * BM);
        }
        load_sfa(i, kb_begin + i);
      }
      bool p_ok = true;
      for (int tj = 0; tj < n_tiles_cta && p_ok; ++tj) {
        const int m_tile = m_first + tj * tile_step;
        const bool small = small_tile(m_tile);
        for (int i = (tj == 0 ? pre : 0); i < nkb; ++i) {
          const int g = tj * nkb + i;              // running k-block count of this CTA
          const int s = g % kStages;
          if (g >= kStages) {
            const uint32_t ph = (g / kStages) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, p.status, kTimeoutEmpty)) { p_ok = false; break; }
          }
          mbar_expect_tx(&full_bar[s], stage_bytes(small));
          tma_load_2d(smem + s * S::kStage + S::kStageA, &tmW, &full_bar[s], (kb_begin + i) * kXStep, wn0);
          if (small) {
            tma_load_2d(smem + s * S::kStage, &tmA2, &full_bar[s], (kb_begin + i) * kXStep, m_tile);
          } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              tma_load_2d(smem + s * S::kStage + mt * (BM * BK * 2), &tmA, &full_bar[s], (kb_begin + i) * kXStep, m_tile + mt * BM);
          }
          load_sfw(s, kb_begin + i);
          load_sfa(s, kb_begin + i);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = FP4 ? umma_idesc_nvfp4(BM, BN) : umma_idesc_bf16(BM, BN);
      bool ok = true;
      for (int tj = 0; tj < n_tiles_cta && ok; ++tj) {
      if (tj > 0) {                 // the epilogue must have read the previous row tile out of tensor memory
        ok = mbar_wait(tmem_free, (tj - 1) & 1, p.status, kTimeoutAccum);
        if (!ok) break;
        tc_fence_after();
      }
      for (int i = 0; i < nkb && ok; ++i) {
        const int g = tj * nkb + i;
        const int s = g % kStages;
        const uint32_t ph = (g / kStages) & 1;
        ok = mbar_wait(&full_bar[s], ph, p.status, kTimeoutFull);
        if (!ok) break;
        if (g == 0) JS_TRACE(2);   // first stage landed
        tc_fence_after();
        const uint64_t a_desc = umma_desc_sw128(smem_u32(smem + s * S::kStage));
        const uint64_t b_desc = umma_desc_sw128(smem_u32(smem + s * S::kStage + S::kStageA));
        if constexpr (FP4) {
          // scale tiles: shared memory -> tensor memory (4 columns per 128 rows x 4 blocks), then
          // four K=64 MMAs, each reading its own 4+4 scale columns
          const uint32_t sf_smem = smem_u32(smem + s * S::kStage + S::kStageA + S::kStageW);
          const uint32_t sf_tmem = tmem_base + 128 + s * 32;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tmem_cp_32x128b_warpx4(sf_tmem + 4 * k, umma_desc_sf(sf_smem + 512 * k));
            tmem_cp_32x128b_warpx4(sf_tmem + 16 + 4 * k, umma_desc_sf(sf_smem + 2048 + 512 * k));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advancing K by 64 e2m1 = 32 bytes inside the swizzle row = +2 in 16-byte units
            umma_nvfp4(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, sf_tmem + 4 * k, sf_tmem + 16 + 4 * k,
                       (i | k) != 0 ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 elements = 32 bytes inside the swizzle row = +2 in 16-byte units
            umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
            if constexpr (MT == 2) {     // second row tile: its own A rows and accumulator, the same weight stage
              const uint64_t a2_desc = umma_desc_sw128(smem_u32(smem + s * S::kStage + BM * BK * 2));
              umma_f16(tmem_base + BN, a2_desc + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
            }
          }
        }
        umma_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
      }
      umma_commit(accum_bar);         // accumulator complete (also releases the epilogue on error)
      }
    }
  }

  // ------------------------------------------------------------------ epilogue
  const bool epi_warp = warp >= 2;
  const int quad = warp & 3;                     // TMEM lane quadrant this warp may read
  const int row = quad * 32 + lane;              // row of the tile owned by this thread
  uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
  // split-K: this CTA's receive area (after the pipeline stages) and the chunk -> owner mapping
  constexpr bool kSwiglu = (EPI == EPI_SWIGLU);
  constexpr int kHC = (kSwiglu ? BN / 2 : BN) / 32;          // owned-chunk index space
  const int per_owner = (kHC + split - 1) / split;
  const int slots_per_src = kSwiglu ? 2 * per_owner : per_owner;
  const uint32_t recv_addr = smem_u32(smem + (alias ? 0 : S::kTiles));
  // TMEM chunk `ch` (32 columns) is finished by CTA owner_of(ch); local_of(ch) is its slot there
  auto owner_of = [&](int ch) { return (ch % kHC) % split; };
  auto local_of = [&](int ch) { return (ch % kHC) / split + (ch >= kHC ? per_owner : 0); };
  bool acc_ok = true;

  // One pass, except: a grouped-mode expert with many rows (the accumulator is reused tile after tile), and the two
  // row tiles of an MT == 2 CTA (two accumulators, both complete when accum_bar fires once).
  const int n_epi = MT == 2 ? (m_first + BM < m_end ? 2 : 1) : n_tiles_cta;
  for (int tj = 0; tj < n_epi; ++tj) {
  m0 = m_first + tj * tile_step;
  if constexpr (MT == 2) t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(tj * BN);
  const int grow = m0 + row;
  if (epi_warp) {
    pdl_wait();   // residual / C may be produced by the previous kernel
    if (MT == 1 || tj == 0) acc_ok = mbar_wait(accum_bar, tj & 1, p.status, kTimeoutAccum);
    tc_fence_after();
    if (threadIdx.x == 64) JS_TRACE(3);   // accumulator complete
  }

  if (split > 1) {
    if (alias) {   // every CTA of the cluster has finished its main loop (its stages are dead) before anyone pushes
      tc_fence_before();
      __syncthreads();
      cluster_sync();
    }
    // push every chunk of the partial tile into its owner's receive area (remote stores are
    // fire-and-forget; the cluster barrier below makes them visible)
    if (epi_warp && acc_ok) {
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + ch * 32, r);
        tmem_ld_wait();
        const uint32_t dst = map_to_cta(recv_addr, owner_of(ch)) +
                             static_cast<uint32_t>((z * slots_per_src + local_of(ch)) * 16384 + row * 4);
#pragma unroll
        for (int j = 0; j < 32; ++j) st_dsmem_f32(dst + j * (BM * 4), __uint_as_float(r[j]));
      }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 64) JS_TRACE(4);   // partial tile pushed
    cluster_sync();
    if (threadIdx.x == 64) JS_TRACE(5);   // every peer's partial has landed here
  }

  if constexpr (EPI == EPI_TOPK) {
    // the few-rows path below synchronises the four epilogue warps with each other: all of them take it or none
    if (epi_warp) acc_ok = epi_bar_and(acc_ok);
  }
  if (epi_warp && acc_ok) {
    const float* recv = reinterpret_cast<const float*>(smem + (alias ? 0 : S::kTiles));
    // fetch 32 consecutive accumulator columns of this thread's row, reduced over the K split
    auto load_chunk = [&](int c0, float* v) {
      if (split == 1) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
        const int lo = local_of(c0 >> 5);
        for (int src = 0; src < split; ++src) {   // fixed source order: deterministic sum
          const float* base = recv + (src * slots_per_src + lo) * 4096 + row;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += base[j * BM];
        }
      }
      if constexpr (FP4) {
        const float alpha = grow < m_end ? p.row_scale[grow] * p.w_scale : 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= alpha;
      }
    };

    if constexpr (EPI == EPI_EP_COMBINE) {
      // Expert-parallel combine fused into the experts' down projection: each output row is scaled
      // by its routing weight and stored into every rank's (token, choice) pair buffer over NVLink;
      // one release-increment per CTA and rank lets the finishing kernel know when all experts of
      // all ranks have delivered.
      // Each 32-column chunk is staged in shared memory so that four neighbouring lanes store one row's 64
      // contiguous bytes: NVLink sees a quarter of the write transactions of a store per lane and row.
      uint8_t* stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 15) & ~uintptr_t(15));
      const int et = threadIdx.x - 64;
      const float wgt = grow < m_end ? p.row_weight[grow] : 0.f;
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        load_chunk(c0, v);
        const int gc = n0 + c0;
        epi_barrier();
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 pk;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(v[8 * t + 2 * u] * wgt, v[8 * t + 2 * u + 1] * wgt);
          *reinterpret_cast<uint4*>(stage + row * 64 + ((t ^ ((row >> 1) & 3)) << 4)) = pk;
        }
        epi_barrier();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int piece = et + 128 * j, prow = piece >> 2, part = piece & 3;
          const int gr = m0 + prow, pc = gc + part * 8;
          if (gr >= m_end || pc >= p.N) continue;
          const uint4 d = *reinterpret_cast<const uint4*>(stage + prow * 64 + ((part ^ ((prow >> 1) & 3)) << 4));
          if (p.row_meta != nullptr) {
            const int2 m = p.row_meta[gr];
            if (m.x < 0 || m.x >= p.world) continue;
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peer_pairs[m.x]) +
                                      ((static_cast<size_t>(m.y) * p.N + pc) >> 1);
            asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(d.x), "r"(1u), "r"(d.y), "r"(1u) : "memory");
            asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "r"(d.z), "r"(1u), "r"(d.w), "r"(1u) : "memory");
            continue;
          }
          const size_t off = static_cast<size_t>(p.row_pair[gr]) * p.N + pc;
          for (int r = 0; r < p.world; ++r) *reinterpret_cast<uint4*>(p.peer_pairs[r] + off) = d;
        }
      }
      epi_barrier();
      if (threadIdx.x == 64 && p.row_meta == nullptr) {      // one release at system scope after the CTA barrier publishes every thread's stores
        __threadfence_system();
        for (int r = 0; r < p.world; ++r) red_release_sys_add(p.peer_cnt[r], 1);
      }
    } else if constexpr (EPI == EPI_ALLREDUCE) {
      // Row-parallel GEMM fused with the tensor-parallel all-reduce (one shot): each finished
      // 32-column chunk of this rank's partial product is stored as bf16 straight into every
      // rank's receive buffer over NVLink, a per-CTA counter on each rank is bumped with release
      // semantics, and the CTA then waits (bounded) until all ranks' chunks have landed in ITS
      // buffer, sums them in rank order together with the residual and writes the output.  All
      // ranks add the same numbers in the same order, so the replicated result is bit-identical.
      const int fidx = (blockIdx.y * gridDim.x + blockIdx.x) * split + z;
      if (p.ar_push_only >= 2) {
        // Low-latency push: every pair of bf16 outputs travels in ONE 8-byte store together with a flag word,
        // so the receiver needs no fence, no counter and no extra round trip: it polls the cells themselves
        // (the finishing kernel) and zeroes them after use.  Receive buffer: (world, m_cap, N/2) cells of 8 bytes.
        // The chunk is staged in shared memory first so that neighbouring lanes store neighbouring bytes of one row:
        // NVLink then sees 128-byte writes (4 lanes x 32 bytes per row) instead of one small write per lane.
        uint8_t* stage = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 15) & ~uintptr_t(15));   // 8 KB behind the barriers
        const int et = threadIdx.x - 64;                                   // 0..127 among the epilogue threads
        for (int c0 = z * 32; c0 < BN; c0 += split * 32) {
          float v[32];
          load_chunk(c0, v);
          const int gc = n0 + c0;
          epi_barrier();                                                   // previous chunk's readers are done
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 pk;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(v[8 * t + 2 * u], v[8 * t + 2 * u + 1]);
            *reinterpret_cast<uint4*>(stage + row * 64 + ((t ^ ((row >> 1) & 3)) << 4)) = pk;
          }
          epi_barrier();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int piece = et + 128 * j, prow = piece >> 2, part = piece & 3;
            const int gr = m0 + prow, pc = gc + part * 8;
            if (gr >= p.M || pc >= p.N) continue;
            const uint4 d = *reinterpret_cast<const uint4*>(stage + prow * 64 + ((part ^ ((prow >> 1) & 3)) << 4));
            if (p.ar_push_only == 3) {
              // reduce-scatter form (two-shot all-reduce): columns [o * N/world, (o+1) * N/world) belong to rank o,
              // which receives only that slice from everybody: (world, m_cap, N/world) cells.  The bytes a rank
              // sends stay at one partial's worth however many ranks there are.
              const int nw = p.N / p.world, o = pc / nw;
              const size_t cell = ((static_cast<size_t>(p.rank) * p.m_cap + gr) * nw + (pc - o * nw)) >> 1;
              unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peer_recv[o]) + cell;
              asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(d.x), "r"(1u), "r"(d.y), "r"(1u) : "memory");
              asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "r"(d.z), "r"(1u), "r"(d.w), "r"(1u) : "memory");
              continue;
            }
            const size_t cell = ((static_cast<size_t>(p.rank) * p.m_cap + gr) * p.N + pc) >> 1;
            for (int r = 0; r < p.world; ++r) {
              unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peer_recv[r]) + cell;
              asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(d.x), "r"(1u), "r"(d.y), "r"(1u) : "memory");
              asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "r"(d.z), "r"(1u), "r"(d.w), "r"(1u) : "memory");
            }
          }
        }
      } else {
      for (int c0 = z * 32; c0 < BN; c0 += split * 32) {
        float v[32];
        load_chunk(c0, v);
        const int gc = n0 + c0;
        if (grow < p.M && gc < p.N) {
          uint4 pk[4];
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(pk);
#pragma unroll
          for (int t = 0; t < 16; ++t) o2[t] = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
          const size_t off = (static_cast<size_t>(p.rank) * p.m_cap + grow) * p.N + gc;
          for (int r = 0; r < p.world; ++r) {
            uint4* dst = reinterpret_cast<uint4*>(p.peer_recv[r] + off);
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (gc + 8 * t < p.N) dst[t] = pk[t];
          }
        }
      }
      epi_barrier();
      bool landed = true;
      if (threadIdx.x == 64) {
        // one release at system scope after the CTA barrier publishes every epilogue thread's stores
        __threadfence_system();
        for (int r = 0; r < p.world; ++r) red_release_sys_add(p.peer_flags[r] + fidx, 1);
        if (p.ar_push_only) {
          *reinterpret_cast<volatile int*>(tmem_slot + 1) = 0;
        } else {
        const int* mine = p.peer_flags[p.rank] + fidx;
        landed = false;
        for (uint32_t it = 0; it < (1u << 22); ++it) {
          if (ld_acquire_sys(mine) >= p.world) { landed = true; break; }
          __nanosleep(64);
        }
        if (!landed) report(p.status, kTimeoutPeer);
        *reinterpret_cast<volatile int*>(tmem_slot + 1) = landed ? 1 : 0;
        }
      }
      epi_barrier();
      landed = *reinterpret_cast<volatile int*>(tmem_slot + 1) != 0;
      if (landed) {
        const __nv_bfloat16* mine = p.peer_recv[p.rank];
        for (int c0 = z * 32; c0 < BN; c0 += split * 32) {
          const int gc = n0 + c0;
          if (grow >= p.M || gc >= p.N) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
          for (int src = 0; src < p.world; ++src) {
            const uint4* sp = reinterpret_cast<const uint4*>(mine + (static_cast<size_t>(src) * p.m_cap + grow) * p.N + gc);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (gc + 8 * t >= p.N) break;
              const uint4 rv = __ldcg(sp + t);     // written by a peer GPU: bypass L1
              const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(r2[u]);
                v[8 * t + 2 * u] += f.x;
                v[8 * t + 2 * u + 1] += f.y;
              }
            }
          }
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(grow) * p.ldc + gc;
          const __nv_bfloat16* res = p.residual ? p.residual + static_cast<size_t>(grow) * p.ldc + gc : nullptr;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (gc + 8 * t >= p.N) break;
            if (res) {
              const uint4 rv = *reinterpret_cast<const uint4*>(res + 8 * t);
              const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f = __bfloat1622float2(r2[u]);
                v[8 * t + 2 * u] += f.x;
                v[8 * t + 2 * u + 1] += f.y;
              }
            }
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(v[8 * t + 2 * u], v[8 * t + 2 * u + 1]);
            *reinterpret_cast<uint4*>(out + 8 * t) = ov;
          }
        }
      }
      epi_barrier();
      if (threadIdx.x == 64 && landed && !p.ar_push_only) p.peer_flags[p.rank][fidx] = 0;   // ready for this buffer's next turn
      }
    } else if constexpr (EPI == EPI_STORE || EPI == EPI_STORE_F32) {
      // 32-column chunks are dealt round-robin to the CTAs of the K-split cluster
      for (int c0 = z * 32; c0 < BN; c0 += split * 32) {
        float v[32];
        load_chunk(c0, v);
        const int gc = n0 + c0;
        if (grow < m_end && gc < p.N) {
          if constexpr (EPI == EPI_STORE_F32) {
            float* out = reinterpret_cast<float*>(p.C) + static_cast<size_t>(grow) * p.ldc + gc;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (gc + j < p.N) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(grow) * p.ldc + gc;
            const __nv_bfloat16* res = p.residual ? p.residual + static_cast<size_t>(grow) * p.ldc + gc : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (gc + j >= p.N) break;
              if (res) {
                uint4 rv = *reinterpret_cast<const uint4*>(res + j);
                const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  float2 f = __bfloat1622float2(r2[t]);
                  v[j + 2 * t] += f.x;
                  v[j + 2 * t + 1] += f.y;
                }
              }
              uint4 ov;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
              for (int t = 0; t < 4; ++t) o2[t] = __floats2bfloat162_rn(v[j + 2 * t], v[j + 2 * t + 1]);
              *reinterpret_cast<uint4*>(out + j) = ov;
            }
          }
        }
      }
    } else if constexpr (EPI == EPI_SWIGLU) {
      constexpr int HALF = BN / 2;
      for (int c0 = z * 32; c0 < HALF; c0 += split * 32) {
        float g[32], u[32];
        load_chunk(c0, g);
        load_chunk(HALF + c0, u);
        const int gc = n0 / 2 + c0;              // output column
        if (grow < m_end && gc < p.N / 2) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(grow) * p.ldc + gc;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 ov;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float a = g[j + 2 * t], b = g[j + 2 * t + 1];
              o2[t] = __floats2bfloat162_rn(a / (1.f + __expf(-a)) * u[j + 2 * t], b / (1.f + __expf(-b)) * u[j + 2 * t + 1]);
            }
            *reinterpret_cast<uint4*>(out + j) = ov;
          }
        }
      }
    } else if constexpr (EPI == EPI_ARGMAX) {
      float best = -INFINITY;
      int best_i = 0x7fffffff;
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        load_chunk(c0, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int gc = n0 + c0 + j;
          // compare the fp32 accumulators: rounding the logits to bf16 first would turn the many
          // near-ties of a 150k-entry vocabulary into exact ties decided by index order
          const float x = v[j];
          if (gc < p.N && x > best) { best = x; best_i = gc; }
        }
      }
      if (grow < p.M) {
        const size_t o = static_cast<size_t>(grow) * gridDim.x + bx;
        p.part_val[o] = best;
        p.part_idx[o] = best_i;
      }
    } else if (p.M <= 32) {
      // EPI_TOPK with at most 32 rows (a draft block): all valid rows sit in the lane quadrant of ONE warp, which
      // would run the whole epilogue alone.  That warp instead drops the tile's logits into shared memory (the
      // pipeline stages are dead by now), column-major so that a warp touches 32 consecutive floats, and all four
      // epilogue warps take 32 columns each of every row; the owner warp then merges the four sorted lists.
      float* buf = reinterpret_cast<float*>(smem);                 // [BN columns][32 rows]
      float* lst_v = buf + BN * 32;                                // [4 column groups][32 rows][8]
      int* lst_i = reinterpret_cast<int*>(lst_v + 4 * 32 * kTopK);
      static_assert(BN == 128, "four column groups of 32");
      float mx = -INFINITY, se = 0.f;
      if (quad == 0) {
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          load_chunk(c0, v);
          const int gc0 = n0 + c0;
          float cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (gc0 + j >= p.N) v[j] = -INFINITY;                  // a column past the vocabulary never enters
            cm = fmaxf(cm, v[j]);
          }
          if (cm != -INFINITY) {
            float cs = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) cs += __expf(v[j] - cm);  // exp(-inf) = 0 for the masked columns
            const float nm = fmaxf(mx, cm);
            se = (mx == -INFINITY ? 0.f : se * __expf(mx - nm)) + cs * __expf(cm - nm);
            mx = nm;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) buf[(c0 + j) * 32 + lane] = v[j];
        }
      }
      epi_bar_sync();
      float tv[kTopK];
      int ti[kTopK];
#pragma unroll
      for (int t = 0; t < kTopK; ++t) { tv[t] = -INFINITY; ti[t] = 0x7fffffff; }
      if (lane < p.M) {
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
          float cv = buf[(quad * 32 + j) * 32 + lane];
          int ci = n0 + quad * 32 + j;
#pragma unroll
          for (int t = 0; t < kTopK; ++t) {                        // columns ascend: "strictly larger" keeps the lower index first
            const bool up = cv > tv[t];
            const float sv = tv[t];
            const int si = ti[t];
            tv[t] = up ? cv : sv;
            ti[t] = up ? ci : si;
            cv = up ? sv : cv;
            ci = up ? si : ci;
          }
        }
      }
      if (quad != 0) {
#pragma unroll
        for (int t = 0; t < kTopK; ++t) {
          lst_v[(quad * 32 + lane) * kTopK + t] = tv[t];
          lst_i[(quad * 32 + lane) * kTopK + t] = ti[t];
        }
      }
      epi_bar_sync();
      if (quad == 0 && lane < p.M) {
        for (int c = 1; c < 4; ++c) {
          for (int e = 0; e < kTopK; ++e) {
            float cv = lst_v[(c * 32 + lane) * kTopK + e];
            int ci = lst_i[(c * 32 + lane) * kTopK + e];
            const bool enters = cv > tv[kTopK - 1] || (cv == tv[kTopK - 1] && ci < ti[kTopK - 1]);
            if (!enters) break;
#pragma unroll
            for (int t = 0; t < kTopK; ++t) {
              if (cv > tv[t] || (cv == tv[t] && ci < ti[t])) {
                const float sv = tv[t]; const int si = ti[t];
                tv[t] = cv; ti[t] = ci; cv = sv; ci = si;
              }
            }
          }
        }
        const size_t o = static_cast<size_t>(grow) * gridDim.x + bx;
#pragma unroll
        for (int t = 0; t < kTopK; ++t) { p.part_val[o * kTopK + t] = tv[t]; p.part_idx[o * kTopK + t] = ti[t]; }
        p.part_lse[o * 2] = mx;
        p.part_lse[o * 2 + 1] = se;
      }
    } else {  // EPI_TOPK: top-8 values + indices and (max, sum exp) over this tile's columns
      // One thread owns a row, and with a few valid rows (a 21-row draft block) one warp does all the work, so the
      // cost is the LENGTH of the dependent chains, not the instruction count.  The sorted insertion therefore runs
      // as four independent chains (columns j % 4, each with its own top-8) that the scheduler interleaves, merged
      // once at the end; the log-sum-exp takes a chunk maximum first and then 32 independent exponentials.
      // Order everywhere: larger value first, lower column index first among equal values.
      constexpr int kChains = 4;
      float tv[kChains][kTopK];
      int ti[kChains][kTopK];
#pragma unroll
      for (int c = 0; c < kChains; ++c)
#pragma unroll
        for (int t = 0; t < kTopK; ++t) { tv[c][t] = -INFINITY; ti[c][t] = 0x7fffffff; }
      float mx = -INFINITY, se = 0.f;
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        load_chunk(c0, v);
        const int gc0 = n0 + c0;
        float cm = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc0 + j < p.N) cm = fmaxf(cm, v[j]);
        if (cm != -INFINITY) {
          float cs = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (gc0 + j < p.N) cs += __expf(v[j] - cm);
          const float nm = fmaxf(mx, cm);
          se = (mx == -INFINITY ? 0.f : se * __expf(mx - nm)) + cs * __expf(cm - nm);
          mx = nm;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          constexpr int kLast = kTopK - 1;
          const int c = j & (kChains - 1);
          const int gc = gc0 + j;
          float cv = gc < p.N ? v[j] : -INFINITY;      // a column past the vocabulary never enters
          int ci = gc;
          (void)kLast;
          // Branch-free compare-exchange down the list (selects only), so the four chains interleave.  Within a
          // chain columns arrive in increasing order, so "strictly larger" keeps the lower index first.
#pragma unroll
          for (int t = 0; t < kTopK; ++t) {
            const bool up = cv > tv[c][t];
            const float sv = tv[c][t];
            const int si = ti[c][t];
            tv[c][t] = up ? cv : sv;
            ti[c][t] = up ? ci : si;
            cv = up ? sv : cv;
            ci = up ? si : ci;
          }
        }
      }
      // fold chains 1..3 into chain 0 (each list is sorted, so a chain is done at its first entry that cannot enter)
#pragma unroll
      for (int c = 1; c < kChains; ++c) {
#pragma unroll
        for (int e = 0; e < kTopK; ++e) {
          float cv = tv[c][e];
          int ci = ti[c][e];
          const bool enters = cv > tv[0][kTopK - 1] || (cv == tv[0][kTopK - 1] && ci < ti[0][kTopK - 1]);
          if (!enters) break;
#pragma unroll
          for (int t = 0; t < kTopK; ++t) {
            if (cv > tv[0][t] || (cv == tv[0][t] && ci < ti[0][t])) {
              const float sv = tv[0][t]; const int si = ti[0][t];
              tv[0][t] = cv; ti[0][t] = ci; cv = sv; ci = si;
            }
          }
        }
      }
      if (grow < p.M) {
        const size_t o = static_cast<size_t>(grow) * gridDim.x + bx;
#pragma unroll
        for (int t = 0; t < kTopK; ++t) { p.part_val[o * kTopK + t] = tv[0][t]; p.part_idx[o * kTopK + t] = ti[0][t]; }
        p.part_lse[o * 2] = mx;
        p.part_lse[o * 2 + 1] = se;
      }
    }
  }
  if (MT == 1 && tj + 1 < n_tiles_cta && epi_warp) {        // hand the accumulator back for the CTA's next row tile
    tc_fence_before();
    epi_barrier();
    if (threadIdx.x == 64) mbar_arrive(tmem_free);
  }
  }

  // ------------------------------------------------------------------ teardown
  if (threadIdx.x == 64) JS_TRACE(6);     // epilogue stores issued
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) JS_TRACE(7);      // kernel end
}

// ---------------------------------------------------------------------------- host side
constexpr int kGroupedSmallRows = 32;     // rows of the small activation box of grouped launches (GemmParams::a_small_rows)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols] with leading dimension ld (elements), box = [box_rows, 64]
static int make_map(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// 2-D packed-e2m1 matrix seen as bytes: [rows, row_bytes] with leading dimension ld_bytes, box = [box_rows, 128 bytes]
static int make_map_u8(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t row_bytes, uint64_t ld_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int BN, int EPI, int BUDGET_KB, bool FP4 = false, int MT = 1>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, const GemmParams& p, int split, bool pdl,
                       cudaStream_t stream, int groups = 0, int group_m_tiles = 0, const CUtensorMap* ta_small = nullptr) {
  using S = GemmSmem<BN, BUDGET_KB, FP4, MT>;
  static int configured[kMaxDevicesCached] = {};
  auto kern = gemm_bf16_kernel<BN, EPI, BUDGET_KB, FP4, MT>;
  if (MT != 1 && (split != 1 || groups > 0)) return -19;
  const int recv_total = recv_bytes(split, BN, EPI == EPI_SWIGLU);
  const int data_bytes = recv_aliases_stages(S::kTiles, recv_total) ? (S::kTiles > recv_total ? S::kTiles : recv_total)
                                                                     : S::kTiles + recv_total;
  const int smem_bytes = data_bytes + 1024 /*align slack*/ + 256 /*barriers*/ + ((EPI == EPI_ALLREDUCE || EPI == EPI_EP_COMBINE) ? 8192 + 64 : 0);
  if (smem_bytes > 227 * 1024) return -18;
  if (ensure_dyn_smem(kern, smem_bytes, configured) != 0) return -3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + BN - 1) / BN, (p.M + BM * MT - 1) / (BM * MT), split);
  if (groups > 0) cfg.gridDim = dim3((p.N + BN - 1) / BN, group_m_tiles, groups);   // z = expert, no K split
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = 1;
  attrs[na].val.clusterDim.y = 1;
  attrs[na].val.clusterDim.z = split;
  ++na;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if ((p.a_small_rows > 0) != (ta_small != nullptr)) return -19;
  return cudaLaunchKernelEx(&cfg, kern, ta, tw, ta_small ? *ta_small : ta, p) == cudaSuccess ? 0 : -4;
}

}  // namespace js

// C = A[M,K] * W[N,K]^T.  epi: 0 store(+residual) 1 swiglu 2 argmax partials 3 top-8 + lse partials 4 fp32 store.
// bn in {64,128,256} (SwiGLU also 192: 128 tiles of a 24576-wide gate/up fill one wave); split = K-split cluster size (1..4; store/swiglu only); deep selects the pipeline's
// shared-memory budget: 0 = 96 KB (two CTAs per SM), 2 = 128 KB, 1 = 192 KB (one CTA per SM), 3 = 192 KB with two
// 128-row tiles per CTA sharing each weight stage (bn 256, no split).
// Returns 0 or a negative code.
extern "C" int js_gemm_bf16(const void* A, const void* W, void* C, const void* residual, int M, int N, int K, int lda,
                            int ldw, int ldc, int epi, int bn, int split, int deep, float* part_val, int* part_idx,
                            float* part_lse, int* status, unsigned long long* trace, int pdl,
                            cudaStream_t stream) {
  using namespace js;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8)) return -10;           // TMA: 16-byte aligned rows
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  const int kb_total = (K + BK - 1) / BK;
  if (split < 1 || split > 8 || split > kb_total) return -12;
  if ((epi == EPI_ARGMAX || epi == EPI_TOPK) && split != 1) return -13;
  // SwiGLU: the (gate, up) chunk pairs are dealt to the CTAs of the K-split cluster; with more CTAs than pairs
  // (128-column tiles have two) the extra CTAs only contribute their partial products and own no output columns
  if (epi == EPI_SWIGLU && split > 4) return -14;
  if ((epi == EPI_STORE || epi == EPI_STORE_F32) && split > bn / 32) return -14;
  if ((epi == EPI_STORE || epi == EPI_SWIGLU) && (ldc % 8)) return -15;
  CUtensorMap ta, tw;
  if (make_map(&ta, A, M, K, lda, BM) || make_map(&tw, W, N, K, ldw, bn)) return -16;
  GemmParams p{M, N, K, ldc, C, reinterpret_cast<const __nv_bfloat16*>(residual), part_val, part_idx, part_lse, status, trace,
               nullptr, nullptr, 0, 1, 0, nullptr, nullptr, nullptr, nullptr, nullptr};
  p.m_fast = ((epi == EPI_ARGMAX || epi == EPI_TOPK) && M > BM) ? 1 : 0;
  if (deep == 3) {     // two row tiles per CTA (256 x 256 output per CTA, 192 KB pipeline): many-row GEMMs
    if (bn != 256 || split != 1) return -19;
    if (epi == EPI_STORE) return launch_gemm<256, EPI_STORE, 192, false, 2>(ta, tw, p, 1, pdl != 0, stream);
    if (epi == EPI_SWIGLU) return launch_gemm<256, EPI_SWIGLU, 192, false, 2>(ta, tw, p, 1, pdl != 0, stream);
    return -19;
  }
#define JS_CASE(BN_, EPI_)                                                                              \
  if (bn == BN_ && epi == EPI_)                                                                         \
    return deep == 2 ? launch_gemm<BN_, EPI_, 128>(ta, tw, p, split, pdl != 0, stream)   \
           : deep == 1 ? launch_gemm<BN_, EPI_, 192>(ta, tw, p, split, pdl != 0, stream)   \
                       : launch_gemm<BN_, EPI_, 96>(ta, tw, p, split, pdl != 0, stream);
  JS_CASE(64, EPI_STORE) JS_CASE(128, EPI_STORE) JS_CASE(256, EPI_STORE)
  JS_CASE(128, EPI_STORE_F32)
  JS_CASE(128, EPI_SWIGLU) JS_CASE(192, EPI_SWIGLU) JS_CASE(256, EPI_SWIGLU)
  JS_CASE(128, EPI_ARGMAX)
  JS_CASE(128, EPI_TOPK)
#undef JS_CASE
  return -17;
}

// Tensor-parallel row-parallel GEMM fused with the all-reduce: out = residual + sum over ranks of
// (A_rank[M,K_local] * W_rank[N,K_local]^T).  peer_recv / peer_flags are DEVICE arrays of `world`
// pointers (every rank's receive buffer (world, m_cap, N) bf16 and per-CTA flag counters, this
// rank's own included).  Every rank must call this with the same shapes, bn and split.
extern "C" int js_gemm_bf16_allreduce(const void* A, const void* W, void* C, const void* residual, int M, int N, int K,
                                      int lda, int ldw, int ldc, int split, void* const* peer_recv,
                                      int* const* peer_flags, int rank, int world, int m_cap, int n_flags,
                                      int* status, int pdl, int push_only, cudaStream_t stream) {
  using namespace js;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (ldc % 8) || (N % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  const int kb_total = (K + BK - 1) / BK;
  if (split < 1 || split > 4 || split > kb_total) return -12;
  if (M > m_cap || world < 1 || rank < 0 || rank >= world) return -19;
  const int ctas = ((N + 127) / 128) * ((M + BM - 1) / BM) * split;
  if (push_only < 2) {                                    // the cell modes use neither counters nor waits in the GEMM
    if (ctas > n_flags) return -20;
    if (push_only == 0 && ctas > (split > 1 ? 148 : 2 * 148)) return -21;   // CTAs that wait for peers must all be resident
  }
  if (push_only == 3 && (N % (8 * world)) != 0) return -23;
  CUtensorMap ta, tw;
  if (make_map(&ta, A, M, K, lda, BM) || make_map(&tw, W, N, K, ldw, 128)) return -16;
  GemmParams p{M, N, K, ldc, C, reinterpret_cast<const __nv_bfloat16*>(residual), nullptr, nullptr, nullptr, status,
               nullptr, reinterpret_cast<__nv_bfloat16* const*>(peer_recv), peer_flags, rank, world, m_cap,
               nullptr, nullptr, nullptr, nullptr, nullptr};
  p.ar_push_only = push_only;
  return split > 1 ? launch_gemm<128, EPI_ALLREDUCE, 128>(ta, tw, p, split, pdl != 0, stream)
                   : launch_gemm<128, EPI_ALLREDUCE, 96>(ta, tw, p, split, pdl != 0, stream);
}

// Grouped GEMM over `groups` experts in one launch.  A (total_rows, K) holds the rows sorted by expert,
// expert e owning rows group_off[e] .. group_off[e+1] (device array, groups+1 entries); W is the stacked
// (groups*N, K) weight; C (total_rows, N or N/2).  epi: 0 store, 1 swiglu (per-expert tile-interleaved
// gate/up), 6 expert-parallel combine (weighted rows pushed to every rank's pair buffer).
// max_rows_per_group bounds the row tiles launched per expert.
extern "C" int js_gemm_bf16_grouped(const void* A, const void* W, void* C, int total_rows, int N, int K, int lda,
                                    int ldw, int ldc, int epi, int groups, const int* group_off,
                                    int max_rows_per_group, const int* row_pair, const float* row_weight,
                                    void* const* peer_pairs, int* const* peer_cnt, int world, int* status, int pdl,
                                    cudaStream_t stream) {
  using namespace js;
  if (total_rows <= 0 || groups <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (N % 128)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  CUtensorMap ta, tw, ta_small;
  if (make_map(&ta, A, total_rows, K, lda, BM) || make_map(&tw, W, static_cast<uint64_t>(groups) * N, K, ldw, 128) ||
      make_map(&ta_small, A, total_rows, K, lda, kGroupedSmallRows))
    return -16;
  GemmParams p{total_rows, N, K, ldc, C, nullptr, nullptr, nullptr, nullptr, status, nullptr,
               nullptr, nullptr, 0, world, 0, group_off, row_pair, row_weight,
               reinterpret_cast<__nv_bfloat16* const*>(peer_pairs), peer_cnt};
  p.a_small_rows = kGroupedSmallRows;
  const int m_tiles = (max_rows_per_group + BM - 1) / BM;
  if (m_tiles < 1) return 0;
  if (epi == EPI_STORE) return launch_gemm<128, EPI_STORE, 96>(ta, tw, p, 1, pdl != 0, stream, groups, m_tiles, &ta_small);
  if (epi == EPI_SWIGLU) return launch_gemm<128, EPI_SWIGLU, 96>(ta, tw, p, 1, pdl != 0, stream, groups, m_tiles, &ta_small);
  if (epi == EPI_EP_COMBINE) {
    if (!row_pair || !row_weight || !peer_pairs || !peer_cnt) return -22;
    return launch_gemm<128, EPI_EP_COMBINE, 96>(ta, tw, p, 1, pdl != 0, stream, groups, m_tiles, &ta_small);
  }
  return -17;
}

// Experts' down projection of a token-sharded expert-parallel layer: grouped GEMM over this rank's receive slab
// whose epilogue returns every weighted output row to the rank that owns the token (see GemmParams::row_meta).
// A (slab_rows, K) rows grouped by local expert (group_off, groups + 1 entries), W (groups * N, K).
extern "C" int js_gemm_bf16_grouped_ep(const void* A, const void* W, int slab_rows, int N, int K, int lda, int ldw,
                                       int groups, const int* group_off, int max_rows_per_group, const void* row_meta,
                                       const float* row_weight, void* const* peer_pairs, int world, int* status,
                                       int pdl, cudaStream_t stream) {
  using namespace js;
  if (slab_rows <= 0 || groups <= 0) return 0;
  if ((K % 8) || (lda % 8) || (ldw % 8) || (N % 128)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -11;
  if (!row_meta || !row_weight || !peer_pairs || world < 1) return -22;
  CUtensorMap ta, tw, ta_small;
  if (make_map(&ta, A, slab_rows, K, lda, BM) || make_map(&tw, W, static_cast<uint64_t>(groups) * N, K, ldw, 128) ||
      make_map(&ta_small, A, slab_rows, K, lda, kGroupedSmallRows))
    return -16;
  GemmParams p{};
  p.a_small_rows = kGroupedSmallRows;
  p.M = slab_rows; p.N = N; p.K = K; p.ldc = N; p.status = status; p.world = world;
  p.group_off = group_off; p.row_weight = row_weight;
  p.peer_pairs = reinterpret_cast<__nv_bfloat16* const*>(peer_pairs);
  p.row_meta = reinterpret_cast<const int2*>(row_meta);
  const int m_tiles = (max_rows_per_group + BM - 1) / BM;
  if (m_tiles < 1) return 0;
  return launch_gemm<128, EPI_EP_COMBINE, 96>(ta, tw, p, 1, pdl != 0, stream, groups, m_tiles, &ta_small);
}

// NVFP4 GEMM: C[M,N] = (Aq * sfa * row_scale) * (Wq * sfw * w_scale)^T.  Aq (M, K/2) and Wq (N, K/2) hold two
// e2m1 codes per byte; sfa / sfw are the e4m3 block scales in 512-byte tiles of 128 rows x 4 blocks, row tiles
// outermost (sfa must cover ceil(M/128)*128 rows, sfw ceil(N/128)*128); row_scale has M floats.
// epi: 0 store(+residual), 1 swiglu, 4 fp32 store.  K % 256 == 0.
extern "C" int js_gemm_nvfp4(const void* Aq, const void* sfa, const float* row_scale, const void* Wq, const void* sfw,
                             float w_scale, void* C, const void* residual, int M, int N, int K, int lda_bytes,
                             int ldw_bytes, int ldc, int epi, int split, int* status, int pdl, cudaStream_t stream) {
  using namespace js;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 256) || (lda_bytes % 16) || (ldw_bytes % 16)) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(sfa) |
       reinterpret_cast<uintptr_t>(sfw)) & 15) return -11;
  if (split < 1 || split > 4 || split > K / 256) return -12;
  if (epi == EPI_SWIGLU && split > 2) return -14;
  if ((epi == EPI_STORE || epi == EPI_SWIGLU) && (ldc % 8)) return -15;
  if (!row_scale) return -22;
  CUtensorMap ta, tw;
  if (make_map_u8(&ta, Aq, M, K / 2, lda_bytes, BM) || make_map_u8(&tw, Wq, N, K / 2, ldw_bytes, 128)) return -16;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.status = status; p.world = 1;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfw = reinterpret_cast<const uint8_t*>(sfw);
  p.row_scale = row_scale; p.w_scale = w_scale;
#define JS_CASE4(EPI_)                                                                                   \
  if (epi == EPI_)                                                                                        \
    return split > 1 ? launch_gemm<128, EPI_, 128, true>(ta, tw, p, split, pdl != 0, stream)              \
                     : launch_gemm<128, EPI_, 160, true>(ta, tw, p, split, pdl != 0, stream);
  JS_CASE4(EPI_STORE) JS_CASE4(EPI_SWIGLU) JS_CASE4(EPI_STORE_F32)
#undef JS_CASE4
  return -17;
}

// Row-parallel NVFP4 GEMM fused with the tensor-parallel all-reduce (same protocol as js_gemm_bf16_allreduce).
extern "C" int js_gemm_nvfp4_allreduce(const void* Aq, const void* sfa, const float* row_scale, const void* Wq,
                                       const void* sfw, float w_scale, void* C, const void* residual, int M, int N,
                                       int K, int lda_bytes, int ldw_bytes, int ldc, int split, void* const* peer_recv,
                                       int* const* peer_flags, int rank, int world, int m_cap, int n_flags, int* status,
                                       int pdl, int push_only, cudaStream_t stream) {
  using namespace js;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 256) || (lda_bytes % 16) || (ldw_bytes % 16) || (ldc % 8) || (N % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(sfa) |
       reinterpret_cast<uintptr_t>(sfw)) & 15) return -11;
  if (split < 1 || split > 4 || split > K / 256) return -12;
  if (M > m_cap || world < 1 || rank < 0 || rank >= world || !row_scale) return -19;
  const int ctas = ((N + 127) / 128) * ((M + BM - 1) / BM) * split;
  if (push_only < 2) {
    if (ctas > n_flags) return -20;
    if (push_only == 0 && ctas > 148) return -21;           // CTAs that wait for peers must all be resident
  }
  if (push_only == 3 && (N % (8 * world)) != 0) return -23;
  CUtensorMap ta, tw;
  if (make_map_u8(&ta, Aq, M, K / 2, lda_bytes, BM) || make_map_u8(&tw, Wq, N, K / 2, ldw_bytes, 128)) return -16;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.status = status;
  p.peer_recv = reinterpret_cast<__nv_bfloat16* const*>(peer_recv); p.peer_flags = peer_flags;
  p.rank = rank; p.world = world; p.m_cap = m_cap;
  p.sfa = reinterpret_cast<const uint8_t*>(sfa); p.sfw = reinterpret_cast<const uint8_t*>(sfw);
  p.row_scale = row_scale; p.w_scale = w_scale;
  p.ar_push_only = push_only;
  return launch_gemm<128, EPI_ALLREDUCE, 128, true>(ta, tw, p, split, pdl != 0, stream);
}
