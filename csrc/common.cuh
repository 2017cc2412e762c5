// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM, clusters.
//
// Every wait in these kernels is bounded.  A wait that runs out records a code in the
// kernel's status word and returns false; the caller then leaves its role loop and walks
// to the common teardown (TMEM is released, cluster barriers are still joined), so a lost
// signal ends in an error the host can read instead of a hung GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

#define JS_DEVICE __device__ __forceinline__

namespace js {

// status codes written to the per-launch status word (0 = ok)
enum : int {
  kOk = 0,
  kTimeoutFull = 1,     // consumer waited for a TMA stage that never arrived
  kTimeoutEmpty = 2,    // producer waited for a stage that was never released
  kTimeoutAccum = 3,    // epilogue waited for the accumulator
  kTimeoutPeer = 4,     // waited for a flag another GPU should have written
  kBadSlot = 5,         // a slot / page index fell outside the pool
  kBadNode = 6,         // a tree index fell outside the node range
  kTimeoutEpCounts = 7,   // expert-parallel dispatch: a rank's per-expert counts never arrived
  kTimeoutEpArrive = 8,   // expert-parallel dispatch: a source rank's rows never arrived
  kTimeoutCellsReduce = 9,    // all-reduce tail, reduce step (or the expert-parallel combine): partial cells missing
  kTimeoutCellsGather = 10,   // all-reduce tail, gather step: a slice owner's result cells missing
  kTimeoutTopk = 11,      // vocabulary-parallel top-k: a rank's record never arrived
  kEpOverflow = 12,       // more rows for one expert (or one rank) than the receive slab / the grouped launch covers
};

constexpr uint32_t kSpinLimit = 1u << 20;  // polls; each try_wait already suspends for a while

JS_DEVICE uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

JS_DEVICE void report(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

// ---------------------------------------------------------------- host: per-device launch attributes
// cudaFuncSetAttribute applies to the CURRENT device only, so the "already configured" cache of a kernel is one
// slot per device (a process may drive several GPUs).  `slots` is a zero-initialised static array of
// kMaxDevicesCached ints owned by the caller; the value is the largest dynamic shared-memory size set so far.
constexpr int kMaxDevicesCached = 64;
template <typename Kern>
inline int ensure_dyn_smem(Kern kern, int bytes, int* slots) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -3;
  if (dev < 0 || dev >= kMaxDevicesCached) {   // beyond the cache: set it every time
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -3;
  }
  if (bytes > __atomic_load_n(&slots[dev], __ATOMIC_ACQUIRE)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -3;
    __atomic_store_n(&slots[dev], bytes, __ATOMIC_RELEASE);
  }
  return 0;
}

// ---------------------------------------------------------------- mbarrier
JS_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
JS_DEVICE void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
JS_DEVICE void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

JS_DEVICE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
JS_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
JS_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test (try_wait may suspend the thread for microseconds before answering "not yet").
JS_DEVICE bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false on timeout (status gets `code`).
JS_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  report(status, code);
  return false;
}

// ---------------------------------------------------------------- TMA
JS_DEVICE void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load, completion counted on `bar` (x = innermost coordinate, must be 16-byte aligned in bytes)
JS_DEVICE void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, bytes a multiple of 16).
JS_DEVICE void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
JS_DEVICE void tmem_alloc(uint32_t* smem_result, uint32_t cols) {  // whole warp, cols = power of two >= 32
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
JS_DEVICE void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
JS_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t cols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
JS_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
JS_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
JS_DEVICE void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
JS_DEVICE void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp reads lane (base_lane + t).
JS_DEVICE void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
JS_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major bf16 tile stored as rows of 128 bytes
// (64 elements) with the 128-byte swizzle TMA produces: groups of 8 rows are 1024 bytes
// apart (stride byte offset), the leading offset is unused for swizzled K-major tiles.
JS_DEVICE uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset (ignored) = 1
  d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset = 1024 B
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                     // layout: 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M x N tile.
JS_DEVICE constexpr uint32_t umma_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ---- NVFP4 (block-scaled e2m1) -------------------------------------------------------------
// Shared-memory descriptor of one 512-byte scale tile (32 rows of 16 bytes, unswizzled; groups of
// 8 rows are 128 bytes apart).
JS_DEVICE uint64_t umma_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;              // stride byte offset = 128 B
  d |= static_cast<uint64_t>(1) << 46;                     // descriptor version (Blackwell)
  return d;
}
// Copy 32 rows x 16 bytes from shared memory into 4 tensor-memory columns, replicated to the four
// 32-lane groups (the placement block-scaled MMAs read their scale factors from).  One thread issues.
JS_DEVICE void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Instruction descriptor: e2m1 x e2m1 with e4m3 scales per 16 elements -> fp32, K-major operands.
JS_DEVICE constexpr uint32_t umma_idesc_nvfp4(int M, int N) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
// D[tmem] (+)= (A * SFA) * (B * SFB), K = 64 per instruction; sfa / sfb are tensor-memory addresses.
JS_DEVICE void umma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}

// ---------------------------------------------------------------- clusters
JS_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
JS_DEVICE void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
JS_DEVICE void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
JS_DEVICE void cluster_sync() { cluster_arrive(); cluster_wait(); }
// Address of `smem_addr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster.
JS_DEVICE uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
JS_DEVICE float ld_dsmem_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

JS_DEVICE void st_dsmem_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
JS_DEVICE void st_dsmem_v4(uint32_t cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
JS_DEVICE float4 ld_dsmem_v4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
  return v;
}

// ---------------------------------------------------------------- programmatic dependent launch
JS_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Named barrier 1 over 128 threads (the four epilogue warps of a GEMM CTA), plain and with an AND reduction.
JS_DEVICE void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
JS_DEVICE bool epi_bar_and(bool pred) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\tselp.s32 %0, 1, 0, p;\n\t}"
      : "=r"(out) : "r"(static_cast<int>(pred)) : "memory");
  return out != 0;
}
JS_DEVICE void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- small math
JS_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
JS_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace js
