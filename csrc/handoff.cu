// Target <-> draft-GPU handoff primitives (the draft head lives on its own GPU).
// (The reference keeps the head on the target's device, jetspec/draft_head_adapter.py:54,73,129; no counterpart there.)
//
// The target's tapped hidden rows are written into the drafter GPU's buffer directly by the
// layer-epilogue copy kernel (its destination is simply a peer address).  What remains is small
// control traffic, done here with peer stores: a few words (accepted path, anchor token, counts;
// or the drafted top-k back to the target) followed by a release-store of a round number.  Both
// sides replay CUDA graphs, so round numbers live in device memory and are advanced by the
// kernels themselves.  Waits are bounded and report through the status word.
#include "common.cuh"

namespace js {

// dst (peer or local) <- src, n 32-bit words
__global__ void push_words_kernel(const int* src, int* dst, int n) {
  pdl_launch_dependents();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// *epoch += 1 and publish it at the peer's flag after everything this stream wrote before
__global__ void flag_push_kernel(int* peer_flag, int* epoch) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    const int v = *epoch + 1;
    *epoch = v;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flag), "r"(v) : "memory");
  }
}

// wait until the local flag reaches *epoch + 1, then advance *epoch
__global__ void flag_wait_kernel(const int* flag, int* epoch, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    const int want = *epoch + 1;
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 24); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v >= want) { ok = true; break; }
      __nanosleep(100);
    }
    if (!ok) report(status, kTimeoutPeer);
    *epoch = want;
  }
}

// drafter side: header = [n_new, anchor_token, done]; state uses the round-state layout
__global__ void draft_apply_header_kernel(const int* header, int* state, int* committed) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    state[2] = header[0];      // ST_NEW: context rows to append
    state[0] = 0;              // ST_PAST: the anchor sits at committed[0]
    committed[0] = header[1];
    state[3] = header[2];      // ST_DONE
  }
}

// target side: header <- [n_new, last committed token, done] from the round state
__global__ void make_header_kernel(const int* state, const int* committed, int* header) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    header[0] = state[2];
    header[1] = committed[state[0]];
    header[2] = state[3];
  }
}


}  // namespace js

#define JS_SMALL_LAUNCH(kern, blocks, threads, ...)                                     \
  do {                                                                                  \
    cudaLaunchConfig_t c = {};                                                          \
    c.gridDim = dim3(blocks);                                                           \
    c.blockDim = dim3(threads);                                                         \
    c.stream = stream;                                                                  \
    cudaLaunchAttribute a;                                                              \
    a.id = cudaLaunchAttributeProgrammaticStreamSerialization;                          \
    a.val.programmaticStreamSerializationAllowed = 1;                                   \
    c.attrs = &a;                                                                       \
    c.numAttrs = pdl ? 1 : 0;                                                           \
    return cudaLaunchKernelEx(&c, kern, __VA_ARGS__) == cudaSuccess ? 0 : -4;           \
  } while (0)

extern "C" int js_push_words(const int* src, int* dst, int n, int pdl, cudaStream_t stream) {
  if (n <= 0) return 0;
  JS_SMALL_LAUNCH(js::push_words_kernel, (n + 255) / 256 > 64 ? 64 : (n + 255) / 256, 256, src, dst, n);
}
extern "C" int js_flag_push(int* peer_flag, int* epoch, int pdl, cudaStream_t stream) {
  JS_SMALL_LAUNCH(js::flag_push_kernel, 1, 32, peer_flag, epoch);
}
extern "C" int js_flag_wait(const int* flag, int* epoch, int* status, int pdl, cudaStream_t stream) {
  JS_SMALL_LAUNCH(js::flag_wait_kernel, 1, 32, flag, epoch, status);
}
extern "C" int js_draft_apply_header(const int* header, int* state, int* committed, int pdl, cudaStream_t stream) {
  JS_SMALL_LAUNCH(js::draft_apply_header_kernel, 1, 32, header, state, committed);
}
extern "C" int js_make_header(const int* state, const int* committed, int* header, int pdl, cudaStream_t stream) {
  JS_SMALL_LAUNCH(js::make_header_kernel, 1, 32, state, committed, header);
}
