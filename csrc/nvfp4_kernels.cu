// On-the-fly NVFP4 quantisation of activations, optionally fused with the RMSNorm that produces them.
//
// One CTA per row.  The row is held in registers (16 elements = one scale block per thread and step):
//   outer  = amax(row) / (6 * 448)                       fp32, one per row
//   scale  = e4m3(min(amax(block) / 6 / outer, 448))     one per 16 elements
//   code   = e2m1(x / (float(scale) * outer))            round to nearest even, saturating
// Codes are packed two per byte (even element in the low nibble); scales are written straight in the
// 512-byte tile order the block-scaled tensor-core GEMM copies to tensor memory:
//   tile (row / 128, block / 4), byte (row % 32) * 16 + (row / 32 % 4) * 4 + block % 4.
// The arithmetic (two divisions for the scale, one for the value) is kept in the same order as the
// PyTorch quantiser, so both produce identical bytes.
#include "common.cuh"

#include <cuda_fp8.h>

namespace js {

constexpr int kQuantThreads = 256;
constexpr int kQuantMaxSteps = 4;          // K <= 256 * 16 * 4 = 16384

JS_DEVICE float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < kQuantThreads / 32; ++i) r = fmaxf(r, red[i]);
  __syncthreads();
  return r;
}
JS_DEVICE float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kQuantThreads / 32; ++i) r += red[i];
  __syncthreads();
  return r;
}

// two fp32 -> one byte of two e2m1 codes (lo in bits 0..3, hi in bits 4..7)
JS_DEVICE uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t out;
  asm volatile(
      "{\n\t.reg .b8 b;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\t"
      "cvt.u16.u8 %0, b;\n\t}"
      : "=h"(out)
      : "f"(lo), "f"(hi));
  return out;
}

__global__ void __launch_bounds__(kQuantThreads)
quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ norm_w, float eps,
                   int K, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf, float* __restrict__ outer_out,
                   __nv_bfloat16* __restrict__ norm_out, int ld_norm) {
  __shared__ float red[kQuantThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int nblk = K / 16;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  float v[kQuantMaxSteps][16];
  float ss = 0.f;
#pragma unroll
  for (int s = 0; s < kQuantMaxSteps; ++s) {
    const int b = threadIdx.x + s * kQuantThreads;
    if (b < nblk) {
      const uint4 a0 = *reinterpret_cast<const uint4*>(xr + b * 16);
      const uint4 a1 = *reinterpret_cast<const uint4*>(xr + b * 16 + 8);
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&a0);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&a1);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f0 = __bfloat1622float2(h0[t]), f1 = __bfloat1622float2(h1[t]);
        v[s][2 * t] = f0.x; v[s][2 * t + 1] = f0.y;
        v[s][8 + 2 * t] = f1.x; v[s][8 + 2 * t + 1] = f1.y;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) ss += v[s][j] * v[s][j];
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[s][j] = 0.f;
    }
  }
  if (norm_w != nullptr) {
    // RMSNorm in fp32, rounded to bf16 exactly as the stand-alone norm kernel stores it
    const float rstd = rsqrtf(block_reduce_sum(ss, red) / static_cast<float>(K) + eps);
#pragma unroll
    for (int s = 0; s < kQuantMaxSteps; ++s) {
      const int b = threadIdx.x + s * kQuantThreads;
      if (b < nblk) {
        const uint4 w0 = *reinterpret_cast<const uint4*>(norm_w + b * 16);
        const uint4 w1 = *reinterpret_cast<const uint4*>(norm_w + b * 16 + 8);
        const __nv_bfloat16* wh0 = reinterpret_cast<const __nv_bfloat16*>(&w0);
        const __nv_bfloat16* wh1 = reinterpret_cast<const __nv_bfloat16*>(&w1);
        uint4 o[2];
        __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(o);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float wv = __bfloat162float(j < 8 ? wh0[j] : wh1[j - 8]);
          const __nv_bfloat16 y = __float2bfloat16_rn(v[s][j] * rstd * wv);
          oh[j] = y;
          v[s][j] = __bfloat162float(y);
        }
        if (norm_out != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(norm_out + static_cast<size_t>(row) * ld_norm + b * 16);
          dst[0] = o[0];
          dst[1] = o[1];
        }
      }
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int s = 0; s < kQuantMaxSteps; ++s)
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[s][j]));
  amax = block_reduce_max(amax, red);
  const float outer = fmaxf(amax / (6.0f * 448.0f), 1e-30f);
  if (threadIdx.x == 0) outer_out[row] = outer;
  const size_t sf_tile_row = static_cast<size_t>(row / 128) * (K / 64) * 512;
  const int sf_in_tile = (row % 32) * 16 + ((row / 32) % 4) * 4;
#pragma unroll
  for (int s = 0; s < kQuantMaxSteps; ++s) {
    const int b = threadIdx.x + s * kQuantThreads;
    if (b >= nblk) continue;
    float bmax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) bmax = fmaxf(bmax, fabsf(v[s][j]));
    const float want = fminf(bmax / 6.0f / outer, 448.0f);
    const __nv_fp8_e4m3 sc8(want);
    const float scf = static_cast<float>(sc8) * outer;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      const float q0 = scf > 0.f ? v[s][j] / scf : 0.f;
      const float q1 = scf > 0.f ? v[s][j + 1] / scf : 0.f;
      w[j / 8] |= cvt_e2m1x2(q0, q1) << (8 * ((j / 2) % 4));
    }
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (K / 2) + b * 8) = make_uint2(w[0], w[1]);
    sf[sf_tile_row + static_cast<size_t>(b / 4) * 512 + sf_in_tile + (b % 4)] = sc8.__x;
  }
}

}  // namespace js

// x (M, K) bf16 -> packed (M, K/2), sf (ceil(M/128) * K/64 * 512 bytes, tile order), outer (M) fp32.
// norm_w != nullptr: quantise rmsnorm(x) * norm_w instead (norm_out, if given, also receives the bf16 norm).
// K % 64 == 0, K <= 16384, ldx % 8 == 0.
extern "C" int js_quant_nvfp4(const void* x, int ldx, const void* norm_w, float eps, int M, int K, void* packed, void* sf,
                              float* outer, void* norm_out, int ld_norm, int pdl, cudaStream_t stream) {
  using namespace js;
  if (M <= 0) return 0;
  if ((K % 64) || K > kQuantThreads * 16 * kQuantMaxSteps || (ldx % 8) || (norm_out && (ld_norm % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(norm_w) |
       reinterpret_cast<uintptr_t>(norm_out)) & 15) return -11;
  cudaLaunchConfig_t c = {};
  c.gridDim = dim3(M);
  c.blockDim = dim3(kQuantThreads);
  c.stream = stream;
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  c.attrs = &a;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, quant_nvfp4_kernel, reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                            reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, K, reinterpret_cast<uint8_t*>(packed),
                            reinterpret_cast<uint8_t*>(sf), outer, reinterpret_cast<__nv_bfloat16*>(norm_out), ld_norm) ==
                 cudaSuccess
             ? 0
             : -4;
}
