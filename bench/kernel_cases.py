"""Small stand-alone kernel cases for profiling (one kernel family per case, a few launches).

    python bench/kernel_cases.py gemm        # the four decoder GEMM shapes of Qwen3-8B at 128 rows
    python bench/kernel_cases.py attention   # paged tree attention, 128 nodes over a 1.5k-token prefix
    python bench/kernel_cases.py lm_head     # vocabulary GEMM with the argmax epilogue
    python bench/kernel_cases.py nvfp4       # activation quantiser + block-scaled GEMM on the same four shapes

Each case holds well under a few GB on the device and launches its kernel a handful of times, so a
profiler capture of it ends by itself.
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from jetspec_b200.ops import cuda_ext as X  # noqa: E402


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def case_gemm(reps: int = 2):
    M, H, I = 128, 4096, 12288
    x, a = bf(M, H), bf(M, I)
    w = {"qkv": bf(6144, H, scale=0.02), "o": bf(H, H, scale=0.02), "gu": bf(2 * I, H, scale=0.02),
         "down": bf(H, I, scale=0.02)}
    res = bf(M, H)
    for _ in range(reps):
        X.gemm(x, w["qkv"])
        X.gemm(x, w["o"], out=res, residual=res)
        X.gemm(x, w["gu"], epi=X.EPI_SWIGLU)
        X.gemm(a, w["down"], out=res, residual=res)
    torch.cuda.synchronize()


def case_nvfp4(reps: int = 2):
    from jetspec_b200.models.nvfp4 import quantize_nvfp4
    M, H, I = 128, 4096, 12288
    x, a = bf(M, H), bf(M, I)
    w = {k: quantize_nvfp4(v.float()) for k, v in
         {"qkv": bf(6144, H, scale=0.02), "o": bf(H, H, scale=0.02), "gu": bf(2 * I, H, scale=0.02),
          "down": bf(H, I, scale=0.02)}.items()}
    res = bf(M, H)
    for _ in range(reps):
        xq, aq = X.quant_nvfp4(x), X.quant_nvfp4(a)
        X.gemm_nvfp4(xq, w["qkv"])
        X.gemm_nvfp4(xq, w["o"], out=res, residual=res)
        X.gemm_nvfp4(xq, w["gu"], epi=X.EPI_SWIGLU)
        X.gemm_nvfp4(aq, w["down"], out=res, residual=res)
    torch.cuda.synchronize()


def case_lm_head(reps: int = 2):
    h, w = bf(128, 4096), bf(151936, 4096, scale=0.02)
    for _ in range(reps):
        X.lm_head_argmax(h, w)
    torch.cuda.synchronize()


def case_attention(reps: int = 2):
    Hq, Hkv, D, S, past, n = 32, 8, 128, 4096, 1536, 128
    kp, vp, q = bf(Hkv, S, D), bf(Hkv, S, D), bf(n, Hq, D)
    slot_map = torch.randperm(S, device="cuda").to(torch.int32).view(1, S)
    rows = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    pl = torch.tensor([past], dtype=torch.int32, device="cuda")
    bits = torch.zeros(n, 4, dtype=torch.int32, device="cuda")
    for i in range(n):   # a chain: node i sees nodes 0..i
        for j in range(i + 1):
            bits[i, j >> 5] |= (1 << (j & 31)) if (j & 31) < 31 else -(1 << 31)
    for _ in range(reps):
        X.paged_tree_attention(q, kp, vp, slot_map, rows, cu, pl, bits, 1 / math.sqrt(D), False, n, max_keys=S)
    torch.cuda.synchronize()


if __name__ == "__main__":
    X.load()
    {"gemm": case_gemm, "lm_head": case_lm_head, "attention": case_attention, "nvfp4": case_nvfp4}[sys.argv[1]]()
    X.check_status("cuda")
    print("ok")
