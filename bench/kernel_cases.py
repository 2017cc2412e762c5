"""Small stand-alone kernel cases for profiling (one kernel family per case, a few launches).

    python bench/kernel_cases.py gemm        # the four decoder GEMM shapes of Qwen3-8B at 128 rows
    python bench/kernel_cases.py gemm_rows2048   # the same shapes at 2048 rows (batched verify / prefill tiles)
    python bench/kernel_cases.py attention   # paged tree attention, 128 nodes over a 1.5k-token prefix
    python bench/kernel_cases.py lm_head     # vocabulary GEMM with the argmax epilogue
    python bench/kernel_cases.py nvfp4       # activation quantiser + block-scaled GEMM on the same four shapes
    python bench/kernel_cases.py round_small # RMSNorm, norm+RoPE+KV scatter, draft top-k, tree build, accept+commit, KV compaction
    python bench/kernel_cases.py collectives # the fused all-reduce tail + RMSNorm and the expert-parallel dispatch, with a world of ONE
                                             # rank (every "peer" buffer is this GPU's own): the kernels' own cost without NVLink

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


def case_gemm_rows2048(reps: int = 2):
    """The same four shapes at 2048 rows (16 requests x 128 tree nodes, or a prefill chunk), picked configurations:
    256-column tiles, two row tiles per CTA for o_proj / down_proj, 256-interleaved gate/up."""
    M, H, I = 2048, 4096, 12288
    x, a = bf(M, H), bf(M, I)
    g, u = bf(I, H, scale=0.02), bf(I, H, scale=0.02)
    w = {"qkv": bf(6144, H, scale=0.02), "o": bf(H, H, scale=0.02), "gu": X.interleave_gate_up(g, u, 256),
         "down": bf(H, I, scale=0.02)}
    del g, u
    res = bf(M, H)
    for _ in range(reps):
        X.gemm(x, w["qkv"])
        X.gemm(x, w["o"], out=res, residual=res)
        X.gemm(x, w["gu"], epi=X.EPI_SWIGLU, bn=256, split=1, deep=0)
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


def case_round_small(reps: int = 2):
    """The small kernels of a decode round at Qwen3-8B sizes: RMSNorm, per-head norm + RoPE + KV scatter, the
    draft head's vocabulary top-k (GEMM epilogue + merge), device tree build, accept + commit, KV compaction."""
    import ctypes
    import random
    lib = X.load()
    dev = "cuda"
    Hq, Hkv, D, H, S, T = 32, 8, 128, 4096, 8192, 128
    x, wn = bf(T, H), bf(H)
    qkv = bf(T, (Hq + 2 * Hkv) * D)
    qn, kn = bf(D), bf(D)
    kp, vp, q = bf(Hkv, S, D), bf(Hkv, S, D), torch.empty(T, Hq, D, dtype=torch.bfloat16, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    past = 1536
    positions = i32([past + (i % 20) for i in range(T)])
    slots = torch.randperm(S, device=dev)[:T].to(torch.int32)
    freq = X.inv_freq(D, 1e6, dev)
    h21, wv = bf(21, H), bf(151936, H, scale=0.02)
    rng = random.Random(0)
    Dd, K, NB, W, max_len = 20, 7, 128, 4, 4096
    tk = i32([[rng.randrange(151936) for _ in range(K)] for _ in range(Dd)])
    lp = torch.tensor([sorted((-rng.random() * 4 for _ in range(K)), reverse=True) for _ in range(Dd)],
                      dtype=torch.float32, device=dev)
    caps = i32([K] * Dd)
    committed = torch.zeros(max_len, dtype=torch.int32, device=dev)
    slot_row = torch.randperm(max_len, device=dev).to(torch.int32)
    o = {k: torch.zeros(NB, dtype=torch.int32, device=dev) for k in ("tok", "par", "dep", "pos", "slot")}
    bits = torch.zeros(NB, W, dtype=torch.int32, device=dev)
    zero, eos = i32([0]), i32([-1])
    path_idx, result = torch.zeros(64, dtype=torch.int32, device=dev), torch.zeros(64, dtype=torch.int32, device=dev)
    st = X.status_word(dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    keep = i32([0, 3, 9, 17, 40])
    for _ in range(reps):
        X.rmsnorm(x, wn, 1e-6)
        X.qkv_post(qkv, qn, kn, positions, slots, freq, q, kp, vp, Hq, Hkv, 1e-6)
        X.lm_head_topk_logprobs(h21, wv, K)
        state = i32([past, 0, 0, 0, 0, 0, 0, 0])
        s = X._stream()
        X._check(lib.js_tree_build(p(tk), p(lp), p(caps), Dd, K, 128, NB, W, p(committed), p(state), p(slot_row), p(zero),
                                   max_len, p(o["tok"]), p(o["par"]), p(o["dep"]), p(o["pos"]), p(o["slot"]), p(bits),
                                   p(st), 0, s), "js_tree_build")
        greedy = o["tok"].roll(-1).contiguous()          # node i+1's token as the target's pick at node i
        X._check(lib.js_tree_accept_commit(p(o["tok"]), p(o["par"]), p(o["dep"]), p(greedy), NB, p(state), p(slot_row),
                                           p(zero), max_len, p(committed), max_len, p(eos), 1, 1 << 20, p(path_idx),
                                           p(result), p(st), 0, s), "js_tree_accept_commit")
        X.kv_compact(kp[:, :4096].contiguous(), vp[:, :4096].contiguous(), past, keep)
    torch.cuda.synchronize()


def case_collectives(reps: int = 3):
    """The communication kernels on one GPU: a process group of one rank, so every push lands in this GPU's own
    buffers.  Row-parallel o_proj / down_proj with the reduce-scatter epilogue + the finishing kernel that reduces,
    gathers and applies the next RMSNorm (128 rows), and one token-sharded expert-parallel layer of the
    Qwen3-30B-A3B geometry on 128 tokens (count exchange, dispatch, grouped GEMMs, combine + norm)."""
    import torch.distributed as dist
    from jetspec_b200.parallel import TensorParallel, TokenShardedEP
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29761")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    tp = TensorParallel(None, m_cap=128, n_max=4096)
    M, H, I = 128, 4096, 12288
    a, m = bf(M, H), bf(M, I)
    wo, wd, nw = bf(H, H, scale=0.02), bf(H, I, scale=0.02), bf(H)
    x, h = bf(M, H), torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    for _ in range(reps):
        tp.gemm_allreduce(a, wo, x, residual=x, norm_w=nw, norm_out=h)
        tp.gemm_allreduce(m, wd, x, residual=x, norm_w=nw, norm_out=h)
    torch.cuda.synchronize()
    E, He, Ie, k, T = 128, 2048, 768, 8, 128
    ep = TokenShardedEP(None, E, k, He, max_tokens=T)
    gate, wgu, wdn = bf(E, He, scale=0.5), bf(E, 2 * Ie, He, scale=0.03), bf(E, He, Ie, scale=0.03)
    gu_l, dn_l = ep.shard(wgu, wdn)
    xe, hn, nwe = bf(T, He), bf(T, He), bf(He)
    out, h2 = torch.empty_like(xe), torch.empty_like(xe)
    for _ in range(reps):
        ep.moe_layer(xe, hn, gate, gu_l, dn_l, True, out=out, norm_w=nwe, norm_out=h2)
    torch.cuda.synchronize()
    X.check_status("cuda")
    ep.close()
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    X.load()
    {"gemm": case_gemm, "gemm_rows2048": case_gemm_rows2048, "lm_head": case_lm_head, "attention": case_attention, "nvfp4": case_nvfp4,
     "round_small": case_round_small, "collectives": case_collectives}[sys.argv[1]]()
    X.check_status("cuda")
    print("ok")
