"""Fused compute+collective kernels against their NCCL twins (device-timed, max over ranks).

    torchrun --nproc-per-node N bench/parallel_ops.py tp      # row-parallel GEMM + all-reduce (o_proj / down_proj of Qwen3-8B)
    torchrun --nproc-per-node N bench/parallel_ops.py ep      # expert-parallel MoE layer (Qwen3-30B-A3B geometry)

``tp``: ``out = residual + all_reduce(x @ W^T)`` followed by the next RMSNorm, with K sharded over the ranks, for 128
rows (one request, tree budget 128) and 2048 rows (batch 16 x 128 nodes).  Fused = GEMM whose epilogue pushes the
partial tiles over NVLink + one finishing kernel that reduces, adds the residual and normalises
(`TensorParallel.gemm_allreduce(..., norm_w=...)`); twin = ``torch.matmul`` + NCCL ``all_reduce`` + residual add +
``rms_norm``.  Both run as CUDA graphs of back-to-back calls on rotating weights.  Roofline per call = the slower of
weight bytes / measured copy bandwidth and payload bytes crossing NVLink / 770 GB/s (two-shot: 2 (w-1)/w partials
per rank; one-shot: (w-1) partials).

``ep``: one sparse-MoE layer on 1024 tokens, 128 experts, top-8, two plans: tokens sharded over the ranks with
peer-store dispatch and the combine in the down-projection epilogue (`TokenShardedEP.moe_layer`), and the replicated
plan (`ExpertParallel.moe_layer`), each against the same grouped GEMMs with NCCL collectives
(all-gather of the tokens / `moe_layer_grouped_nccl`).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
HBM_GBS, NVLINK_GBS = 6548.0, 770.0


def max_ranks(x: float) -> float:
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_graph(fn, calls: int, reps: int = 5) -> float:
    """Microseconds per call of ``fn(i)`` captured ``calls`` times into one CUDA graph (max over ranks)."""
    for i in range(calls):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    best = 1e30
    for _ in range(reps):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, max_ranks(a.elapsed_time(b)))
    return best * 1e3 / calls


def bench_tp(rank: int, world: int):
    from jetspec_b200.ops import cuda_ext as X
    from jetspec_b200.parallel import TensorParallel
    X.load()
    tp = TensorParallel(None, m_cap=2048, n_max=4096)
    R = 6                                                   # rotating weight copies (cold L2)
    for name, N, K in (("o_proj", 4096, 4096), ("down_proj", 4096, 12288)):
        Kl = K // world
        ws = [(torch.randn(N, Kl, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(R)]
        nw = torch.ones(N, device="cuda", dtype=torch.bfloat16)
        for M in (128, 2048):
            x = torch.randn(M, Kl, device="cuda").to(torch.bfloat16)
            res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
            out, h = torch.empty_like(res), torch.empty_like(res)
            calls = 12
            tp.begin_sequence(calls)
            fused = time_graph(lambda i: tp.gemm_allreduce(x, ws[i % R], out, residual=res, norm_w=nw, norm_out=h), calls)
            tp.begin_sequence(calls)

            def twin_fn(i):
                tp.gemm_allreduce_nccl(x, ws[i % R], out, residual=res)
                h.copy_(torch.nn.functional.rms_norm(out, (N,), nw, 1e-6))
            twin = time_graph(twin_fn, calls)
            X.check_status("cuda")
            w_us = N * Kl * 2 / HBM_GBS / 1e3
            part = M * N * 2
            link_us = (2 * (world - 1) / world if tp.push_only == 3 else (world - 1)) * part / NVLINK_GBS / 1e3
            if rank == 0:
                print(json.dumps({"op": f"gemm + all-reduce + rmsnorm, {name}", "mode": tp.mode, "world": world, "M": M,
                                  "N": N, "K_local": Kl, "fused_us": round(fused, 1), "nccl_twin_us": round(twin, 1),
                                  "speedup": round(twin / fused, 2),
                                  "roofline_us": round(max(w_us, link_us), 1),
                                  "fraction_of_roofline": round(max(w_us, link_us) / fused, 2)}), flush=True)
    tp.close()


def bench_ep(rank: int, world: int):
    from jetspec_b200.ops import cuda_ext as X
    from jetspec_b200.parallel.ep import ExpertParallel, TokenShardedEP
    X.load()
    E, H, I, k, T = 128, 2048, 768, 8, 1024
    g = torch.Generator(device="cuda").manual_seed(7)
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).to(torch.bfloat16)
    x, gate = bf(T, H), bf(E, H, sc=0.5)
    wgu, wd = bf(E, 2 * I, H, sc=0.03), bf(E, H, I, sc=0.03)
    ep = ExpertParallel(None, E, k, H, max_tokens=T)
    gu_l, dn_l = ep.shard(wgu, wd)

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return max_ranks(a.elapsed_time(b)) * 1e3 / iters

    fused = timed(lambda: ep.moe_layer(x, gate, gu_l, dn_l, True))
    twin = timed(lambda: ep.moe_layer_grouped_nccl(x, gate, gu_l, dn_l, True))
    X.check_status("cuda")
    w_us = (E // world) * 3 * H * I * 2 / HBM_GBS / 1e3
    link_us = T * k * H * 2 * (world - 1) / world / NVLINK_GBS / 1e3      # each rank sends its experts' rows to every peer
    if rank == 0:
        print(json.dumps({"op": "ep moe layer, replicated tokens", "world": world, "tokens": T, "experts": E, "top_k": k,
                          "hidden": H, "intermediate": I, "fused_us": round(fused, 1), "nccl_twin_us": round(twin, 1),
                          "speedup": round(twin / fused, 2), "roofline_us": round(max(w_us, link_us), 1),
                          "fraction_of_roofline": round(max(w_us, link_us) / fused, 2)}), flush=True)
    # token-sharded plan: every rank owns T / world of the same tokens
    Tl = T // world
    xl = x[rank * Tl:(rank + 1) * Tl].contiguous()
    hn = torch.nn.functional.rms_norm(xl, (H,), None, 1e-6)
    nw = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    eps = TokenShardedEP(None, E, k, H, max_tokens=max(128, Tl))
    out, h2 = torch.empty_like(xl), torch.empty_like(xl)
    fused2 = timed(lambda: eps.moe_layer(xl, hn, gate, gu_l, dn_l, True, out=out, norm_w=nw, norm_out=h2))
    X.check_status("cuda")
    full = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def twin2():      # NCCL all-gather of the tokens, every rank runs its experts on all of them, NCCL all-reduce
        dist.all_gather_into_tensor(full, hn)
        y = ep.moe_layer_grouped_nccl(full, gate, gu_l, dn_l, True)
        h2.copy_(torch.nn.functional.rms_norm(y[rank * Tl:(rank + 1) * Tl], (H,), nw, 1e-6))
    twin_s = timed(twin2)
    # per rank: its T/world x k rows leave once (bf16) and come back once (bf16 payload), (world-1)/world of them remote
    link2_us = 2 * Tl * k * H * 2 * (world - 1) / world / NVLINK_GBS / 1e3
    if rank == 0:
        print(json.dumps({"op": "ep moe layer, token-sharded dispatch + combine + rmsnorm", "world": world,
                          "tokens_per_rank": Tl, "experts": E, "top_k": k, "hidden": H, "intermediate": I,
                          "fused_us": round(fused2, 1), "nccl_twin_us": round(twin_s, 1),
                          "speedup": round(twin_s / fused2, 2), "roofline_us": round(max(w_us, link2_us), 1),
                          "fraction_of_roofline": round(max(w_us, link2_us) / fused2, 2),
                          "nvlink_payload_bytes_per_rank": int(2 * Tl * k * H * 2 * (world - 1) / world)}), flush=True)
    eps.close()
    ep.close()


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    {"tp": bench_tp, "ep": bench_ep}[sys.argv[1]](rank, world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
