"""Fused compute+collective kernels against their NCCL twins (device-timed, max over ranks).

    torchrun --nproc-per-node N bench/parallel_ops.py tp      # row-parallel GEMM + all-reduce (o_proj / down_proj of Qwen3-8B)
    torchrun --nproc-per-node N bench/parallel_ops.py ep      # expert-parallel MoE layer (Qwen3-30B-A3B geometry)

``tp``: ``out = residual + all_reduce(x @ W^T)`` with K sharded over the ranks, for 128 rows (one request, tree budget
128) and 2048 rows (batch 16 x 128 nodes).  Fused = one kernel per rank (`TensorParallel.gemm_allreduce`, partial tiles
stored into every peer's buffer over NVLink from the GEMM epilogue); twin = ``torch.matmul`` + NCCL ``all_reduce`` +
residual add.  Both run as CUDA graphs of back-to-back calls on rotating weights.  Roofline per call = the slower of
weight bytes / measured copy bandwidth and bytes crossing NVLink / 770 GB/s.

``ep``: one sparse-MoE layer on 1024 tokens, 128 experts, top-8: fused combine in the grouped down-projection epilogue
(`ExpertParallel.moe_layer`) against the same grouped GEMMs + scatter + NCCL all-reduce (`moe_layer_grouped_nccl`).
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
        for M in (128, 2048):
            x = torch.randn(M, Kl, device="cuda").to(torch.bfloat16)
            res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
            out = torch.empty_like(res)
            calls = 12
            slabs = -(-M // (max(1, (2 * X.SM_COUNT) // ((N + 127) // 128)) * 128))      # launches per fused call
            tp.begin_sequence(calls * slabs)
            fused = time_graph(lambda i: tp.gemm_allreduce(x, ws[i % R], out, residual=res), calls)
            tp.begin_sequence(calls)
            twin = time_graph(lambda i: tp.gemm_allreduce_nccl(x, ws[i % R], out, residual=res), calls)
            X.check_status("cuda")
            w_us = N * Kl * 2 / HBM_GBS / 1e3
            # one-shot all-reduce: every rank sends its (M, N) bf16 partial to world-1 peers
            link_us = M * N * 2 * (world - 1) / NVLINK_GBS / 1e3
            if rank == 0:
                print(json.dumps({"op": f"gemm_allreduce {name}", "world": world, "M": M, "N": N, "K_local": Kl,
                                  "fused_us": round(fused, 1), "nccl_twin_us": round(twin, 1),
                                  "speedup": round(twin / fused, 2),
                                  "roofline_us": round(max(w_us, link_us), 1),
                                  "fraction_of_roofline": round(max(w_us, link_us) / fused, 2)}), flush=True)
    tp.close()


def bench_ep(rank: int, world: int):
    from jetspec_b200.ops import cuda_ext as X
    from jetspec_b200.parallel.ep import ExpertParallel
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
        print(json.dumps({"op": "ep moe layer", "world": world, "tokens": T, "experts": E, "top_k": k, "hidden": H,
                          "intermediate": I, "fused_us": round(fused, 1), "nccl_twin_us": round(twin, 1),
                          "speedup": round(twin / fused, 2), "roofline_us": round(max(w_us, link_us), 1),
                          "fraction_of_roofline": round(max(w_us, link_us) / fused, 2)}), flush=True)
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
