"""Multi-metric benchmark of the reference engine (``LLM``): acceptance length, per-position acceptance
(d0..d3), mean tree size, decode and end-to-end tokens/s, speedups over autoregressive and over the
linear block (chain) baseline; JSONL output per algorithm.

Counterpart of ``bench/reference/benchmark.py`` (metrics ``:432-495``), ``dflash_baseline.py`` (the
greedy chain baseline) and ``hf_fa2_decode_baseline.py`` (raw AR decode timing).  Ranks shard the
prompts; per-metric sums are all-reduced (latency-sum accounting: throughput = tokens / summed latency).

    python bench/reference_metrics.py --algos accum_logp,top2gap_fanout --out-dir bench/outputs
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn):
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = fn()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return out, time.perf_counter() - t0


def gpu_clock_warmup(seconds: float = 0.5) -> None:
    """Spin a matmul so the clocks are up before the first timed sample."""
    if not torch.cuda.is_available():
        return
    a = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16)
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        a @ a
    torch.cuda.synchronize()


def position_accept_rates(accept_lengths, positions: int = 4) -> list:
    """d0..d{positions-1}: fraction of rounds whose accepted draft length exceeds each position."""
    n = max(1, len(accept_lengths))
    return [sum(1 for a in accept_lengths if a - 1 > d) / n for d in range(positions)]


def summarize(name: str, outs: list, lat: list, ar_tps: float, chain_tps: float) -> dict:
    acc = [a for o in outs for a in o.get("accept_lengths", [])]
    toks = sum(len(o["token_ids"]) for o in outs)
    dec = sum(o.get("decode_time", 0.0) for o in outs)
    row = {"algo": name, "samples": len(outs), "tokens": toks,
           "accept_len": sum(acc) / len(acc) if acc else 0.0,
           "tree_size": (sum(s for o in outs for s in o.get("tree_sizes", [])) / max(1, len(acc))),
           "decode_tps": toks / dec if dec > 0 else 0.0, "e2e_tps": toks / sum(lat) if sum(lat) > 0 else 0.0}
    for i, r in enumerate(position_accept_rates(acc)):
        row[f"d{i}"] = r
    row["speedup_vs_ar"] = row["e2e_tps"] / ar_tps if ar_tps else None
    row["speedup_vs_chain"] = row["e2e_tps"] / chain_tps if chain_tps else None
    return row


def all_reduce_sum(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t)
    return float(t.item())


def chain_generate(llm, prompt, head_drafter, block_size: int, sp):
    """Linear block speculation with the draft head (greedy): the chain baseline."""
    return llm.generate_chain(prompt, head_drafter, block_size=block_size,
                              target_layer_ids=head_drafter.target_layer_ids, sampling_params=sp)


def main():
    from jetspec_b200 import LLM, SamplingParams, DraftHeadDrafter, DraftHeadTreeDrafter, load_draft_head
    from jetspec_b200.models import Qwen3ForCausalLM, DraftHeadModel, draft_head_config, tiny_config
    from jetspec_b200.tree import list_algorithms
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--head", default=None)
    ap.add_argument("--algos", default="accum_logp")
    ap.add_argument("--samples", type=int, default=4)
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--block-size", type=int, default=5)
    ap.add_argument("--tree-width", type=int, default=2)
    ap.add_argument("--budget", type=int, default=8)
    ap.add_argument("--profile-table", default=None)
    ap.add_argument("--out-dir", default=None)
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    if args.model:
        llm = LLM(args.model, device=dev, dtype=dt)
        head = load_draft_head(args.head, device=dev, dtype=dt)
    else:
        cfg = tiny_config()
        llm = LLM(Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=dt), device=dev, dtype=dt)
        head = DraftHeadModel.random_init(draft_head_config(cfg, 1, args.block_size, target_layer_ids=[0, 1]), seed=1,
                                          dtype=dt, device=dev)
    table = json.load(open(args.profile_table)) if args.profile_table else None
    g = torch.Generator().manual_seed(0)
    bank = [torch.randint(0, llm.model.config.vocab_size, (1, 24), generator=g) for _ in range(args.samples)][rank::world]
    sp = SamplingParams(0.0, args.max_new)
    gpu_clock_warmup()
    ar = [timed(lambda p=p: llm.generate(p, sp)) for p in bank]
    ar_tps = all_reduce_sum(sum(len(o["token_ids"]) for o, _ in ar), world) / max(1e-9, all_reduce_sum(sum(t for _, t in ar), world))
    chain_d = DraftHeadDrafter(head, llm.model, block_size=args.block_size)
    ch = [timed(lambda p=p: chain_generate(llm, p, chain_d, args.block_size, sp)) for p in bank]
    chain_tps = all_reduce_sum(sum(len(o["token_ids"]) for o, _ in ch), world) / max(1e-9, all_reduce_sum(sum(t for _, t in ch), world))
    tree_d = DraftHeadTreeDrafter(head, llm.model, block_size=args.block_size)
    rows = []
    for name in args.algos.split(","):
        if name not in list_algorithms():
            raise SystemExit(f"unknown algorithm {name}")
        res = [timed(lambda p=p: llm.generate_tree(p, tree_d, block_size=args.block_size, tree_width=args.tree_width,
                                                   budget=args.budget, algo=name, target_layer_ids=head.target_layer_ids,
                                                   sampling_params=sp, return_stats=True, profile_phases=True,
                                                   profile_table=table)) for p in bank]
        row = summarize(name, [o for o, _ in res], [t for _, t in res], ar_tps, chain_tps)
        row["phase_ms_per_round"] = res[0][0].get("phase_times", {}) if res else {}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row))
            if args.out_dir:
                os.makedirs(args.out_dir, exist_ok=True)
                with open(os.path.join(args.out_dir, f"{name}.jsonl"), "a") as f:
                    f.write(json.dumps(row) + "\n")
    if rank == 0:
        print(json.dumps({"ar_tps": ar_tps, "chain_tps": chain_tps}))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
