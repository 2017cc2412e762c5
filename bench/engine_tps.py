"""Wall-clock throughput of the paged engine: AR vs tree-speculative, with data-parallel prompt sharding.

Counterpart of the reference's ``bench/engine/tps_walltime.py:164-306`` (rank sharding ``:85-139``, drafter
construction ``:142-161``): every rank (``torchrun``) holds a full
model replica and takes ``bank[rank::world]``; throughput is total tokens over the slowest rank's wall
time, reduced with NCCL (gloo on CPU).  Prompts are synthetic token sequences (no dataset or tokenizer
is needed); ``--prompt-set`` picks a length profile named after the reference's eight prompt sets.

    python bench/engine_tps.py --model DIR --head DIR --drafter graphed --session --warm-all
    torchrun --nproc-per-node 8 bench/engine_tps.py ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# (min prompt length, max prompt length) per named set
PROMPT_SETS = {"gsm8k": (96, 256), "math500": (64, 320), "humaneval": (128, 384), "mbpp": (64, 256),
               "aime25": (96, 320), "livecodebench": (256, 1024), "mtbench": (32, 256), "synthetic": (512, 512)}


def prompt_bank(name: str, samples: int, vocab: int, seed: int = 0) -> list:
    lo, hi = PROMPT_SETS[name]
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (samples,), generator=g).tolist()
    return [torch.randint(0, vocab, (1, n), generator=g) for n in lens]


def shard(bank: list, rank: int, world: int) -> list:
    return bank[rank::world]


def dist_env():
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    return world, rank, local


def reduce_stats(tokens: int, wall: float, acc_sum: float, rounds: int, world: int) -> dict:
    """Total tokens, slowest-rank wall time, global mean tokens/round (the reference's four reductions)."""
    if world > 1:
        import torch.distributed as dist
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        t = torch.tensor([tokens, acc_sum, rounds], dtype=torch.float64, device=dev)
        w = torch.tensor([wall], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        tokens, acc_sum, rounds, wall = t[0].item(), t[1].item(), t[2].item(), w.item()
    return {"tokens": int(tokens), "wall_s": wall, "tps": tokens / wall if wall > 0 else 0.0,
            "accept_len": acc_sum / rounds if rounds else 0.0}


def build_drafter(kind: str, head, engine, block_size: int):
    from jetspec_b200 import DraftHeadTreeDrafter, GraphedDraftHead, CompiledDraftHead
    cls = {"eager": DraftHeadTreeDrafter, "graphed": GraphedDraftHead, "compiled": CompiledDraftHead}[kind]
    return cls(head, engine.model, block_size=block_size, target_layer_ids=head.target_layer_ids)


def walltime(fn, prompts) -> tuple:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = [fn(p) for p in prompts]
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    return time.perf_counter() - t0, outs


def main():
    from jetspec_b200 import JetSpecEngine, SamplingParams, load_draft_head
    from jetspec_b200.models import Qwen3ForCausalLM, DraftHeadModel, draft_head_config, tiny_config
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--head", default=os.environ.get("JETSPEC_DRAFT_HEAD"))
    ap.add_argument("--prompt-set", default="gsm8k", choices=sorted(PROMPT_SETS))
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--tree-depth", type=int, default=20)
    ap.add_argument("--tree-width", type=int, default=7)
    ap.add_argument("--budget", type=int, default=128)
    ap.add_argument("--algo", default="accum_logp")
    ap.add_argument("--drafter", default="graphed", choices=["eager", "compiled", "graphed"])
    ap.add_argument("--session", action="store_true")
    ap.add_argument("--warm-all", action="store_true")
    ap.add_argument("--warmup-samples-per-rank", type=int, default=1)
    args = ap.parse_args()
    world, rank, local = dist_env()
    dev = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    if args.model:
        eng = JetSpecEngine(args.model, device=dev, dtype=dt, block_size=16)
        head = load_draft_head(args.head, device=dev, dtype=dt)
    else:   # smoke configuration: tiny random model, runs on CPU
        cfg = tiny_config()
        args.tree_depth, args.tree_width, args.budget, args.max_tokens = 4, 2, 8, min(args.max_tokens, 32)
        eng = JetSpecEngine(Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=dt), device=dev, dtype=dt)
        head = DraftHeadModel.random_init(draft_head_config(cfg, 1, args.tree_depth + 1, target_layer_ids=[0, 1]),
                                          seed=1, dtype=dt, device=dev)
    bs = args.tree_depth + 1
    drafter = build_drafter(args.drafter, head, eng, bs)
    prompts = shard(prompt_bank(args.prompt_set, args.samples, eng.cfg.vocab_size), rank, world)
    sp = SamplingParams(0.0, args.max_tokens)
    kw = dict(tree_depth=args.tree_depth, tree_width=args.tree_width, budget=args.budget, algo=args.algo,
              target_layer_ids=head.target_layer_ids, return_stats=True, sampling_params=sp)
    if args.session and prompts:
        kw.update(session=True, session_prompt_capacity=((max(p.shape[1] for p in prompts) + 255) // 256) * 256)
    for p in (prompts if args.warm_all else prompts[: args.warmup_samples_per_rank]):
        eng.generate(p, sp)
        eng.generate_tree(p, drafter, **kw)
    ar_wall, ar_out = walltime(lambda p: eng.generate(p, sp), prompts)
    tr_wall, tr_out = walltime(lambda p: eng.generate_tree(p, drafter, **kw), prompts)
    ar = reduce_stats(sum(len(o["token_ids"]) for o in ar_out), ar_wall, 0.0, 0, world)
    tr = reduce_stats(sum(len(o["token_ids"]) for o in tr_out), tr_wall,
                      float(sum(sum(o["accept_lengths"]) for o in tr_out)), sum(o["rounds"] for o in tr_out), world)
    if rank == 0:
        print(json.dumps({"prompt_set": args.prompt_set, "ranks": world, "ar_tps": round(ar["tps"], 2),
                          "tree_tps": round(tr["tps"], 2), "accept_len": round(tr["accept_len"], 3),
                          "speedup": round(tr["tps"] / ar["tps"], 3) if ar["tps"] else None}))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
