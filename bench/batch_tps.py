"""Continuous-batching tree decode: aggregate tokens/s of B concurrent requests on one GPU.

Counterpart of the reference's batched entry points (``JetSpecEngine.generate_batch`` /
``generate_tree_batch``, ``jetspec/inference_engine/engine.py:1186-1608``): B requests with prompt
lengths uniform in ``[lo, hi]`` decode together; every round verifies all live trees in one ragged
forward through the paged pool.  Acceptance is scripted per request by an oracle drafter built from
that request's own greedy continuation (iterated to the verify path's fixed point), as in ``bench.py``.

    python bench/batch_tps.py --batch 16 --new 256            # Qwen3-8B, random init
    python bench/batch_tps.py --model small --batch 4 --new 32   # runs on CPU too

Prints one JSON line: aggregate tokens/s for the AR batch and the tree batch (wall clock around the
public call, synchronised on both sides), tokens per round, and rounds.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def main():
    from bench import model_config
    from jetspec_b200 import JetSpecEngine, OracleTreeDrafter, SamplingParams
    from jetspec_b200.models import Qwen3ForCausalLM
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b", choices=["qwen3-8b", "small"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prompt-lo", type=int, default=256)
    ap.add_argument("--prompt-hi", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--tree-depth", type=int, default=20)
    ap.add_argument("--tree-width", type=int, default=7)
    ap.add_argument("--budget", type=int, default=128)
    ap.add_argument("--mean-accept", type=float, default=7.0)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev, dt = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    cfg = model_config(args.model)
    model = Qwen3ForCausalLM.random_init(cfg, seed=args.seed, dtype=dt, device=dev, init="stable")
    gen = torch.Generator().manual_seed(args.seed)
    lens = torch.randint(args.prompt_lo, args.prompt_hi + 1, (args.batch,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (1, n), generator=gen) for n in lens]
    eng = JetSpecEngine(model, device=dev, dtype=dt, block_size=16,
                        max_seq_len=args.prompt_hi + args.new + 2 * args.budget + 64)
    sp = SamplingParams(0.0, args.new)
    # AR batch: the oracle's script and the baseline of the speedup
    eng.generate_batch(prompts, SamplingParams(0.0, 3))                # warm-up: module load, pool, graph capture
    _sync()
    t0 = time.perf_counter()
    ar = eng.generate_batch(prompts, sp)
    _sync()
    ar_s = time.perf_counter() - t0
    ar_tokens = sum(len(o["token_ids"]) for o in ar)
    max_accept = min(args.tree_depth, (args.budget - 2) // args.tree_width + 1)
    oracles = [OracleTreeDrafter(p[0].tolist() + o["token_ids"], cfg.vocab_size, tree_width=args.tree_width,
                                 mean_accept=args.mean_accept, max_accept=max_accept, seed=args.seed + i)
               for i, (p, o) in enumerate(zip(prompts, ar))]
    kw = dict(block_size=args.tree_depth + 1, tree_width=args.tree_width, budget=args.budget, sampling_params=sp,
              return_stats=True)
    converged = False
    for it in range(6):                                                 # fixed point of the verify path's own greedy tokens
        out = eng.generate_tree_batch(prompts, oracles, **kw)
        same = 0
        for p, o, orc in zip(prompts, out, oracles):
            seq = p[0].tolist() + o["token_ids"]
            if seq == orc.sequence[:len(seq)]:
                same += 1
            else:
                orc.set_continuation(seq)
        print(f"[oracle] iteration {it}: {same}/{len(prompts)} scripts hold", file=sys.stderr, flush=True)
        if same == len(prompts):
            converged = True
            break
    _sync()
    t0 = time.perf_counter()
    out = eng.generate_tree_batch(prompts, oracles, **kw)
    _sync()
    tree_s = time.perf_counter() - t0
    toks = sum(len(o["token_ids"]) for o in out)
    rounds = sum(o["rounds"] for o in out)
    acc = sum(sum(o["accept_lengths"]) for o in out)
    print(json.dumps({
        "bench": "continuous-batching tree decode", "model": args.model, "batch": args.batch,
        "prompt_lens": f"uniform [{args.prompt_lo}, {args.prompt_hi}]", "new_tokens": args.new,
        "tree": f"depth {args.tree_depth} width {args.tree_width} budget {args.budget}",
        "drafter": "oracle script per request (no draft-head forward in this bench)",
        "ar_tokens_per_s": round(ar_tokens / ar_s, 1), "tree_tokens_per_s": round(toks / tree_s, 1),
        "speedup": round((toks / tree_s) / (ar_tokens / ar_s), 3), "tokens_per_round": round(acc / max(1, rounds), 3),
        "batch_rounds": max(o["rounds"] for o in out), "ms_per_batch_round": round(tree_s * 1e3 / max(o["rounds"] for o in out), 2),
        "oracle_converged": converged, "timing": "wall clock around the public call, prefill included"}))


if __name__ == "__main__":
    main()
