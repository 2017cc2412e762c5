"""Continuous-batching tree decode: aggregate tokens/s of B concurrent requests on one GPU, or tensor-parallel
over the N GPUs of one node when launched with ``torch.distributed.run`` (``--nproc-per-node N``).

Counterpart of the reference's batched entry points (``JetSpecEngine.generate_batch`` /
``generate_tree_batch``, ``jetspec/inference_engine/engine.py:1186-1608``): B requests with prompt
lengths uniform in ``[lo, hi]`` decode together; every round verifies all live trees in one ragged
forward through the paged pool.  Acceptance is scripted per request by an oracle drafter built from
that request's own greedy continuation (iterated to the verify path's fixed point), as in ``bench.py``.

    python bench/batch_tps.py --batch 16 --new 256            # Qwen3-8B, random init
    python bench/batch_tps.py --model small --batch 4 --new 32   # runs on CPU too
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 bench/batch_tps.py --batch 16 --new 1024
        # one batch tensor-parallel over 4 GPUs: every verify forward is 16 x 128 rows through the fused
        # row-parallel GEMM + all-reduce kernels; --weights nvfp4 runs the 4-bit linears

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
    ap.add_argument("--weights", default="bf16", choices=["bf16", "nvfp4"])
    ap.add_argument("--skip-ar", action="store_true", help="skip the timed AR batch (the oracle script is derived "
                                                           "from the model's known continuation instead)")
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    tp = None
    if world > 1:
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from jetspec_b200.engine.engine import bucket_for_n
        from jetspec_b200.parallel import TensorParallel
        tp = TensorParallel(None, m_cap=max(512, args.batch * bucket_for_n(args.budget)))
    dev, dt = ((f"cuda:{torch.cuda.current_device()}" if world > 1 else "cuda"), torch.bfloat16) if cuda else ("cpu", torch.float32)
    cfg = model_config(args.model)
    model = Qwen3ForCausalLM.random_init(cfg, seed=args.seed, dtype=dt, device=dev, init="stable")
    if args.weights == "nvfp4":
        from jetspec_b200.models.nvfp4 import quantize_model_nvfp4
        quantize_model_nvfp4(model)
        torch.cuda.empty_cache()
    gen = torch.Generator().manual_seed(args.seed)
    lens = torch.randint(args.prompt_lo, args.prompt_hi + 1, (args.batch,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (1, n), generator=gen) for n in lens]
    eng = JetSpecEngine(model, device=dev, dtype=dt, block_size=16,
                        max_seq_len=args.prompt_hi + args.new + 2 * args.budget + 64, tensor_parallel=tp)
    sp = SamplingParams(0.0, args.new)
    # AR batch: the oracle's script and the baseline of the speedup
    eng.generate_batch(prompts, SamplingParams(0.0, 3))                # warm-up: module load, pool, graph capture
    _sync()
    t0 = time.perf_counter()
    if args.skip_ar:       # the wide-margin synthetic model counts upwards: its greedy continuation is known
        ar = [{"token_ids": [(int(p[0, -1]) + 1 + i) % cfg.vocab_size for i in range(args.new)]} for p in prompts]
    else:
        ar = eng.generate_batch(prompts, sp)
    _sync()
    ar_s = max(time.perf_counter() - t0, 1e-9)
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
        if rank == 0:
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
    if rank != 0:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        return
    print(json.dumps({
        "bench": "continuous-batching tree decode", "model": args.model, "batch": args.batch,
        "parallelism": f"tp{world}" + (f" ({tp.mode} all-reduce)" if tp is not None else ""), "weights": args.weights,
        "prompt_lens": f"uniform [{args.prompt_lo}, {args.prompt_hi}]", "new_tokens": args.new,
        "tree": f"depth {args.tree_depth} width {args.tree_width} budget {args.budget}",
        "drafter": "oracle script per request (no draft-head forward in this bench)",
        "ar_tokens_per_s": None if args.skip_ar else round(ar_tokens / ar_s, 1),
        "tree_tokens_per_s": round(toks / tree_s, 1),
        "speedup": None if args.skip_ar else round((toks / tree_s) / (ar_tokens / ar_s), 3),
        "tokens_per_round": round(acc / max(1, rounds), 3),
        "batch_rounds": max(o["rounds"] for o in out), "ms_per_batch_round": round(tree_s * 1e3 / max(o["rounds"] for o in out), 2),
        "tokens_per_s_per_request": round(toks / tree_s / args.batch, 1),
        "oracle_converged": converged, "timing": "wall clock around the public call, prefill included"}))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
