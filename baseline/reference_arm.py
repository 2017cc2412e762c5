"""Runs the UNMODIFIED reference package (installed under ``baseline/_ref``) on the benchmark
configuration and prints the same JSON line as ``bench.py`` with ``"impl": "reference"``.

The reference loads models with Hugging Face ``from_pretrained``, so the synthetic target and
draft head are first written to a scratch directory in the stock checkpoint format (the same
seeded weights our own arm uses) together with a minimal word-level tokenizer; prompts are
passed as token ids.  The engine is then built and driven exactly as the reference's own
throughput script does (``bench/engine/tps_walltime.py:205-275``): backend
``triton_paged_tree_cudagraph_nogather``, fused GEMMs, ``GraphedDraftHead``, ``session=True``.
The reference's multi-GPU mode is data parallel (every rank a full replica,
``bench/engine/tps_walltime.py:178-203``); it cannot split one request over GPUs.  For N > 1 every
rank therefore serves a replica of the SAME request from one shared scratch checkpoint, and the
line reports tokens per second PER REQUEST over the slowest rank's time, the quantity this repo's
own arm reports when it runs the one request tensor-parallel over the N GPUs.

If any step the reference needs cannot run on this box, the function prints
``{"impl": "reference", "unavailable": "<why>"}`` and returns.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def write_tokenizer(path: str, vocab_size: int) -> None:
    """A word-level tokenizer with ``vocab_size`` dummy entries, enough for ``AutoTokenizer``."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {f"t{i}": i for i in range(vocab_size)}
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="t0", pad_token="t0").save_pretrained(path)


def write_hf_config(path: str, cfg, extra: dict | None = None) -> None:
    """``config.json`` in the stock Qwen3 layout."""
    d = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": cfg.vocab_size,
        "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
        "num_hidden_layers": cfg.num_hidden_layers, "num_attention_heads": cfg.num_attention_heads,
        "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "hidden_act": "silu",
        "max_position_embeddings": cfg.max_position_embeddings, "rms_norm_eps": cfg.rms_norm_eps,
        "rope_theta": cfg.rope_theta, "tie_word_embeddings": False, "attention_bias": False,
        "attention_dropout": 0.0, "use_cache": True, "torch_dtype": "bfloat16", "sliding_window": None,
        "use_sliding_window": False, "max_window_layers": cfg.num_hidden_layers,
    }
    d.update(extra or {})
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(d, f, indent=1)


def build_checkpoints(args, scratch: str, device: str):
    """Write target + draft head (our seeded synthetic weights) in Hugging Face format."""
    import torch
    from bench import model_config
    from jetspec_b200.models import Qwen3ForCausalLM, DraftHeadModel, draft_head_config
    from jetspec_b200.models.loader import save_state
    cfg = model_config(args.model)
    bs = args.tree_depth + 1
    tdir, hdir = os.path.join(scratch, "target"), os.path.join(scratch, "head")
    model = Qwen3ForCausalLM.random_init(cfg, seed=args.seed, dtype=torch.bfloat16, device=device, init="stable")
    write_hf_config(tdir, cfg)
    save_state(dict(model.state_dict()), tdir)
    write_tokenizer(tdir, cfg.vocab_size)
    del model
    hcfg = draft_head_config(cfg, num_layers=1, block_size=bs, num_taps=5)
    head = DraftHeadModel.random_init(hcfg, seed=args.seed + 1, dtype=torch.bfloat16, device=device)
    write_hf_config(hdir, hcfg, {"architectures": ["DFlashDraftModel"], "block_size": bs,
                                 "num_target_layers": cfg.num_hidden_layers, "dflash_config": hcfg.dflash_config,
                                 "layer_types": ["full_attention"] * hcfg.num_hidden_layers})
    save_state(dict(head.state_dict()), hdir)
    del head
    torch.cuda.empty_cache()
    return cfg, tdir, hdir


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl")
    scratch = os.path.join(tempfile.gettempdir(), f"jetspec_ref_{os.environ.get('MASTER_PORT', os.getpid())}")
    try:
        res = _run(args, world, rank, scratch)
    except Exception as e:  # noqa: BLE001 - any failure of the reference stack is reported, not raised
        tb = traceback.format_exc().strip().splitlines()
        res = {"unavailable": f"{type(e).__name__}: {e} | {tb[-3] if len(tb) >= 3 else ''}"}
    try:
        if world > 1:
            import torch.distributed as dist
            allres = [None] * world
            dist.all_gather_object(allres, res)
        else:
            allres = [res]
        if rank == 0:
            _report(args, allres)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            shutil.rmtree(scratch, ignore_errors=True)


def _sync_ranks(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def _run(args, world: int, rank: int, scratch: str) -> dict:
    if not os.path.isdir(os.path.join(REF, "jetspec")):
        return {"unavailable": "reference package is not installed under baseline/_ref"}
    import torch
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device"}
    sys.path.insert(0, REF)
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(1, root)
    os.environ.setdefault("JETSPEC_FUSE_GEMMS", "1")
    cache = os.path.join(tempfile.gettempdir(), f"jetspec_ref_cache_{rank}")
    os.environ.setdefault("TORCHINDUCTOR_CACHE_DIR", os.path.join(cache, "inductor"))
    os.environ.setdefault("TRITON_CACHE_DIR", os.path.join(cache, "triton"))
    from bench import ClockSampler, model_config
    from jetspec_b200.drafters import OracleTreeDrafter, OracleOverrideDrafter
    dev = "cuda:0" if world == 1 else f"cuda:{os.environ.get('LOCAL_RANK', '0')}"
    err = None
    if rank == 0:
        try:
            build_checkpoints(args, scratch, dev)
        except Exception as e:  # noqa: BLE001
            err = f"checkpoint export failed: {type(e).__name__}: {e}"
    _sync_ranks(world)
    if err or not os.path.isdir(os.path.join(scratch, "head")):
        return {"unavailable": err or "checkpoint export failed on rank 0"}
    cfg = model_config(args.model)
    tdir, hdir = os.path.join(scratch, "target"), os.path.join(scratch, "head")
    from jetspec.inference_engine import JetSpecEngine, SamplingParams
    from jetspec import load_draft_head
    from jetspec.draft_head_adapter import GraphedDraftHead
    eng = JetSpecEngine(tdir, device=dev, dtype=torch.bfloat16, block_size=16, attn_implementation="sdpa",
                        attn_backend="triton_paged_tree_cudagraph_nogather", fuse_gemms=True)
    head = load_draft_head(hdir, device=dev, dtype=torch.bfloat16, attn_implementation=eng.resolved_attn_implementation)
    bs = args.tree_depth + 1
    real = GraphedDraftHead(head, target=eng.model, block_size=bs, target_layer_ids=head.target_layer_ids,
                            draft_shift=False)
    req_seed = args.seed            # every rank serves the same request
    prompt = torch.randint(0, cfg.vocab_size, (1, args.prompt_len),
                           generator=torch.Generator().manual_seed(req_seed)).pin_memory()
    sp = SamplingParams(0.0, args.max_new)
    cont = prompt[0].tolist() + eng.generate(prompt, sp)["token_ids"]
    max_accept = min(args.tree_depth, (args.budget - 2) // args.tree_width + 1)
    oracle = OracleTreeDrafter(cont, cfg.vocab_size, tree_width=args.tree_width, mean_accept=args.mean_accept,
                               max_accept=max_accept, seed=req_seed)
    drafter = OracleOverrideDrafter(real, oracle)
    kw = dict(block_size=bs, tree_width=args.tree_width, budget=args.budget, tree_depth=args.tree_depth,
              algo="accum_logp", target_layer_ids=head.target_layer_ids, return_stats=True, sampling_params=sp,
              session=True, session_prompt_capacity=((args.prompt_len + 255) // 256) * 256)
    converged = False
    for it in range(6):
        out = eng.generate_tree(prompt, drafter, **kw)
        seq = prompt[0].tolist() + out["token_ids"]
        if seq == oracle.sequence[:len(seq)]:
            converged = True
            break
        oracle.set_continuation(seq)
    for _ in range(args.warmup):
        eng.generate_tree(prompt, drafter, **kw)
    sampler = ClockSampler(torch.cuda.current_device())
    torch.cuda.synchronize()
    _sync_ranks(world)
    sampler.start()
    toks, rounds, accept, dev_ms = 0, 0, [], 0.0
    oracle.host_seconds = 0.0
    for _ in range(args.steps):        # one event pair around each whole request, as in this repo's own arm
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = eng.generate_tree(prompt, drafter, **kw)
        e1.record()
        torch.cuda.synchronize()
        dev_ms += e0.elapsed_time(e1)
        toks += len(out["token_ids"])
        rounds += out["rounds"]
        accept += out["accept_lengths"]
    oracle_s = oracle.host_seconds
    _sync_ranks(world)
    t0 = time.perf_counter()
    e2e_toks = 0
    for _ in range(args.steps):        # end to end by the wall clock, a second set of steps
        e2e_toks += len(eng.generate_tree(prompt, drafter, **kw)["token_ids"])
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    return {"toks": toks, "rounds": rounds, "acc_sum": float(sum(accept)), "acc_n": len(accept), "wall": wall,
            "e2e_toks": e2e_toks, "dev_ms": dev_ms, "oracle_s": oracle_s, "clocks": sampler.stop(),
            "converged": converged}


def _report(args, allres: list) -> None:
    from bench import BASELINE_TOK_S, TIMING_NOTE, bench_config
    bad = [r for r in allres if "unavailable" in r]
    if bad:
        return _unavailable(bad[0]["unavailable"])
    n = len(allres)
    r0 = allres[0]                       # every rank served the same request: rank 0's counts, slowest rank's time
    dev_ms, wall = max(r["dev_ms"] for r in allres), max(r["wall"] for r in allres)
    value = r0["toks"] / (dev_ms / 1e3)
    rounds = r0["rounds"]
    D, K = args.tree_depth, args.tree_width
    print(json.dumps({
        "metric": "decode tokens/s/request, Qwen3-8B tree budget 128", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dev_ms / args.steps, 3), "higher_is_better": True,
        "scaling": "strong" if n == 1 else "weak",
        "vs_baseline": round(value / BASELINE_TOK_S, 4), "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": bench_config(
            args, n_req=n, parallelism=f"dp{n}" + (" (one replica of the request per GPU; no tensor parallelism exists)" if n > 1 else ""),
            drafter="1-layer head (5 taps, GraphedDraftHead) + oracle script",
            backend="triton_paged_tree_cudagraph_nogather + fuse_gemms + GraphedDraftHead + session",
            mean_tokens=r0["acc_sum"] / max(1, r0["acc_n"]), ms_per_round=None, prefill_ms=None,
            oracle_ms_per_round=r0["oracle_s"] * 1e3 / max(1, rounds),
            converged=all(r["converged"] for r in allres), timing=TIMING_NOTE,
            request_ms_per_round=round(dev_ms / max(1, rounds), 4),
            decode_only_tokens_per_s=None, aggregate_tokens_per_s=round(value * n, 2)),
        "clocks": r0["clocks"],
        "e2e": {"value": round(r0["e2e_toks"] / wall, 2), "unit": "tokens/s",
                "h2d_bytes_per_step": args.prompt_len * 8 + int(rounds / args.steps * (D * K * 8)),
                "d2h_bytes_per_step": int(rounds / args.steps * 16)},
        "gpu_launches": 0,
    }), flush=True)
