"""Profiling helpers: device-time splits, tree diagnostics, depth-rank acceptance profiles and the
conditioned-vs-marginal drafter probe.

Counterparts of the reference's ``bench/profiling/*.py``.  Everything that computes a statistic is a
pure function (unit-tested on CPU); the ``main`` at the bottom runs them on a model:

    python bench/profiling.py diagnostics      [--model DIR] [--head DIR]
    python bench/profiling.py depth-rank       --out profile.json     # engine path, accepted chain only
    python bench/profiling.py llm-depth-rank   --out profile.json     # reference-engine path, every tree node
    python bench/profiling.py conditioned-probe                       # does path conditioning help the drafter?
    python bench/profiling.py verify-split
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional, Sequence

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


# ----------------------------------------------------------------------------- device-time split
class GpuTimer:
    """Wraps a callable and accumulates its CUDA-event time (skipped while a graph is captured).
    ``GpuTimer.patch(obj, "method")`` swaps the method for a timed one, the way the reference splits
    verify / draft / prefill time (``compare_engine_with_vllm_integration.py:57-81,124-177``)."""

    def __init__(self, fn, name: str = ""):
        self.fn, self.name = fn, name
        self.pairs, self.calls = [], 0

    def __call__(self, *a, **k):
        if not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
            return self.fn(*a, **k)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = self.fn(*a, **k)
        e.record()
        self.pairs.append((s, e))
        self.calls += 1
        return out

    def total_s(self) -> float:
        if not self.pairs:
            return 0.0
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.pairs) / 1e3

    @classmethod
    def patch(cls, obj, attr: str) -> "GpuTimer":
        t = cls(getattr(obj, attr), attr)
        setattr(obj, attr, t)
        return t


def decode_cuda_speedup(ar_decode_s: float, ar_tokens: int, tree_decode_s: float, tree_tokens: int) -> float:
    """Per-token device-time ratio AR / tree (drafter excluded): the reference's verify-only metric."""
    if ar_tokens <= 0 or tree_tokens <= 0 or tree_decode_s <= 0:
        return 0.0
    return (ar_decode_s / ar_tokens) / (tree_decode_s / tree_tokens)


# ----------------------------------------------------------------------------- tree diagnostics
def summarize_tree_diag(*, accept_lengths: Sequence[int], tree_nodes_per_depth: Sequence[int], output_tokens: int,
                        num_samples: int, block_size: int, max_depth: Optional[int] = None) -> dict:
    """Acceptance histogram, per-depth acceptance rate and mean tree nodes per depth.

    ``accept_lengths`` holds ``accepted + 1`` per round (the correction included), as the engines
    report it.  Same fields as the reference's summary (``collect_tree_diagnostics.py:38-82``)."""
    rounds = len(accept_lengths)
    slots = block_size if max_depth is None else int(max_depth)
    if slots <= 0:
        raise ValueError(f"max_depth must be positive; got {slots}")
    hist = [0] * slots
    for a in accept_lengths:
        d = int(a) - 1
        if not 0 <= d < slots:
            raise ValueError(f"accept length {a} maps to draft length {d}, outside [0, {slots - 1}]")
        hist[d] += 1
    denom = rounds or 1
    nodes = ([int(v) for v in tree_nodes_per_depth] + [0] * slots)[:slots]
    return {
        "output_tokens": int(output_tokens), "num_drafts": rounds, "num_samples": int(num_samples),
        "tokens_per_sample": float(output_tokens) / num_samples if num_samples else 0.0,
        "acceptance_length": sum(accept_lengths) / rounds if rounds else 0.0,
        "acceptance_length_histogram": [c / denom for c in hist],
        "per_depth_acceptance_rate": [sum(1 for a in accept_lengths if int(a) - 1 > d) / denom for d in range(slots - 1)],
        "avg_tree_nodes_per_depth": [nodes[d] / denom for d in range(1, slots)],
    }


def format_metrics_report(metrics: dict, *, attention_backend: str, block_size: int, tree_width: int, budget: int,
                          algo: str, drafter: str) -> str:
    """``key=value`` lines, one per metric (the external serving stack's report format)."""
    rows = [("mode", "dflash"), ("engine", "jetspec_b200"), ("prompt_set", metrics.get("prompt_set", "synthetic")),
            ("attention_backend", attention_backend), ("head_type", "causal"), ("block_size", block_size),
            ("tree_width", tree_width), ("max_tree_budget", budget), ("tree_draft", algo), ("drafter", drafter),
            ("num_samples", metrics["num_samples"]), ("output_tokens", metrics["output_tokens"]),
            ("tokens_per_sample", f"{metrics['tokens_per_sample']:.6f}"), ("num_drafts", metrics["num_drafts"]),
            ("acceptance_length", f"{metrics['acceptance_length']:.6f}"),
            ("per_depth_acceptance_rate", ",".join(f"{v:.6f}" for v in metrics["per_depth_acceptance_rate"])),
            ("acceptance_length_histogram", ",".join(f"{v:.6f}" for v in metrics["acceptance_length_histogram"])),
            ("avg_tree_nodes_per_depth", ",".join(f"{v:.2f}" for v in metrics["avg_tree_nodes_per_depth"]))]
    return "\n".join(f"{k}={v}" for k, v in rows) + "\n"


# ----------------------------------------------------------------------------- depth-rank profile
class RoundRecorder:
    """Drafter wrapper that keeps each round's per-depth top-k tokens (for profiles and diagnostics)."""

    def __init__(self, drafter, width: int):
        self.drafter, self.width = drafter, width
        self.rounds = []   # list of (context_len, tokens[D][K])

    def reset_cache(self):
        self.rounds = []
        if hasattr(self.drafter, "reset_cache"):
            self.drafter.reset_cache()

    def propose_logits(self, context_ids, depth, target_hidden=None, **kw):
        logits = self.drafter.propose_logits(context_ids, depth, target_hidden=target_hidden, **kw)
        top = torch.topk(torch.log_softmax(logits[0].float(), -1), self.width, dim=-1).indices
        self.rounds.append((int(context_ids.shape[-1]), top.tolist()))
        return logits


def depth_rank_counts(rounds, sequence: Sequence[int], width: int, depth: int):
    """For each recorded round, the rank (within the drafter's top-k) of the token the target actually
    emitted at each depth along the accepted chain.  Returns ``(hits[D][K], trials[D])``: depth ``d`` is
    counted while every shallower depth was a hit, i.e. P(accepted | rank-r present at depth d)."""
    hits = [[0] * width for _ in range(depth)]
    trials = [0] * depth
    for ctx_len, toks in rounds:
        for d in range(min(depth, len(toks))):
            pos = ctx_len + d
            if pos >= len(sequence):
                break
            trials[d] += 1
            row = toks[d]
            if sequence[pos] in row:
                hits[d][row.index(sequence[pos])] += 1
            else:
                break
    return hits, trials


def depth_rank_profile(hits, trials, meta: Optional[dict] = None) -> dict:
    """Profile table in the schema the ``depth_rank_histogram`` algorithm reads."""
    table = [[(h / t if t else 0.0) for h in row] for row, t in zip(hits, trials)]
    return {"depth_rank_accept": table, "meta": dict(meta or {}, trials=list(trials))}


def all_node_rank_counts(depths: Sequence[int], target_pick: Sequence[int], topk_tokens: Sequence[Sequence[int]],
                         hits=None, totals=None):
    """Every node of a verified tree at depth ``d < D`` is a parent the drafter offered ``K`` children to
    (its depth-``d`` top-k); count the rank of the token the TARGET picked there.  ``hits[d][r]`` / ``totals[d]``
    = P(target pick at a depth-``d`` parent is the drafter's rank ``r``): the table ``depth_rank_histogram`` reads
    (reference collector: ``bench/profiling/collect_depth_rank_stats.py:32-101``, which counts the same event)."""
    D = len(topk_tokens)
    K = len(topk_tokens[0]) if D else 0
    hits = hits if hits is not None else [[0] * K for _ in range(D)]
    totals = totals if totals is not None else [0] * D
    rank = [{int(t): r for r, t in enumerate(row)} for row in topk_tokens]
    for d, pick in zip(depths, target_pick):
        if d >= D:
            continue
        totals[d] += 1
        r = rank[d].get(int(pick))
        if r is not None:
            hits[d][r] += 1
    return hits, totals


class LLMRoundCollector:
    """``on_round`` hook for :meth:`jetspec_b200.LLM.generate_tree`: per-node depth-rank counts and, when the
    drafter can condition on a path, the conditioned-vs-marginal rank of every correction token."""

    def __init__(self, width: int, depth: int, drafter=None, probe: bool = False):
        self.width, self.depth, self.drafter, self.probe = int(width), int(depth), drafter, bool(probe)
        self.hits = [[0] * self.width for _ in range(self.depth)]
        self.totals = [0] * self.depth
        self.marginal_ranks: list = []
        self.conditioned_ranks: list = []

    def __call__(self, info: dict) -> None:
        lp = torch.log_softmax(info["draft_logits"][0].float(), -1)
        top = torch.topk(lp, self.width, dim=-1).indices.tolist()
        tree = info["tree"]
        all_node_rank_counts(tree.depth.tolist(), info["target_argmax"].tolist(), top, self.hits, self.totals)
        acc = info["accepted"]
        if not self.probe or acc >= lp.shape[0] or acc == 0:
            return           # nothing was accepted, or the whole chain was: no failed depth to look at
        cond_fn = getattr(self.drafter, "propose_logits_conditioned", None)
        if cond_fn is None:
            return
        path_tokens = tree.token_ids[info["path"][1:]]
        cond = cond_fn(info["committed"], path_tokens, target_hidden=info["target_hidden"])
        self.marginal_ranks.append(rank_of(info["correction"], lp[acc]))
        self.conditioned_ranks.append(rank_of(info["correction"], cond[0, acc].float()))

    def profile(self, meta: Optional[dict] = None) -> dict:
        return depth_rank_profile(self.hits, self.totals, meta)


# ----------------------------------------------------------------------------- conditioned vs marginal probe
def rank_of(token: int, logits_row: torch.Tensor) -> int:
    """0-based rank of ``token`` in a logits row."""
    return int((logits_row > logits_row[token]).sum())


def conditioned_probe_verdict(marginal_ranks: Sequence[int], conditioned_ranks: Sequence[int], top: int = 7,
                              lift_threshold: float = 0.15) -> dict:
    """Does feeding the accepted path back to the drafter help it predict the correction token?
    Compares the top-``top`` hit rate of the correction under marginal and path-conditioned logits;
    the verdict is ``P3_BUILD`` when the lift reaches ``lift_threshold`` (reference:
    ``compare_conditioned_draft_logits.py:272-296``)."""
    n = max(1, len(marginal_ranks))
    m = sum(1 for r in marginal_ranks if r < top) / n
    c = sum(1 for r in conditioned_ranks if r < top) / n
    return {"n": len(marginal_ranks), f"marginal_top{top}": m, f"conditioned_top{top}": c, "lift": c - m,
            "verdict": "P3_BUILD" if c - m >= lift_threshold else "P3_SKIP"}


# ----------------------------------------------------------------------------- command line
def _setup(args):
    from jetspec_b200 import JetSpecEngine, DraftHeadTreeDrafter, load_draft_head
    from jetspec_b200.models import Qwen3ForCausalLM, DraftHeadModel, draft_head_config, tiny_config
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    if args.model:
        eng = JetSpecEngine(args.model, device=dev, dtype=dt)
        head = load_draft_head(args.head, device=dev, dtype=dt)
    else:
        cfg = tiny_config()
        eng = JetSpecEngine(Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=dt), device=dev, dtype=dt, use_kernels=False)
        head = DraftHeadModel.random_init(draft_head_config(cfg, 1, args.depth + 1, target_layer_ids=[0, 1]), seed=1,
                                          dtype=dt, device=dev)
    drafter = DraftHeadTreeDrafter(head, eng.model, block_size=args.depth + 1)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.cfg.vocab_size, (1, 24), generator=g) for _ in range(args.samples)]
    return eng, head, drafter, prompts


def main():
    from jetspec_b200 import SamplingParams
    ap = argparse.ArgumentParser()
    ap.add_argument("mode", choices=["diagnostics", "depth-rank", "llm-depth-rank", "conditioned-probe", "verify-split"])
    ap.add_argument("--model", default=None)
    ap.add_argument("--head", default=None)
    ap.add_argument("--depth", type=int, default=4)
    ap.add_argument("--width", type=int, default=2)
    ap.add_argument("--budget", type=int, default=8)
    ap.add_argument("--samples", type=int, default=2)
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--algo", default="accum_logp")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    eng, head, drafter, prompts = _setup(args)
    sp = SamplingParams(0.0, args.max_new)
    kw = dict(tree_depth=args.depth, tree_width=args.width, budget=args.budget, algo=args.algo,
              target_layer_ids=head.target_layer_ids, sampling_params=sp, return_stats=True)
    if args.mode == "diagnostics":
        acc, nodes, toks = [], [0] * (args.depth + 2), 0
        for p in prompts:
            out = eng.generate_tree(p, drafter, tree_diag=True, **kw)
            acc += out["accept_lengths"]
            toks += len(out["token_ids"])
            nodes = [a + b for a, b in zip(nodes, out["tree_nodes_per_depth"] + [0] * len(nodes))]
        m = summarize_tree_diag(accept_lengths=acc, tree_nodes_per_depth=nodes, output_tokens=toks,
                                num_samples=len(prompts), block_size=args.depth + 1, max_depth=args.depth + 1)
        print(format_metrics_report(m, attention_backend=eng.resolved_attn_implementation, block_size=args.depth + 1,
                                    tree_width=args.width, budget=args.budget, algo=args.algo, drafter="draft_head"))
    elif args.mode == "depth-rank":
        hits, trials = [[0] * args.width for _ in range(args.depth)], [0] * args.depth
        for p in prompts:
            rec = RoundRecorder(drafter, args.width)
            out = eng.generate_tree(p, rec, **kw)
            seq = p[0].tolist() + out["token_ids"]
            h, t = depth_rank_counts(rec.rounds, seq, args.width, args.depth)
            hits = [[a + b for a, b in zip(r1, r2)] for r1, r2 in zip(hits, h)]
            trials = [a + b for a, b in zip(trials, t)]
        prof = depth_rank_profile(hits, trials, {"samples": len(prompts), "algo": args.algo})
        text = json.dumps(prof, indent=1)
        if args.out:
            open(args.out, "w").write(text)
        print(text)
    elif args.mode in ("llm-depth-rank", "conditioned-probe"):
        # the reference-engine path (full tree in one masked forward): the hook sees every node of every round
        from jetspec_b200 import LLM
        llm = LLM(eng.model, device=eng.device, dtype=eng.dtype, tokenizer=eng.tokenizer)
        col = LLMRoundCollector(args.width, args.depth, drafter, probe=args.mode == "conditioned-probe")
        for p in prompts:
            llm.generate_tree(p, drafter, block_size=args.depth + 1, tree_width=args.width, budget=args.budget,
                              algo=args.algo, target_layer_ids=head.target_layer_ids, sampling_params=sp,
                              return_text=False, on_round=col)
        if args.mode == "llm-depth-rank":
            text = json.dumps(col.profile({"samples": len(prompts), "algo": args.algo, "width": args.width,
                                           "budget": args.budget, "block_size": args.depth + 1}), indent=1)
            if args.out:
                open(args.out, "w").write(text)
            print(text)
        else:
            print(json.dumps(conditioned_probe_verdict(col.marginal_ranks, col.conditioned_ranks, top=args.width)))
    else:
        ar_t = GpuTimer.patch(eng, "_forward")
        ar = eng.generate(prompts[0], sp)
        ar_s, ar_n = ar_t.total_s(), len(ar["token_ids"])
        ar_t.pairs.clear()
        out = eng.generate_tree(prompts[0], drafter, **kw)
        print(json.dumps({"ar_decode_cuda_s": ar_s, "tree_decode_cuda_s": ar_t.total_s(), "accept_len": out["tpf"],
                          "decode_cuda_speedup": decode_cuda_speedup(ar_s, ar_n, ar_t.total_s(), len(out["token_ids"]))}))


if __name__ == "__main__":
    main()
