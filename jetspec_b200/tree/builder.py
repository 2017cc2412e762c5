"""Best-first tree construction under a node budget.

Input is the per-depth top-k of the drafter: ``tokens[d][j]`` / ``logprobs[d][j]``
for depth ``d`` and rank ``j``, log-probabilities normalised over the *full*
vocabulary and shared by every parent at that depth.  Expansion order is by
cumulative log-probability (a max-heap, ties broken by insertion order).  Each
expansion of a node at depth ``d`` appends ``min(cap[d], K, budget - n)``
children in rank order.  The budget counts the root.

Behaviour matches ``jetspec/tree/_core/fanout_cap_builder.py:18-75`` and
``jetspec/tree/baselines/accum_logp.py:93-147``; an identical device-side
builder exists for the graph-captured round.
"""
from __future__ import annotations

import heapq
from typing import Optional, Sequence

import torch

from .ancestor import ancestor_matrix_np
from .types import DraftTree


def child_maps_from_lists(tokens: Sequence[int], parents: Sequence[int]) -> list:
    """Per node ``{token: child}``; a later sibling with the same token overrides an earlier one."""
    maps = [dict() for _ in tokens]
    for c in range(1, len(tokens)):
        p = parents[c]
        if 0 <= p < len(tokens):
            maps[p][tokens[c]] = c
    return maps


def expand_best_first(root_token: int, topk_tokens, topk_logprobs, caps: Optional[Sequence[int]], budget: int):
    """Pure-Python expansion; returns ``(tokens, parents, depths, cum_logprobs)`` lists."""
    D = len(topk_tokens)
    K = len(topk_tokens[0]) if D else 0
    tokens, parents, depths, cums = [int(root_token)], [-1], [0], [0.0]
    frontier = [(0.0, 0, 0)]  # (-cum_logprob, insertion order, node)
    order = 0
    while frontier and len(tokens) < budget:
        neg, _, node = heapq.heappop(frontier)
        d = depths[node]
        if d >= D:
            continue
        cap = caps[d] if (caps is not None and d < len(caps)) else K
        take = min(cap, K, budget - len(tokens))
        row_t, row_lp = topk_tokens[d], topk_logprobs[d]
        for j in range(take):
            cum = -neg + row_lp[j]
            idx = len(tokens)
            tokens.append(int(row_t[j]))
            parents.append(node)
            depths.append(d + 1)
            cums.append(cum)
            order += 1
            heapq.heappush(frontier, (-cum, order, idx))
    return tokens, parents, depths, cums


def tree_from_lists(tokens, parents, depths, cums, device) -> DraftTree:
    n = len(tokens)
    if isinstance(device, str) and device == "host":
        # host-only tree for consumers that stage their own device buffers (the batched verify graph): no tensors
        return DraftTree(token_ids=None, parent_indices=None, depth=None, num_nodes=n,
                         host=(list(tokens), list(parents), list(depths)))
    anc = ancestor_matrix_np(parents, n)
    anc_t = torch.from_numpy(anc)
    return DraftTree(
        token_ids=torch.tensor(tokens, dtype=torch.long, device=device),
        parent_indices=torch.tensor(parents, dtype=torch.long, device=device),
        depth=torch.tensor(depths, dtype=torch.long, device=device),
        num_nodes=n,
        cum_logprob=torch.tensor(cums, dtype=torch.float32, device=device) if cums is not None else None,
        child_maps=child_maps_from_lists(tokens, parents),
        ancestor=anc_t.to(device, non_blocking=True),
        ancestor_packed=anc_t.to(torch.uint8).to(device, non_blocking=True),
        host=(list(tokens), list(parents), list(depths)),
    )


def build_with_per_depth_cap(root_token: int, topk_tokens_cpu, topk_logprobs_cpu, b_per_depth, budget: int,
                             device) -> DraftTree:
    """Heap expansion with a per-depth fan-out cap; ``cap >= K`` everywhere is plain ``accum_logp``."""
    t, p, d, c = expand_best_first(root_token, topk_tokens_cpu, topk_logprobs_cpu, b_per_depth, int(budget))
    return tree_from_lists(t, p, d, c, device)


def topk_rows(draft_logits: torch.Tensor, width: int):
    """``log_softmax`` over the vocabulary, then top-``width`` per depth, moved to host lists in
    one transfer (tokens and log-probs stacked as float64, exact for ids below 2**53)."""
    lp = torch.log_softmax(draft_logits.squeeze(0).float(), dim=-1)
    vals, idx = torch.topk(lp, width, dim=-1)
    if vals.device.type == "cpu":
        return idx.tolist(), vals.tolist()
    both = torch.stack((idx.to(torch.float64), vals.to(torch.float64)), -1).cpu()
    return both[..., 0].to(torch.long).tolist(), both[..., 1].tolist()


def _rows(x):
    return x.tolist() if hasattr(x, "tolist") else [list(r) for r in x]      # tensors and numpy arrays alike


def build_from_topk(name: str, root_token: int, topk_tokens, topk_logprobs, budget: int, device,
                    algo_kwargs: Optional[dict] = None, tree_width: Optional[int] = None,
                    **build_kwargs) -> DraftTree:
    """Build the tree of algorithm ``name`` from pre-extracted per-depth top-k.

    The log-probs are used as given (already full-vocabulary normalised), so the
    result equals ``get_algorithm(name).build(dense_logits, …)`` when the top-k came
    from ``log_softmax(dense_logits)`` (reference: ``jetspec/tree/_core/topk_build.py:29-63``).
    """
    from .registry import get_algorithm
    toks, lps = _rows(topk_tokens), _rows(topk_logprobs)
    K = len(lps[0]) if lps else (tree_width or 0)
    algo = get_algorithm(name, **(algo_kwargs or {}))
    caps_fn = getattr(algo, "caps_from_topk", None)
    if caps_fn is None:
        raise NotImplementedError(f"tree algorithm {name!r} has no caps_from_topk")
    caps = caps_fn(lps, tree_width if tree_width is not None else K, **build_kwargs)
    return build_with_per_depth_cap(int(root_token), toks, lps, caps, int(budget), device)
