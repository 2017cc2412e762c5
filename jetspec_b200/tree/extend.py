"""Gated tree extension ("ceiling raise").

When the drafter is confident along the best chain, a second, path-conditioned
drafter pass proposes tokens *below* a leaf; those nodes are spliced under it.
Reference: ``jetspec/tree/_core/extend.py:12-225``.
"""
from __future__ import annotations

import torch

from .builder import build_with_per_depth_cap, tree_from_lists
from .types import DraftTree


def should_extend(topk_lp, best_path_ranks, *, gap_threshold: float) -> bool:
    """True when the mean confidence gap along the best path exceeds ``gap_threshold``.

    For a depth where the path uses rank 0 the gap is top-1 minus top-2; for any
    other rank it is that rank minus rank 0 (negative), which suppresses the gate
    for paths that were not locally top-1.
    """
    lp = torch.as_tensor(topk_lp)
    if lp.dim() != 2:
        raise ValueError(f"topk_lp must be (D, K); got {tuple(lp.shape)}")
    ranks = (best_path_ranks.to(lp.device, torch.long) if torch.is_tensor(best_path_ranks)
             else torch.as_tensor(list(best_path_ranks), dtype=torch.long, device=lp.device))
    if ranks.numel() == 0:
        return False
    if ranks.numel() != lp.shape[0]:
        raise ValueError(f"best_path_ranks length {ranks.numel()} must match topk depth {lp.shape[0]}")
    if lp.shape[1] < 2:
        return False
    if bool(((ranks < 0) | (ranks >= lp.shape[1])).any()):
        raise ValueError("best_path_ranks contains a rank outside topk_lp width")
    chosen = lp.gather(1, ranks[:, None]).squeeze(1)
    rival = torch.where(ranks == 0, lp[:, 1], lp[:, 0])
    return bool((chosen - rival).float().mean().item() > float(gap_threshold))


def splice_extension(tree: DraftTree, leaf_index, ext_logits: torch.Tensor, *, ext_budget: int,
                     tree_width: int, mode: str = "chain") -> DraftTree:
    """Return a new tree with ``ext_budget`` nodes appended below ``leaf_index``.

    ``mode="chain"``: the argmax token of each conditioned row, one under the other.
    ``mode="subtree"``: a small ``top2gap_fanout`` tree built from the conditioned
    logits, its synthetic root dropped.
    """
    ext_budget = int(ext_budget)
    if ext_budget < 0:
        raise ValueError("ext_budget must be non-negative")
    if ext_budget == 0:
        return tree
    leaf = int(leaf_index)
    n = int(tree.num_nodes)
    if not 0 <= leaf < n:
        raise IndexError(f"leaf_index {leaf} outside tree with {n} nodes")
    if bool((tree.parent_indices[:n] == leaf).any()):
        raise ValueError(f"leaf_index {leaf} is not a leaf")
    if not torch.is_tensor(ext_logits):
        raise TypeError("ext_logits must be a torch.Tensor")
    if ext_logits.dim() != 3 or ext_logits.shape[0] != 1:
        raise ValueError(f"ext_logits must be (1, D, V); got {tuple(ext_logits.shape)}")
    if ext_logits.shape[2] < 1:
        raise ValueError("ext_logits vocabulary dimension must be non-empty")
    if int(tree_width) < 1:
        raise ValueError("tree_width must be >= 1")
    base_depth = int(tree.depth[leaf])
    base_lp = float(tree.cum_logprob[leaf]) if tree.cum_logprob is not None else 0.0
    if mode == "chain":
        if ext_logits.shape[1] < ext_budget:
            raise ValueError(f"chain extension needs {ext_budget} logit rows; got {ext_logits.shape[1]}")
        lp = torch.log_softmax(ext_logits[0, :ext_budget].float(), dim=-1)
        best_lp, best_tok = lp.max(dim=-1)
        new_tokens = best_tok.tolist()
        new_parents = [leaf] + [n + i for i in range(ext_budget - 1)]
        new_depths = [base_depth + i + 1 for i in range(ext_budget)]
        run, new_cum = base_lp, []
        for v in best_lp.tolist():
            run += v
            new_cum.append(run)
    elif mode == "subtree":
        from .algorithms import Top2GapFanout
        lp = torch.log_softmax(ext_logits[0].float(), dim=-1)
        w = min(int(tree_width), lp.shape[-1])
        vals, idx = torch.topk(lp, w, dim=-1)
        caps = Top2GapFanout().caps_from_topk(vals.tolist(), w)
        sub = build_with_per_depth_cap(int(tree.token_ids[leaf]), idx.tolist(), vals.tolist(), caps,
                                       ext_budget + 1, tree.token_ids.device)
        if sub.num_nodes - 1 != ext_budget:
            raise ValueError(f"subtree extension produced {sub.num_nodes - 1} nodes, expected {ext_budget}")
        sp = sub.parent_indices.tolist()
        new_tokens = sub.token_ids.tolist()[1:]
        new_parents = [leaf if sp[i] == 0 else n + sp[i] - 1 for i in range(1, sub.num_nodes)]
        new_depths = [base_depth + d for d in sub.depth.tolist()[1:]]
        new_cum = [base_lp + c for c in sub.cum_logprob.tolist()[1:]]
    else:
        raise ValueError(f"unknown extension mode {mode!r}; expected 'chain' or 'subtree'")
    tokens = tree.token_ids[:n].tolist() + [int(t) for t in new_tokens]
    parents = tree.parent_indices[:n].tolist() + new_parents
    depths = tree.depth[:n].tolist() + new_depths
    cums = (tree.cum_logprob[:n].tolist() + new_cum) if tree.cum_logprob is not None else None
    return tree_from_lists(tokens, parents, depths, cums, tree.token_ids.device)
