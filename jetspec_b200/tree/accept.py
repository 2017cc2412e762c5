"""Lossless acceptance: find the longest root-to-leaf path the target agrees with.

Greedy rule: node ``i`` matches when its token equals the target's argmax at its
parent and no *later* sibling carries the same (parent, token) pair (the later
one wins, as a ``dict`` child map would make it).  The accepted node is the
deepest node whose whole root path matches; the correction token is the
target's argmax at that node.  Reference: ``jetspec/tree/_core/accept.py:73-183``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .builder import child_maps_from_lists
from .types import DraftTree


def _posterior(logits: torch.Tensor, temperature: float, generator=None) -> torch.Tensor:
    if temperature <= 0.0:
        return logits.argmax(dim=-1)
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    flat = probs.reshape(-1, probs.shape[-1])
    return torch.multinomial(flat, 1, generator=generator).squeeze(-1).reshape(probs.shape[:-1])


def tree_accept(tree: DraftTree, target_logits: torch.Tensor, temperature: float = 0.0, generator=None):
    """Host walk over the child maps.

    ``target_logits`` is ``(1, N, V)`` (or ``(N, V)``; extra leading rows are
    dropped).  With ``temperature > 0`` one token is sampled per node and the walk
    follows the sampled tokens.  Returns ``(accepted_path, acceptance_length,
    correction_token)`` — path is root-inclusive node indices.
    """
    logits = target_logits.reshape(-1, target_logits.shape[-1])
    n = tree.num_nodes
    if logits.shape[0] < n:
        raise ValueError(f"target_logits has {logits.shape[0]} positions, expected at least {n}")
    logits = logits[-n:]
    post = [int(t) for t in _posterior(logits, temperature, generator).reshape(-1).tolist()]
    if tree.child_maps is None:
        tree.child_maps = child_maps_from_lists(tree.token_ids.tolist(), tree.parent_indices.tolist())
    path, cur = [0], 0
    while True:
        nxt = tree.child_maps[cur].get(post[cur])
        if nxt is None:
            break
        path.append(nxt)
        cur = nxt
    return path, len(path) - 1, post[cur]


def gpu_tree_accept(tree_tokens: torch.Tensor, greedy_targets: torch.Tensor, parent_indices: torch.Tensor,
                    depths: torch.Tensor, max_depth: Optional[int] = None):
    """Vectorised greedy acceptance on flat tensors with a single host read.

    Returns ``(accepted_path LongTensor(L,), accepted_len int, correction 0-d tensor)``.
    """
    dev = tree_tokens.device
    n = tree_tokens.shape[0]
    greedy = greedy_targets.reshape(-1)
    if n <= 1:
        return torch.zeros(1, dtype=torch.long, device=dev), 0, greedy[0]
    if max_depth is None:
        max_depth = n - 1
    ids = torch.arange(n, device=dev)
    par = parent_indices.clamp(0, n - 1)
    has_parent = (parent_indices >= 0) & (parent_indices < n)
    dup_later = ((parent_indices[:, None] == parent_indices[None, :])
                 & (tree_tokens[:, None] == tree_tokens[None, :])
                 & (ids[None, :] > ids[:, None])).any(dim=1)
    ok = has_parent & ~dup_later & (tree_tokens == greedy[par])
    ok[0] = True
    # pointer jumping: after r rounds ok[i] covers 2**r ancestors
    hop = par.clone()
    for _ in range(max(1, int(max_depth).bit_length())):
        ok = ok & ok[hop]
        hop = hop[hop]
    score = torch.where(ok, depths, torch.full_like(depths, -1))
    best = torch.argmax(score)
    correction = greedy[best]
    chain = torch.empty(max_depth + 1, dtype=torch.long, device=dev)
    cur = best.reshape(1)
    for d in range(max_depth, -1, -1):
        chain[d:d + 1] = cur
        cur = par[cur]
    acc = int(depths[best].item())
    return chain[max_depth - acc:max_depth + 1].contiguous(), acc, correction


def host_tree_accept(tokens, parents, depths, greedy):
    """Greedy acceptance on Python lists: the rule of :func:`gpu_tree_accept` (a node matches when its token is the
    target's argmax at its parent and no LATER sibling carries the same token; the deepest fully matching root
    path wins, lowest index on equal depth) without a kernel launch or a device read.  ``greedy[i]`` is the
    target's argmax at node ``i``.  Returns ``(path list, accepted_len, correction)``."""
    n = len(tokens)
    last = {}
    for i in range(1, n):
        last[(parents[i], tokens[i])] = i            # the later of two equal siblings wins
    ok = [False] * n
    ok[0] = True
    best, best_d = 0, 0
    for i in range(1, n):                            # parents precede children
        p = parents[i]
        if 0 <= p < i and ok[p] and tokens[i] == greedy[p] and last[(p, tokens[i])] == i:
            ok[i] = True
            if depths[i] > best_d:
                best, best_d = i, depths[i]
    path = []
    c = best
    while c >= 0:
        path.append(c)
        c = parents[c]
    path.reverse()
    return path, best_d, int(greedy[best])
