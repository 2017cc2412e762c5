"""The tree contract shared by every tree algorithm and every engine.

A ``DraftTree`` is a flat list of nodes in *creation order*: a parent always
precedes its children and siblings are contiguous, but nodes are not sorted by
depth.  Node 0 is the root (the anchor token, parent -1, depth 0).  The field
names are those of the reference contract (``jetspec/tree/_core/base.py:17-34``).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch


@dataclass
class DraftTree:
    token_ids: torch.Tensor            # (N,) long
    parent_indices: torch.Tensor       # (N,) long, -1 for the root
    depth: torch.Tensor                # (N,) long, root = 0
    num_nodes: int
    cum_logprob: Optional[torch.Tensor] = None      # (N,) float32
    child_maps: Optional[list] = None               # per node: {token: child index}
    ancestor: Optional[torch.Tensor] = None         # (N, N) bool, self-inclusive
    ancestor_packed: Optional[torch.Tensor] = None  # (N, N) uint8
    ancestor_mask: Optional[torch.Tensor] = None    # optional engine-side precomputed mask
    host: Optional[tuple] = None                    # (tokens, parents, depths) as Python lists when the builder ran on the host


class TreeAlgorithm(ABC):
    """Turns per-depth draft logits ``(1, D, V)`` into a :class:`DraftTree` within ``budget`` nodes.

    ``D = block_size - 1``.  ``refresh_drafter_fn``, ``profile_table`` and
    ``prompt_info`` are optional context an engine may pass; an algorithm must
    tolerate ``None`` (reference: ``jetspec/tree/_core/base.py:37-91``).
    """

    name: str = ""

    @abstractmethod
    def build(self, root_token: int, draft_logits: torch.Tensor, block_size: int, tree_width: int,
              budget: int, device, refresh_drafter_fn: Optional[Callable] = None,
              profile_table: Optional[dict] = None, prompt_info: Optional[dict] = None,
              **kwargs) -> DraftTree:
        ...
