"""Ancestor (tree-causal) matrices.

``anc[i, j]`` is true when node ``j`` lies on the path root → ``i`` (``i`` itself
included).  Because parents precede children, one forward sweep that ORs each
row with its parent's row suffices.
"""
from __future__ import annotations

import numpy as np
import torch

from .types import DraftTree


def ancestor_matrix_np(parents, num_nodes: int) -> np.ndarray:
    anc = np.zeros((num_nodes, num_nodes), dtype=np.bool_)
    for i in range(num_nodes):
        p = parents[i]
        if i > 0 and 0 <= p < num_nodes:
            anc[i] = anc[p]
        anc[i, i] = True
    return anc


def ancestor_bits_np(parents, num_nodes: int, words: int) -> np.ndarray:
    """Packed form: ``(num_nodes, words)`` uint32, bit ``j%32`` of word ``j//32`` = ``anc[i, j]``."""
    bits = np.zeros((num_nodes, words), dtype=np.uint32)
    for i in range(num_nodes):
        p = parents[i]
        if i > 0 and 0 <= p < num_nodes:
            bits[i] = bits[p]
        bits[i, i >> 5] |= np.uint32(1) << np.uint32(i & 31)
    return bits


def build_ancestor_matrix(tree: DraftTree) -> torch.Tensor:
    """Bool ``(N, N)`` ancestor matrix on the tree's device (cached on the tree)."""
    if tree.ancestor is None:
        anc = ancestor_matrix_np(tree.parent_indices.tolist(), tree.num_nodes)
        tree.ancestor = torch.from_numpy(anc).to(tree.parent_indices.device)
    return tree.ancestor


def build_packed_ancestor_matrix(tree: DraftTree) -> torch.Tensor:
    """uint8 ``(N, N)`` form of the ancestor matrix."""
    if tree.ancestor_packed is None:
        tree.ancestor_packed = build_ancestor_matrix(tree).to(torch.uint8).contiguous()
    return tree.ancestor_packed
