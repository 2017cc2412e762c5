"""Ancestor (tree-causal) matrices.

``anc[i, j]`` is true when node ``j`` lies on the path root → ``i`` (``i`` itself
included).  Because parents precede children, one forward sweep that ORs each
row with its parent's row suffices.  Reference counterpart: ``jetspec/tree/_core/ancestor.py:19-55`` (bool and
uint8-packed matrices); the int32 bit words the attention kernels read are this framework's own.
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


def pack_ancestor_bits(ancestor: torch.Tensor) -> torch.Tensor:
    """Bool ``(N, N)`` matrix -> ``(N, ceil(N/32))`` int32 words, bit ``j % 32`` of word ``j // 32`` = ``anc[i, j]``:
    the mask format of the tree-attention kernels.  Works on the matrix's own device (no host round trip)."""
    n = ancestor.shape[0]
    words = max(1, (n + 31) // 32)
    pad = torch.zeros(n, words * 32, dtype=torch.int64, device=ancestor.device)
    pad[:, :n] = ancestor.to(torch.int64)
    weights = (torch.ones(32, dtype=torch.int64, device=ancestor.device) << torch.arange(32, device=ancestor.device))
    packed = (pad.view(n, words, 32) * weights).sum(-1)                  # values in [0, 2^32)
    packed = torch.where(packed >= (1 << 31), packed - (1 << 32), packed)   # reinterpret as signed 32-bit
    return packed.to(torch.int32).contiguous()
