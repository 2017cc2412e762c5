"""Ragged-batch attention metadata.

Describes one forward over several sequences' new tokens (tree nodes, a prefill
chunk, or one decode token each) to the paged attention op.  Counterpart of
``jetspec/inference_engine/attn_metadata.py:32-144``; the tree mask is carried as
packed ancestor bits (``ceil(N/32)`` words per query row) instead of an fp32
``(total_q, total_q)`` bias: 128 nodes cost 2 KB instead of 64 KB.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..tree.ancestor import ancestor_bits_np


@dataclass
class AttnMeta:
    seq_rows: torch.Tensor      # (B,) int32   slot-map row of each sequence
    cu_q: torch.Tensor          # (B+1,) int32 query-row offsets
    past_lens: torch.Tensor     # (B,) int32   committed KV length of each sequence
    positions: torch.Tensor     # (T,) int32   rotary position of each query row
    slots: torch.Tensor         # (T,) int32   KV slot each new row is written to
    mask_bits: Optional[torch.Tensor]  # (T, words) int32, None when causal
    causal: bool
    max_q: int                  # largest per-sequence query count
    num_tokens: int


def build_attn_metadata(pool, seq_ids: Sequence[int], past_lens: Sequence[int],
                        trees: Optional[Sequence] = None, num_query_nodes: Optional[Sequence[int]] = None,
                        device=None, mask_words: Optional[int] = None) -> AttnMeta:
    """Metadata for one ragged forward.

    ``trees[b]`` (a ``DraftTree``) makes sequence ``b`` a tree verify: row ``i`` sits at
    position ``past + depth[i]`` and sees tree key ``j`` iff ``j`` is an ancestor-or-self.
    With ``trees=None`` every sequence contributes ``num_query_nodes[b]`` causal rows at
    positions ``past, past+1, …`` (prefill chunk or plain decode).
    New row ``i`` of sequence ``b`` is stored at ``slot_map[row_b, past_b + i]``.
    """
    device = device or pool.device
    B = len(seq_ids)
    causal = trees is None
    counts = [int(t.num_nodes) for t in trees] if not causal else [int(n) for n in num_query_nodes]
    cu = np.zeros(B + 1, dtype=np.int32)
    cu[1:] = np.cumsum(counts)
    T = int(cu[-1])
    rows = np.array([pool.state(s).row for s in seq_ids], dtype=np.int32)
    pos = np.empty(T, dtype=np.int32)
    bits = None
    if not causal:
        words = mask_words or max(1, (max(counts) + 31) // 32)
        bits = np.zeros((T, words), dtype=np.uint32)
    slot_rows = []
    for b in range(B):
        s, e, past = int(cu[b]), int(cu[b + 1]), int(past_lens[b])
        if causal:
            pos[s:e] = past + np.arange(e - s, dtype=np.int32)
        else:
            t = trees[b]
            host = getattr(t, "host", None)          # builder's own lists: no device read per sequence
            depth_h = np.asarray(host[2], dtype=np.int32) if host is not None else t.depth.cpu().numpy().astype(np.int32)
            parents_h = host[1] if host is not None else t.parent_indices.tolist()
            pos[s:e] = past + depth_h
            bits[s:e, : max(1, (counts[b] + 31) // 32)] = ancestor_bits_np(
                parents_h, counts[b], max(1, (counts[b] + 31) // 32))
        slot_rows.append(pool.slot_map[int(rows[b]), past:past + (e - s)])
    slots = torch.cat(slot_rows) if slot_rows else torch.zeros(0, dtype=torch.int32, device=device)
    to = lambda a: torch.from_numpy(a).to(device)
    return AttnMeta(
        seq_rows=to(rows), cu_q=to(cu), past_lens=to(np.asarray(past_lens, dtype=np.int32)),
        positions=to(pos), slots=slots,
        mask_bits=(torch.from_numpy(bits.view(np.int32)).to(device) if bits is not None else None),
        causal=causal, max_q=max(counts) if counts else 0, num_tokens=T)
