"""Drafters backed by a trained causal-parallel draft head.

One head forward yields logits for ``block_size - 1`` future positions.  The head
borrows the target's embedding table and LM head; the conditioning feature is the
target's tapped hidden states.  Reference: ``jetspec/draft_head_adapter.py:27-206``.

Difference from the reference: the head's context K/V is a persistent cache that is
*extended* with the rows of newly committed tokens on every call (the reference's
graphed variant recomputes the whole padded context each round,
``draft_head_adapter.py:330-348``).  ``propose_topk`` additionally returns the
per-depth top-k with full-vocabulary log-probabilities without ever forming the
``(depth, V)`` logits on the host side.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Drafter, TreeDrafter


class _HeadForward:
    def __init__(self, head, target, block_size: int, target_layer_ids, draft_shift: bool = False):
        self.head, self.target = head, target
        self.block_size = int(block_size)
        self.target_layer_ids = list(target_layer_ids) if target_layer_ids is not None else list(head.target_layer_ids)
        self.draft_shift = bool(draft_shift)
        p = next(head.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.mask_token_id = head.mask_token_id
        self.cache = head.new_cache()
        # the target's tables may live on another device than the head (disaggregated
        # drafting): the drafter then keeps its own copies next to the head
        emb, lmh = target.model.embed_tokens.weight, target.lm_head.weight
        self.embed_w = emb if emb.device == self.device else emb.to(self.device)
        self.lm_head_w = lmh if lmh.device == self.device else lmh.to(self.device)

    def reset_cache(self) -> None:
        self.cache.reset()

    def block_ids(self, context_ids: torch.Tensor, fill_tokens=None) -> torch.Tensor:
        """``[anchor, fill…, mask…]`` of length ``block_size``; the anchor is the last committed token."""
        bs = self.block_size
        if self.mask_token_id is None:
            raise ValueError("draft head config carries no mask_token_id")
        ids = torch.full((bs,), int(self.mask_token_id), dtype=torch.long, device=self.device)
        ids[0] = context_ids.reshape(-1)[-1].to(self.device)
        if fill_tokens is not None:
            path = torch.as_tensor(fill_tokens, dtype=torch.long, device=self.device).reshape(-1)[: bs - 1]
            ids[1:1 + path.numel()] = path
        return ids

    def hidden_rows(self, context_ids, target_hidden, fill_tokens=None) -> torch.Tensor:
        """Advance the context cache to ``target_hidden``'s length, run the block, and return
        the ``block_size - 1`` prediction rows ``(bs-1, H)``."""
        if target_hidden is None:
            raise ValueError("draft-head drafters require target_hidden (tapped target hidden states)")
        th = target_hidden.reshape(-1, target_hidden.shape[-1])
        ctx_len = th.shape[0]
        if self.cache.length > ctx_len:
            self.cache.reset()
        new = th[self.cache.length:].to(device=self.device, dtype=self.dtype)
        self.head.append_context(self.cache, new)
        noise = torch.nn.functional.embedding(self.block_ids(context_ids, fill_tokens), self.embed_w)
        hidden = self.head.forward_block(noise, self.cache)
        bs = self.block_size
        return hidden[: bs - 1] if self.draft_shift else hidden[1:bs]

    def logits(self, context_ids, target_hidden, depth: int, fill_tokens=None) -> torch.Tensor:
        rows = self.hidden_rows(context_ids, target_hidden, fill_tokens)
        return ops.linear(rows[:depth].contiguous(), self.lm_head_w).unsqueeze(0)


class _HeadDrafterMixin:
    def _init(self, head, target, block_size, target_layer_ids, draft_shift):
        self._fwd = _HeadForward(head, target, block_size, target_layer_ids, draft_shift)
        self.head, self.target = head, target
        self.block_size = int(block_size)
        self.target_layer_ids = self._fwd.target_layer_ids
        self.draft_shift = bool(draft_shift)

    def reset_cache(self) -> None:
        self._fwd.reset_cache()


class DraftHeadDrafter(_HeadDrafterMixin, Drafter):
    """Chain drafter: argmax of each per-position draft logit row."""

    def __init__(self, head, target, block_size: int, target_layer_ids=None, draft_shift: bool = False):
        self._init(head, target, block_size, target_layer_ids, draft_shift)

    @torch.inference_mode()
    def propose(self, context_ids, k, target_hidden=None, **kwargs):
        rows = self._fwd.hidden_rows(context_ids, target_hidden)[:k].contiguous()
        idx, _ = ops.lm_head_argmax(rows, self._fwd.lm_head_w)
        return idx


class DraftHeadTreeDrafter(_HeadDrafterMixin, TreeDrafter):
    """Tree drafter: raw per-depth logits (or their top-k) from one head forward."""

    def __init__(self, head, target, block_size: int, target_layer_ids=None, draft_shift: bool = False):
        self._init(head, target, block_size, target_layer_ids, draft_shift)

    @torch.inference_mode()
    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        return self._fwd.logits(context_ids, target_hidden, depth)

    @torch.inference_mode()
    def propose_logits_conditioned(self, context_ids, path_tokens, target_hidden=None, **kwargs):
        return self._fwd.logits(context_ids, target_hidden, self.block_size - 1, fill_tokens=path_tokens)

    @torch.inference_mode()
    def propose_topk(self, context_ids, depth, width: int, target_hidden=None, **kwargs):
        """``(tokens (depth, width), logprobs (depth, width))`` with full-vocabulary log-probs."""
        rows = self._fwd.hidden_rows(context_ids, target_hidden)[:depth].contiguous()
        return ops.lm_head_topk_logprobs(rows, self._fwd.lm_head_w, width)


class GraphedDraftHead(DraftHeadTreeDrafter):
    """Draft head whose step is replayed from a CUDA graph.

    In the reference this is a separate wrapper that owns one graph per context bucket and
    recomputes the padded context every round (``jetspec/draft_head_adapter.py:446-602``).  Here the
    engine's kernel path already captures the head's step inside the round's graph and extends a
    persistent context K/V cache, so this class only marks the intent: handing it to
    ``JetSpecEngine.generate_tree`` on a GPU selects the in-graph head; on CPU it behaves as the
    eager :class:`DraftHeadTreeDrafter`.  ``propose`` gives the chain (argmax) view.
    """

    @torch.inference_mode()
    def propose(self, context_ids, k, target_hidden=None, **kwargs):
        return self.propose_logits(context_ids, k, target_hidden=target_hidden)[0].argmax(-1)

    def clone(self) -> "GraphedDraftHead":
        """A drafter sharing the weights but with its own context cache (one per sequence in a batch)."""
        return type(self)(self.head, self.target, self.block_size, self.target_layer_ids, self.draft_shift)


class CompiledDraftHead(GraphedDraftHead):
    """Name kept for API parity with the reference's ``torch.compile`` variant
    (``jetspec/draft_head_adapter.py:225-443``); there is no tracing compiler here, the kernels are
    the same hand-written ones."""
