"""Drafter contracts and the model-free stub drafters.

Speculative decoding here is lossless: only tokens the target itself would emit
are committed, so *any* drafter, however bad, must reproduce plain greedy output.
The stubs exist to exercise the verify / accept / commit plumbing
(reference: ``jetspec/draft.py:20-161``).
"""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch


class Drafter(ABC):
    """Chain drafter: proposes the next ``k`` tokens."""

    @abstractmethod
    def propose(self, context_ids: torch.Tensor, k: int, target_hidden: torch.Tensor = None, **kwargs) -> torch.Tensor:
        """``context_ids (1, T)`` → ``(k,)`` proposed token ids.  ``target_hidden``
        ``(1, T-1, taps*H)`` is what a real draft head conditions on; stubs ignore it."""


class TreeDrafter(ABC):
    """Tree drafter: emits per-depth logits ``(1, depth, V)``; a tree algorithm shapes the tree."""

    @abstractmethod
    def propose_logits(self, context_ids: torch.Tensor, depth: int, target_hidden: torch.Tensor = None,
                       **kwargs) -> torch.Tensor:
        ...


class RepeatDrafter(Drafter):
    """Repeats the last context token ``k`` times (usually rejected: tests the rollback path)."""

    def propose(self, context_ids, k, target_hidden=None, **kwargs):
        return context_ids[0, -1].repeat(k)


class RandomTreeDrafter(TreeDrafter):
    """Gaussian per-depth logits → a random tree."""

    def __init__(self, vocab_size: int, seed: int | None = None):
        self.vocab_size = vocab_size
        self._gen = torch.Generator().manual_seed(seed) if seed is not None else None

    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        x = torch.randn(1, depth, self.vocab_size, generator=self._gen)
        return x.to(context_ids.device)


class _EchoBase:
    def __init__(self, model):
        self.model = model

    def _rollout(self, context_ids: torch.Tensor, steps: int):
        """Greedy-decode ``steps`` tokens with the target itself; yields the logits row of each step."""
        from ..core.model_runner import ModelRunner
        runner = ModelRunner(self.model)
        ids = context_ids.reshape(1, -1)
        cache = runner.new_cache(ids.shape[1] + steps + 1)
        logits, cache, _ = runner.forward(ids, cache, last_position_logits_only=True)
        rows = [logits[0, -1]]
        for _ in range(steps - 1):
            nxt = rows[-1].argmax().reshape(1, 1)
            logits, cache, _ = runner.forward(nxt, cache, last_position_logits_only=True)
            rows.append(logits[0, -1])
        return rows


class TargetEchoDrafter(_EchoBase, Drafter):
    """Proposes the target's own greedy next ``k`` tokens: every draft is accepted."""

    @torch.inference_mode()
    def propose(self, context_ids, k, target_hidden=None, **kwargs):
        return torch.stack([r.argmax() for r in self._rollout(context_ids, k)])


class TargetEchoTreeDrafter(_EchoBase, TreeDrafter):
    """Per-depth logits = the target's own greedy-rollout logits: the rank-1 chain is fully accepted."""

    @torch.inference_mode()
    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        return torch.stack(self._rollout(context_ids, depth)).unsqueeze(0)
