"""Oracle-mode tree drafter with a seeded, fixed acceptance-length distribution.

Benchmarks on random-init weights cannot use a trained head (nothing would be
accepted), so acceptance is *scripted*: the drafter is given the target's greedy
continuation of the prompt and, each round, draws an accepted length ``a`` from a
geometric distribution (default mean 7).  It then emits per-depth candidates whose
rank-1 token is the true continuation for depths ``< a``, and which exclude the
true token from every rank at depth ``a`` — so the verifier accepts exactly ``a``
tokens plus its own correction.  Candidates are peaked (rank-1 mass 0.9), which
makes the cumulative-logprob builder follow the rank-1 chain to full depth, like
a confident trained head.

The draw depends only on ``(seed, context length)``, so two engines handed the
same drafter see the same trees and the same acceptance sequence.  The drafter
speaks both contracts: dense ``propose_logits`` ``(1, D, V)`` and the direct
``propose_topk`` ``(D, K)`` (the ``TreeDrafter`` contract of ``jetspec/draft.py:36-161``, whose stub drafters play
the same role for plumbing tests: full-accept ``TargetEchoTreeDrafter``, low-accept ``RandomTreeDrafter``).
"""
from __future__ import annotations

import math
import random
import time
from typing import Optional, Sequence

import torch

from .base import TreeDrafter

_BASE_LOGIT = -30.0  # every non-candidate vocabulary entry


class OracleTreeDrafter(TreeDrafter):
    host_scripted = True     # the proposal depends on the context length only: engines may stage it from the host

    def __init__(self, continuation: Sequence[int], vocab_size: int, tree_width: int = 7,
                 mean_accept: float = 7.0, max_accept: Optional[int] = None, seed: int = 0,
                 top1_mass: float = 0.9):
        self.sequence = [int(t) for t in continuation]   # prompt + greedy continuation
        self.vocab_size = int(vocab_size)
        self.tree_width = int(tree_width)
        self.mean_accept = float(mean_accept)
        self.max_accept = max_accept
        self.seed = int(seed)
        w = self.tree_width
        rest = [(1.0 - top1_mass) * 0.5 ** (j + 1) for j in range(max(0, w - 1))]
        self._cand_logits = [math.log(top1_mass)] + [math.log(r) for r in rest]
        self.calls = 0
        self.planned: list = []  # accepted lengths drawn so far (diagnostics)
        self._lp_cache = None
        self._np_cache = None
        self._logit_buf = None       # (key, persistent (1, D, V) logits, indices scattered by the previous call)
        self.host_seconds = 0.0      # host time spent producing proposals (benchmarks report it per round)

    def set_continuation(self, continuation: Sequence[int]) -> None:
        self.sequence = [int(t) for t in continuation]

    def reset_cache(self) -> None:
        self.calls = 0
        self.planned = []

    # -- scripted acceptance ---------------------------------------------------
    def planned_accept(self, context_len: int, depth: int) -> int:
        p = 1.0 / (1.0 + self.mean_accept)
        u = random.Random(self.seed * 1_000_003 + context_len).random()
        a = int(math.log(max(u, 1e-300)) / math.log(1.0 - p)) if p < 1.0 else 0
        cap = depth if self.max_accept is None else min(depth, int(self.max_accept))
        return max(0, min(a, cap))

    def _candidates(self, context_len: int, depth: int):
        """Token ids ``(depth, K)`` (host lists) realising the planned accepted length."""
        V, K = self.vocab_size, self.tree_width
        a = self.planned_accept(context_len, depth)
        self.planned.append(a)
        rows = []
        for d in range(depth):
            pos = context_len + d
            truth = self.sequence[pos] if pos < len(self.sequence) else -1
            start = (context_len * 2_654_435_761 + d * 40_503 + 17) % V
            row, c = [], start
            if d < a and truth >= 0:
                row.append(truth)
            while len(row) < K:
                if c != truth and c not in row:
                    row.append(c)
                c = (c + 1) % V
            rows.append(row)
        return rows

    def _logprobs(self) -> list:
        K, V = self.tree_width, self.vocab_size
        z = sum(math.exp(v) for v in self._cand_logits[:K]) + (V - K) * math.exp(_BASE_LOGIT)
        lse = math.log(z)
        return [v - lse for v in self._cand_logits[:K]]

    # -- drafter contracts -----------------------------------------------------
    def propose_topk(self, context_ids, depth: int, width: Optional[int] = None, target_hidden=None, **kwargs):
        t0 = time.perf_counter()
        self.calls += 1
        T = int(context_ids.shape[-1])
        rows = self._candidates(T, depth)
        lp = self._logprobs()
        dev = context_ids.device
        out = (torch.tensor(rows, dtype=torch.long, device=dev),
               torch.tensor([lp] * depth, dtype=torch.float32, device=dev))
        self.host_seconds += time.perf_counter() - t0
        return out

    def propose_topk_at(self, context_len: int, depth: int, width: Optional[int] = None):
        """The same proposal as :meth:`propose_topk` from the context LENGTH alone (the script depends only on the
        position): ``(tokens (depth, K) int32 array, log-probs (depth, K) list)``.  Engines that stage the top-k on
        the host use this to skip building tensors every round."""
        import numpy as np
        t0 = time.perf_counter()
        self.calls += 1
        T, V, K = int(context_len), self.vocab_size, self.tree_width
        a = self.planned_accept(T, depth)
        self.planned.append(a)
        c = self._np_cache
        if c is None or c[0] != (depth, K) or c[1] is not self.sequence:
            seq = np.full(len(self.sequence) + depth, -1, dtype=np.int64)
            seq[:len(self.sequence)] = self.sequence
            c = self._np_cache = ((depth, K), self.sequence, seq, np.arange(depth, dtype=np.int64) * 40_503 + 17,
                                  np.arange(K + 1, dtype=np.int64)[None, :], np.arange(K, dtype=np.int64)[None, :],
                                  np.arange(depth, dtype=np.int64)[:, None])
        _, _, seq, d_term, kk1, j, rowi = c
        truth = seq[T:T + depth] if T + depth <= len(seq) else np.full(depth, -1, dtype=np.int64)
        start = (T * 2_654_435_761 + d_term) % V
        # K + 1 consecutive fillers per depth, the true token struck out, then the first K (or K - 1 behind the truth)
        cand = (start[:, None] + kk1) % V
        same = cand == truth[:, None]
        hit = np.where(same.any(axis=1), same.argmax(axis=1), K + 1)          # where the truth sits among the fillers
        fill = cand[rowi, j + (j >= hit[:, None])]                            # fillers with the truth skipped
        rows = fill
        if a > 0:
            lead = (rowi[:, 0] < a) & (truth >= 0)
            rows = np.where(lead[:, None], np.concatenate([truth[:, None], fill[:, :K - 1]], axis=1), fill)
        if self._lp_cache is None:
            self._lp_cache = self._logprobs()
        out = rows.astype(np.int32), [self._lp_cache] * depth
        self.host_seconds += time.perf_counter() - t0
        return out

    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        """Dense ``(1, depth, V)`` logits.  The tensor is a persistent buffer that the NEXT call rewrites (only the
        candidate entries change between rounds, so a round costs one small upload and two scatters instead of
        filling ``depth x V`` floats); callers consume it within the round, as every engine here does."""
        t0 = time.perf_counter()
        self.calls += 1
        T = int(context_ids.shape[-1])
        rows = self._candidates(T, depth)
        dev = context_ids.device
        key = (str(dev), int(depth))
        if self._logit_buf is None or self._logit_buf[0] != key:
            vals = torch.tensor(self._cand_logits[: self.tree_width], dtype=torch.float32, device=dev)
            self._logit_buf = [key, torch.full((1, depth, self.vocab_size), _BASE_LOGIT, dtype=torch.float32, device=dev),
                               None, vals.expand(depth, -1).contiguous(),
                               torch.full((depth, self.tree_width), _BASE_LOGIT, dtype=torch.float32, device=dev)]
        _, logits, prev, vals, base = self._logit_buf
        if prev is not None:
            logits[0].scatter_(1, prev, base)
        idx = torch.tensor(rows, dtype=torch.long, device=dev)
        logits[0].scatter_(1, idx, vals)
        self._logit_buf[2] = idx
        self.host_seconds += time.perf_counter() - t0
        return logits


class OracleOverrideDrafter(TreeDrafter):
    """Runs a real drafter for its cost, then substitutes the oracle's candidates.

    The benchmark configuration asks for the real draft head to run every round
    *and* for acceptance to be scripted; this wrapper does both.
    """

    def __init__(self, real: TreeDrafter, oracle: OracleTreeDrafter):
        self.real, self.oracle = real, oracle
        self.block_size = getattr(real, "block_size", None)
        self.target_layer_ids = getattr(real, "target_layer_ids", None)

    def reset_cache(self) -> None:
        if hasattr(self.real, "reset_cache"):
            self.real.reset_cache()
        self.oracle.reset_cache()

    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        real = self.real.propose_logits(context_ids, depth, target_hidden=target_hidden, **kwargs)
        fake = self.oracle.propose_logits(context_ids, depth)
        # keep a data dependency on the real logits so their computation is not skipped
        return fake.to(real.device) + 0.0 * real[..., :1].float()

    def propose_topk(self, context_ids, depth, width=None, target_hidden=None, **kwargs):
        if hasattr(self.real, "propose_topk"):
            self.real.propose_topk(context_ids, depth, width or self.oracle.tree_width, target_hidden=target_hidden)
        else:
            self.real.propose_logits(context_ids, depth, target_hidden=target_hidden)
        return self.oracle.propose_topk(context_ids, depth, width)
