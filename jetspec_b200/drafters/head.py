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


# context capacities a graphed head is captured for (the next one up is taken when a context outgrows the current)
CTX_BUCKETS = (512, 1024, 2048, 4096, 8192, 16384, 32768)


def ctx_bucket(n: int) -> int:
    for b in CTX_BUCKETS:
        if n <= b:
            return b
    step = CTX_BUCKETS[-1]
    return ((n + step - 1) // step) * step


class GraphedDraftHead(DraftHeadTreeDrafter):
    """Draft head whose step is ONE CUDA-graph replay, usable on its own (any engine, any batch member).

    Counterpart of the reference's wrapper with one graph per context bucket
    (``jetspec/draft_head_adapter.py:446-602``, buckets ``:208-222``).  Differences: the captured step is this
    framework's kernel sequence (context update for the NEW rows only: fc GEMM, RMSNorm, fused K|V GEMM, per-head
    norm + RoPE + scatter into a persistent context K/V cache; block forward; LM-head top-k epilogue), so a round
    costs O(new rows), not O(context); the graph is captured per context *capacity* (the cache it addresses) and
    requested top-k width; the host stages the new tapped rows, the anchor token and three integers per call.
    A prompt longer than one block goes through the same kernels eagerly once.  On a CPU (or with weights the
    kernels do not cover) every method falls back to the eager :class:`DraftHeadTreeDrafter`.
    ``JetSpecEngine.generate_tree`` on a GPU recognises the class and captures the head inside its own round graph.
    """

    def __init__(self, head, target, block_size: int, target_layer_ids=None, draft_shift: bool = False):
        super().__init__(head, target, block_size, target_layer_ids, draft_shift)
        self._gs = None            # graph state: stub runner, buffers, graphs per (width, want_topk)
        self.replays = 0

    # ---- capability and state ---------------------------------------------------------------
    def _graph_ok(self) -> bool:
        p = self.head.fc.weight
        if not (p.is_cuda and p.dtype == torch.bfloat16) or getattr(self.head, "hidden_dim_adapter", None) is not None:
            return False
        hc = self.head.config
        return hc.head_dim == 128 and self.block_size - 1 <= 48

    def _state(self, need_ctx: int):
        cap = ctx_bucket(need_ctx + 2 * self.block_size)
        if self._gs is not None and self._gs["cap"] >= cap:
            return self._gs
        import types
        from ..engine.fast_round import FastRound
        fr = FastRound.__new__(FastRound)
        dev = self.head.fc.weight.device
        fr.device, fr.draft_cache, fr.tp = torch.device(dev), {}, None
        fr.cfg = types.SimpleNamespace(vocab_size=self._fwd.lm_head_w.shape[0])
        fr.eng = types.SimpleNamespace(pool=types.SimpleNamespace(max_seq_len=cap))
        bs, i32 = self.block_size, torch.int32
        tapw = len(self.target_layer_ids) * self.head.config.hidden_size
        r = {"K": 8, "head": self, "state": torch.zeros(8, dtype=i32, device=dev),
             "committed": torch.zeros(8, dtype=i32, device=dev),
             "taps": torch.zeros(bs, tapw, dtype=torch.bfloat16, device=dev),
             "path_idx": torch.arange(bs, dtype=i32, device=dev)}
        fr._draft_buffers(r, self)
        self._gs = {"cap": cap, "fr": fr, "r": r, "graphs": {}, "ctx": 0,
                    "stage": torch.zeros(16, dtype=i32).pin_memory(), "stage_dev": torch.zeros(16, dtype=i32, device=dev)}
        return self._gs

    def reset_cache(self) -> None:
        super().reset_cache()
        if self._gs is not None:
            self._gs["ctx"] = 0

    def clone(self) -> "GraphedDraftHead":
        """A drafter sharing the weights but with its own context cache and graphs (one per sequence in a batch)."""
        return type(self)(self.head, self.target, self.block_size, self.target_layer_ids, self.draft_shift)

    # ---- one graphed step -------------------------------------------------------------------
    def _step(self, context_ids, target_hidden, want_topk: bool):
        from ..engine.fast_round import ST_CTX, ST_NEW, ST_PAST, _PDL
        if target_hidden is None:
            raise ValueError("draft-head drafters require target_hidden (tapped target hidden states)")
        th = target_hidden.reshape(-1, target_hidden.shape[-1])
        n = th.shape[0]
        gs = self._state(n)
        fr, r, bs = gs["fr"], gs["r"], self.block_size
        if gs["ctx"] > n:
            gs["ctx"] = 0
        new = n - gs["ctx"]
        if new > bs:                    # a prompt (or a long jump): bulk rows through the eager kernel path
            fr._draft_prompt_context(r, th, start=gs["ctx"])
            gs["ctx"], new = n, 0
        if new:
            r["taps"][:new].copy_(th[gs["ctx"]:n])
        if gs.get("staged") is not None:
            gs["staged"].synchronize()      # the previous call's upload has left the pinned words
        h = gs["stage"]
        h.zero_()
        h[ST_PAST], h[ST_CTX], h[ST_NEW] = 0, gs["ctx"], new
        h[8] = int(context_ids.reshape(-1)[-1])
        gs["stage_dev"].copy_(h, non_blocking=True)
        key = bool(want_topk)
        g = gs["graphs"].get(key)
        if g is None:
            r["no_topk"] = not want_topk
            self._launch(gs, pdl=False)                  # module load, function attributes
            torch.cuda.synchronize()
            gs["stage_dev"].copy_(h, non_blocking=True)   # the warm-up consumed ST_NEW: stage again for the replay
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch(gs, pdl=_PDL)
            gs["graphs"][key] = g
        r["no_topk"] = not want_topk
        if gs.get("staged") is None:
            gs["staged"] = torch.cuda.Event()
        gs["staged"].record()
        g.replay()
        self.replays += 1
        gs["ctx"] = n
        return r["draft"]

    def _launch(self, gs, pdl: bool) -> None:
        r = gs["r"]
        r["state"].copy_(gs["stage_dev"][:8])
        r["committed"][:1].copy_(gs["stage_dev"][8:9])
        gs["fr"]._launch_draft(r, pdl)

    # ---- drafter contracts ------------------------------------------------------------------
    @torch.inference_mode()
    def propose_topk(self, context_ids, depth, width: int, target_hidden=None, **kwargs):
        if not self._graph_ok():
            return super().propose_topk(context_ids, depth, width, target_hidden=target_hidden, **kwargs)
        d = self._step(context_ids, target_hidden, want_topk=True)
        # the graph scores the 8 best per depth (sorted); a narrower request is a prefix of each row
        return d["topk_tok"][:depth, :width].long(), d["topk_lp"][:depth, :width].clone()

    @torch.inference_mode()
    def propose_logits(self, context_ids, depth, target_hidden=None, **kwargs):
        if not self._graph_ok():
            return super().propose_logits(context_ids, depth, target_hidden=target_hidden, **kwargs)
        d = self._step(context_ids, target_hidden, want_topk=False)
        bs = self.block_size
        rows = d["hn"][:bs - 1] if self.draft_shift else d["hn"][1:bs]
        return ops.linear(rows[:depth].contiguous(), self._fwd.lm_head_w).unsqueeze(0)

    @torch.inference_mode()
    def propose(self, context_ids, k, target_hidden=None, **kwargs):
        return self.propose_logits(context_ids, k, target_hidden=target_hidden)[0].argmax(-1)


class CompiledDraftHead(GraphedDraftHead):
    """Name kept for API parity with the reference's ``torch.compile`` variant
    (``jetspec/draft_head_adapter.py:225-443``); there is no tracing compiler here: the step is the same
    hand-written kernel sequence, replayed from a CUDA graph exactly as in :class:`GraphedDraftHead`."""
