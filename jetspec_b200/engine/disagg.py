"""Disaggregated drafting: target on one GPU (process), draft head on another.

Target process::

    chan = HandoffChannel(group, nodes=bucket_for_n(budget), tap_width=len(taps) * H, depth=D, width=K)
    drafter = RemoteDraftHead(chan, target_layer_ids=taps, block_size=D + 1, oracle=None)
    engine.generate_tree(prompt, drafter, tree_depth=D, tree_width=K, budget=budget, ...)

Drafter process::

    DraftWorker(head, embed_weight, lm_head_weight, chan, width=K).serve()    # one request

Both replay CUDA graphs; see :mod:`jetspec_b200.parallel.handoff` for the protocol.  The reference keeps the head on
the target's device because it borrows the target's embedding and LM-head modules
(``jetspec/draft_head_adapter.py:54,73,129``); here the drafter process holds its own copies of the two matrices.
"""
from __future__ import annotations

import types
from typing import Optional

import torch

from ..drafters.base import TreeDrafter
from ..drafters.head import DraftHeadTreeDrafter
from ..ops import cuda_ext as X
from ..ops import reference as ref

ST_PAST, ST_CTX, ST_NEW, ST_DONE = 0, 1, 2, 3


class RemoteDraftHead(TreeDrafter):
    """Handle of a draft head that runs on another GPU; only the engine's graph path can drive it."""

    def __init__(self, channel, target_layer_ids, block_size: int, oracle=None):
        self.channel = channel
        self.target_layer_ids = list(target_layer_ids)
        self.block_size = int(block_size)
        self.oracle = oracle

    def reset_cache(self):
        if self.oracle is not None:
            self.oracle.reset_cache()

    def propose_logits(self, context_ids, depth, target_hidden=None, **kw):
        raise RuntimeError("a remote draft head is driven by the engine's graph path, not called directly")


class DraftWorker:
    """The drafter GPU's side: serves draft steps for one request at a time."""

    def __init__(self, head_model, embed_w: torch.Tensor, lm_head_w: torch.Tensor, channel, width: int,
                 vocab_size: int, max_ctx: int = 4096, draft_shift: bool = False):
        from .fast_round import FastRound, _PDL
        self.channel, self.width = channel, int(width)
        dev = embed_w.device
        stub_target = types.SimpleNamespace(model=types.SimpleNamespace(embed_tokens=types.SimpleNamespace(weight=embed_w)),
                                            lm_head=types.SimpleNamespace(weight=lm_head_w))
        self.drafter = DraftHeadTreeDrafter(head_model, stub_target, block_size=channel.depth + 1, draft_shift=draft_shift)
        fr = FastRound.__new__(FastRound)
        fr.device, fr.draft_cache, fr.tp = torch.device(dev), {}, None
        fr.cfg = types.SimpleNamespace(vocab_size=vocab_size)
        fr.eng = types.SimpleNamespace(pool=types.SimpleNamespace(max_seq_len=max_ctx))
        self.fr = fr
        i32 = torch.int32
        self.r = {"K": self.width, "head": self.drafter, "state": torch.zeros(8, dtype=i32, device=dev),
                  "committed": torch.zeros(8, dtype=i32, device=dev),
                  "taps": channel.taps_buf.tensor(channel.rank, (channel.nodes, channel.tap_width), torch.bfloat16),
                  "path_idx": channel.path_on_drafter}
        fr._draft_buffers(self.r, self.drafter)
        self._pdl = _PDL
        self.graph = None
        self.done_host = torch.zeros(8, dtype=i32).pin_memory()

    def _step(self, pdl: bool):
        ch, r = self.channel, self.r
        ch.draft_wait_header(r["state"], r["committed"], pdl)
        self.fr._launch_draft(r, pdl)
        d = r["draft"]
        D = ch.depth
        ch.draft_push_topk(d["topk_tok"], d["topk_lp"].view(torch.int32), pdl)
        self.done_host.copy_(r["state"], non_blocking=True)

    @torch.inference_mode()
    def load_context(self, hidden: torch.Tensor) -> None:
        """Project the prompt's tapped hidden rows into the head's context K/V (once per request)."""
        n = self.fr._draft_prompt_context(self.r, hidden)     # the same kernels as the in-graph context update
        st = torch.zeros(8, dtype=torch.int32)
        st[ST_CTX] = n
        self.r["state"].copy_(st)

    @torch.inference_mode()
    def serve(self, max_rounds: int = 1 << 20) -> int:
        """Serve one request: receive the prompt's hidden rows, then answer draft steps until the target
        reports ``done``.  Returns the number of steps served."""
        import torch.distributed as dist
        ch = self.channel
        ch.reset()
        meta = torch.zeros(2, dtype=torch.int64, device="cuda")
        dist.recv(meta, src=ch.target_rank, group=ch.group)
        T, w = int(meta[0]), int(meta[1])
        hidden = torch.empty(T, w, dtype=torch.bfloat16, device="cuda")
        dist.recv(hidden, src=ch.target_rank, group=ch.group)
        self.load_context(hidden)
        torch.cuda.synchronize()
        done_view = self.done_host.numpy()
        steps = 0
        stream = torch.cuda.current_stream()
        if self.graph is None:
            # the very first step runs eagerly (it loads every kernel), the rest replay its capture
            self._step(False)
            stream.synchronize()
            steps = 1
            X.check_status("cuda")
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step(self._pdl)
            self.graph = g
            if int(done_view[ST_DONE]) != 0:
                return steps
        while steps < max_rounds:
            self.graph.replay()
            stream.synchronize()
            steps += 1
            X.check_status("cuda")
            if int(done_view[ST_DONE]) != 0:
                break
        return steps
