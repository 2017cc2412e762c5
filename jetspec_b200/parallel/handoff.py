"""Target GPU <-> draft-head GPU handoff.

The reference cannot place the draft head on another GPU (its adapter calls the target's
``embed_tokens`` / ``lm_head`` with head-device tensors, ``jetspec/draft_head_adapter.py:54,73,129``).
Here the head runs in its own process on its own GPU with its own copies of the two tables:

* the target's layer-epilogue copy kernel writes the tapped residual rows of all tree nodes straight
  into the drafter GPU's ``taps`` buffer (its destination is a peer address);
* after acceptance the target pushes a header ``[new rows, anchor token, done]`` plus the accepted
  path's node indices, then release-stores a round number at the drafter;
* the drafter's graph waits for that round number, appends the accepted rows to its context K/V,
  runs the block and pushes the per-depth top-k (tokens, full-vocabulary log-probs) into the
  target's buffer, release-storing a round number back; the target's graph waits for it before the
  tree build.

Prompt-time hidden states (one transfer per request) travel by NCCL point-to-point.
All device waits are bounded (status word).  Control words live in one 4 KB buffer per rank:
ints ``[0:4]`` header, ``[16:80]`` path indices, ``[128]`` header flag, ``[129]`` top-k flag.
"""
from __future__ import annotations

import torch

from .symm import SymmetricBuffer

HDR, PATH, HDR_FLAG, TOPK_FLAG = 0, 16, 128, 129


class HandoffChannel:
    """Both ranks of a (target, drafter) pair construct this with identical arguments."""

    def __init__(self, group, nodes: int, tap_width: int, depth: int, width: int, target_rank: int = 0,
                 draft_rank: int = 1):
        import torch.distributed as dist
        from ..ops import cuda_ext as X
        self._X, self.group = X, group
        self.rank = dist.get_rank(group)
        self.target_rank, self.draft_rank = target_rank, draft_rank
        self.is_target = self.rank == target_rank
        self.peer = draft_rank if self.is_target else target_rank
        self.nodes, self.tap_width, self.depth, self.width = nodes, tap_width, depth, width
        self.taps_buf = SymmetricBuffer(nodes * tap_width * 2, group)
        self.ctrl_buf = SymmetricBuffer(4096, group)
        self.topk_buf = SymmetricBuffer(max(64, depth * width * 8), group)
        i32 = torch.int32
        self.ctrl_local = self.ctrl_buf.tensor(self.rank, (1024,), i32)
        self.ctrl_peer = self.ctrl_buf.tensor(self.peer, (1024,), i32)
        # what the TARGET writes into: the drafter's tap rows
        self.taps_on_drafter = self.taps_buf.tensor(draft_rank, (nodes, tap_width), torch.bfloat16)
        # what the DRAFTER writes into: the target's top-k (tokens, then log-prob bits)
        self.topk_on_target = self.topk_buf.tensor(target_rank, (2, depth, width), i32)
        self.epoch_wait = torch.zeros(1, dtype=i32, device="cuda")
        self.epoch_push = torch.zeros(1, dtype=i32, device="cuda")
        self.header_tmp = torch.zeros(4, dtype=i32, device="cuda")
        self._warm()

    def _warm(self) -> None:
        """Launch every handoff kernel once on private scratch so none is first loaded inside a graph capture."""
        X = self._X
        lib = X.load()
        a = torch.zeros(8, dtype=torch.int32, device="cuda")
        b = torch.zeros(8, dtype=torch.int32, device="cuda")
        f = torch.ones(1, dtype=torch.int32, device="cuda")
        e = torch.zeros(1, dtype=torch.int32, device="cuda")
        e2 = torch.zeros(1, dtype=torch.int32, device="cuda")     # kept alive until the kernels have run
        status = X.status_word("cuda")
        s = X._stream()
        lib.js_push_words(X._p(a), X._p(b), 8, 0, s)
        lib.js_flag_push(X._p(b), X._p(e), 0, s)
        lib.js_flag_wait(X._p(f), X._p(e2), X._p(status), 0, s)
        lib.js_make_header(X._p(a), X._p(b), X._p(a[4:]), 0, s)
        lib.js_draft_apply_header(X._p(a), X._p(b), X._p(a[4:]), 0, s)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ per request
    def reset(self) -> None:
        """Zero flags and round numbers on both sides (call at the start of every request)."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.ctrl_local.zero_()
        self.epoch_wait.zero_()
        self.epoch_push.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ target side (graph-capturable)
    def target_wait_topk(self, pdl=False):
        X = self._X
        X._check(X.load().js_flag_wait(X._p(self.ctrl_local[TOPK_FLAG:]), X._p(self.epoch_wait),
                                       X._p(X.status_word("cuda")), int(pdl), X._stream()), "js_flag_wait")

    def target_push_header(self, state, committed, path_idx, pdl=False):
        X = self._X
        lib = X.load()
        X._check(lib.js_make_header(X._p(state), X._p(committed), X._p(self.header_tmp), int(pdl), X._stream()), "hdr")
        X._check(lib.js_push_words(X._p(self.header_tmp), X._p(self.ctrl_peer[HDR:]), 4, int(pdl), X._stream()), "push")
        X._check(lib.js_push_words(X._p(path_idx), X._p(self.ctrl_peer[PATH:]), 64, int(pdl), X._stream()), "push")
        X._check(lib.js_flag_push(X._p(self.ctrl_peer[HDR_FLAG:]), X._p(self.epoch_push), int(pdl), X._stream()), "flag")

    def target_push_raw_header(self, n_new: int, anchor: int, done: int):
        """Eager header (after prefill, and the final ``done`` notice)."""
        X = self._X
        lib = X.load()
        self.header_tmp.copy_(torch.tensor([n_new, anchor, done, 0], dtype=torch.int32))
        X._check(lib.js_push_words(X._p(self.header_tmp), X._p(self.ctrl_peer[HDR:]), 4, 0, X._stream()), "push")
        X._check(lib.js_flag_push(X._p(self.ctrl_peer[HDR_FLAG:]), X._p(self.epoch_push), 0, X._stream()), "flag")

    # ------------------------------------------------------------------ drafter side (graph-capturable)
    def draft_wait_header(self, state, committed, pdl=False):
        X = self._X
        lib = X.load()
        X._check(lib.js_flag_wait(X._p(self.ctrl_local[HDR_FLAG:]), X._p(self.epoch_wait), X._p(X.status_word("cuda")),
                                  int(pdl), X._stream()), "js_flag_wait")
        X._check(lib.js_draft_apply_header(X._p(self.ctrl_local[HDR:]), X._p(state), X._p(committed), int(pdl),
                                           X._stream()), "apply header")

    def draft_push_topk(self, tok: torch.Tensor, lp: torch.Tensor, pdl=False):
        X = self._X
        lib = X.load()
        n = self.depth * self.width
        X._check(lib.js_push_words(X._p(tok), X._p(self.topk_on_target[0]), n, int(pdl), X._stream()), "push tok")
        X._check(lib.js_push_words(X._p(lp), X._p(self.topk_on_target[1]), n, int(pdl), X._stream()), "push lp")
        X._check(lib.js_flag_push(X._p(self.ctrl_peer[TOPK_FLAG:]), X._p(self.epoch_push), int(pdl), X._stream()), "flag")

    @property
    def path_on_drafter(self) -> torch.Tensor:
        return self.ctrl_local[PATH:PATH + 64]

    def close(self):
        for b in (self.taps_buf, self.ctrl_buf, self.topk_buf):
            b.close()
