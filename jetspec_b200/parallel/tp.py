"""Tensor parallelism for the verify forward.

Sharding plan (``world`` ranks, one process per GPU):

* QKV and gate/up projections are column-parallel (each rank owns ``Hq/world`` query heads,
  ``Hkv/world`` KV heads and ``I/world`` MLP channels, so attention and the KV pool are local);
* ``o_proj`` and ``down_proj`` are row-parallel: every rank multiplies its K-slice and the
  partial products are summed by an all-reduce whose first half is FUSED into the GEMM epilogue —
  finished tiles are stored into peers' buffers over NVLink from inside the kernel
  (``csrc/gemm_sm100.cu``, ``EPI_ALLREDUCE``) — and whose second half is fused into the NEXT
  RMSNorm (``csrc/tp_kernels.cu``, ``tp_finish_norm_kernel``), so a tensor-parallel layer launches
  as many kernels as a single-GPU layer.  Two forms: two shot (default: reduce-scatter in the GEMM
  epilogue, all-gather inside the finishing kernel; bytes per rank do not grow with the rank
  count) and one shot (every rank receives every partial);
* the LM head is vocabulary-parallel; local (value, token) maxima are combined by a peer-store
  kernel, and so are the draft head's per-shard top-k lists and log-sum-exp (``csrc/tp_kernels.cu``);
* embeddings, norms and the residual stream are replicated; all ranks add the same numbers in
  the same order, so the replicated state stays bit-identical without further communication.

The reference has no tensor parallelism (its TP numbers come from an external serving stack),
so the measured baseline for these paths is this module's own unfused twin: ``torch.matmul`` +
NCCL ``all_reduce`` (:meth:`TensorParallel.gemm_allreduce_nccl`).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .symm import SymmetricBuffer


# --------------------------------------------------------------------------- sharding math (device-free)
def shard_rows(w, rank: int, world: int):
    """Column-parallel: split the OUTPUT features (rows of an ``nn.Linear`` weight, bf16 or NVFP4)."""
    n = w.shape[0]
    assert n % world == 0, f"{n} output features do not divide over {world} ranks"
    if not isinstance(w, torch.Tensor):
        return w.rows(rank * (n // world), (rank + 1) * (n // world))
    return w[rank * (n // world):(rank + 1) * (n // world)].contiguous()


def shard_cols(w, rank: int, world: int):
    """Row-parallel: split the INPUT features (columns of an ``nn.Linear`` weight, bf16 or NVFP4)."""
    k = w.shape[1]
    assert k % world == 0, f"{k} input features do not divide over {world} ranks"
    if not isinstance(w, torch.Tensor):
        return w.cols(rank * (k // world), (rank + 1) * (k // world))
    return w[:, rank * (k // world):(rank + 1) * (k // world)].contiguous()


def stack_rows(parts: list):
    """Row stack of weights that are all bf16 matrices or all NVFP4 matrices sharing one outer scale."""
    if not isinstance(parts[0], torch.Tensor):
        return type(parts[0]).cat_rows(list(parts))
    return torch.cat(tuple(parts), 0).contiguous()


def shard_attention(layer, cfg, rank: int, world: int) -> dict:
    """This rank's fused ``[q | k | v]`` rows (whole heads) and ``o_proj`` columns."""
    a = layer.self_attn
    assert cfg.num_attention_heads % world == 0 and cfg.num_key_value_heads % world == 0
    q, k, v = (shard_rows(t.weight, rank, world) for t in (a.q_proj, a.k_proj, a.v_proj))
    return {"qkv": stack_rows([q, k, v]), "o": shard_cols(a.o_proj.weight, rank, world),
            "qn": a.q_norm.weight, "kn": a.k_norm.weight}


def shard_mlp(mlp, rank: int, world: int, interleave) -> dict:
    g, u = shard_rows(mlp.gate_proj.weight, rank, world), shard_rows(mlp.up_proj.weight, rank, world)
    return {"gu": interleave(g, u), "gate": g, "up": u, "down": shard_cols(mlp.down_proj.weight, rank, world)}


# --------------------------------------------------------------------------- buffer-ring rule (device-free)
def ring_mod_for(calls_per_replay: int) -> int:
    """Cycle length of the receive-buffer ring for a CUDA graph that issues ``calls_per_replay`` collectives.

    Call ``c`` of a replay uses buffer ``c % ring_mod`` (baked into the graph).  Two collectives that follow
    each other must not share a buffer (a fast rank's next push would meet cells its slow peer is still
    reading), and that includes the last call of one replay and the first of the next:
    ``calls_per_replay % ring_mod`` must not be 1.  A distance of two is preferred where a cycle length offers it.
    For the few counts no cycle length of 2..6 satisfies (1, 61, 121, ...) the answer is 4 and the wrap-around is
    covered by what every round of this engine ends with: the vocabulary-parallel argmax exchange, in which every
    rank waits for every other rank, i.e. a full barrier between replays."""
    for bad in ((1, 2), (1,)):
        for r in (4, 5, 3, 6, 2):
            if calls_per_replay % r not in bad:
                return r
    return 4


class AllReduceRingModel:
    """Executable model of the cell protocol of the fused all-reduce (two-shot by default, ``two_shot=False`` for
    the one-shot form, whose finishing step consumes every rank's whole partial and has no gather step), for
    checking the buffer-reuse rule without a GPU.

    ``world`` ranks each run the same sequence of collectives; collective ``c`` uses ring buffer ``bufs[c]``.
    A rank's steps per collective mirror the kernels: *push* (the GEMM epilogue stores this rank's slice cells
    into every owner's first-phase buffer), *reduce* (the finishing kernel waits for all sources' cells of its
    own slice, consumes and zeroes them, and stores the result cell into every rank's gather buffer), *gather*
    (it waits for every owner's result cell, consumes and zeroes it).  ``run(schedule)`` interleaves the ranks
    in any order the schedule function picks and raises ``AssertionError`` as soon as a store lands on a cell
    whose previous content has not been consumed, or a rank consumes a value of another collective."""

    def __init__(self, world: int, bufs: list, two_shot: bool = True):
        self.world, self.bufs, self.two_shot = int(world), list(bufs), bool(two_shot)
        n_buf = max(self.bufs) + 1
        # rs[rank][buf][src] and ag[rank][buf][owner]: 0 = empty, else 1 + index of the collective that wrote it
        self.rs = [[[0] * world for _ in range(n_buf)] for _ in range(world)]
        self.ag = [[[0] * world for _ in range(n_buf)] for _ in range(world)]
        self.pc = [0] * world          # 3 * collective + step

    def _ready(self, r: int) -> bool:
        c, step = divmod(self.pc[r], 3)
        if c >= len(self.bufs):
            return False
        b = self.bufs[c]
        if step == 0:
            return True
        cells = self.rs[r][b] if step == 1 else self.ag[r][b]
        return all(v != 0 for v in cells)

    def _step(self, r: int) -> None:
        c, step = divmod(self.pc[r], 3)
        b, tag = self.bufs[c], c + 1
        if step == 0:
            for o in range(self.world):
                assert self.rs[o][b][r] == 0, f"collective {c}: rank {r} overwrote an unread first-phase cell of rank {o}"
                self.rs[o][b][r] = tag
        elif step == 1:
            assert all(v == tag for v in self.rs[r][b]), f"collective {c}: rank {r} reduced cells of another collective"
            self.rs[r][b] = [0] * self.world
            for q in range(self.world):
                if not self.two_shot:            # one shot: nothing to send, the "gather" step finds its cells set
                    self.ag[r][b] = [tag] * self.world
                    break
                assert self.ag[q][b][r] == 0, f"collective {c}: rank {r} overwrote an unread gather cell of rank {q}"
                self.ag[q][b][r] = tag
        else:
            assert all(v == tag for v in self.ag[r][b]), f"collective {c}: rank {r} gathered cells of another collective"
            self.ag[r][b] = [0] * self.world
        self.pc[r] += 1

    def run(self, pick) -> int:
        """Run to completion; ``pick(list of runnable ranks) -> rank``.  Returns the number of steps taken."""
        steps = 0
        while True:
            ready = [r for r in range(self.world) if self._ready(r)]
            if not ready:
                break
            self._step(pick(ready))
            steps += 1
        assert all(p == 3 * len(self.bufs) for p in self.pc), "the model deadlocked"
        return steps


# --------------------------------------------------------------------------- runtime
class TensorParallel:
    """Process-group handle plus the peer buffers of the fused collectives."""

    RING = 6   # buffers allocated; `ring_mod` of them are cycled through

    # A rank is never more than one collective ahead of its slowest peer, so a buffer is safe to
    # reuse once two other collectives have been issued in between.  Inside a CUDA graph the
    # buffer of each call is baked in and the sequence repeats every replay, so the cycle length
    # is chosen such that the wrap-around (last calls of one replay, first calls of the next)
    # keeps that distance too: `calls_per_replay % ring_mod` must not be 1 or 2.

    def __init__(self, group=None, m_cap: int = 512, n_max: int = 4096):
        import torch.distributed as dist
        from ..ops import cuda_ext as X
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.m_cap, self.n_max = int(m_cap), int(n_max)
        self.n_flags = 2 * X.SM_COUNT
        self._X = X
        self._turn = 0
        self.ring_mod = 4
        # all-reduce form (JETSPEC_TP_ALLREDUCE):
        #   ll   one shot, 8-byte cells {two bf16 outputs, flag word}: no fence, no counter, one NVLink crossing;
        #        every rank receives every rank's whole partial, so bytes per rank grow with the rank count
        #   ll2  two shot, same cells: the GEMM epilogue sends each rank only the column slice it owns
        #        (reduce-scatter), the finishing kernel reduces the slice and stores the result to all ranks
        #        (all-gather); bytes per rank stay flat
        #   flags  bf16 tiles + one release counter per CTA, a finishing kernel reduces
        #   wait   the GEMM CTA waits for its peers in its own epilogue (single kernel)
        # auto = ll2: measured faster than ll already at 2 ranks (Qwen3-8B round 4.60 against 4.66 ms: half the
        # bytes per phase outweigh the extra hop), and the only form whose traffic does not grow with the world.
        mode = os.environ.get("JETSPEC_TP_ALLREDUCE", "auto")
        if mode == "auto":
            mode = "ll2"
        self.mode = mode
        self.push_only = {"ll": 2, "ll2": 3, "flags": 1, "wait": 0}[mode]
        if os.environ.get("JETSPEC_TP_WAIT_IN_GEMM", "0") == "1":
            self.push_only = 0
        self.recv = [SymmetricBuffer(self.world * self.m_cap * self.n_max * 4, group) for _ in range(self.RING)]
        self.flags = [SymmetricBuffer(self.n_flags * 4, group) for _ in range(self.RING)]
        # second-phase (all-gather) cells of the two-shot form: (m_cap, n_max / 2) cells of 8 bytes per buffer
        self.gather = ([SymmetricBuffer(self.m_cap * self.n_max * 4, group) for _ in range(self.RING)]
                       if self.push_only == 3 else [])
        self.am_rows = max(256, min(4096, self.m_cap))
        self.am_buf = [SymmetricBuffer(self.world * self.am_rows * 8, group) for _ in range(2)]
        self.am_flag = [SymmetricBuffer(64, group) for _ in range(2)]
        self.tk_rows = 64
        self.tk_buf = [SymmetricBuffer(self.world * self.tk_rows * 18 * 8, group) for _ in range(2)]
        self._am_turn = 0
        self._tk_turn = 0
        self.launches = 0
        self.bytes_pushed = 0          # bytes this rank stored into peers' memory (diagnostic; counted on the host)

    @classmethod
    def from_env(cls, **kw) -> "TensorParallel":
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl")
        return cls(None, **kw)

    # ---- fused row-parallel GEMM + all-reduce --------------------------------------------------
    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                       residual: Optional[torch.Tensor] = None, split: Optional[int] = None, pdl: bool = False,
                       norm_w: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None,
                       eps: float = 1e-6):
        """``out = residual + all_reduce(x @ w.T)``; with ``norm_w`` also ``norm_out = rmsnorm(out) * norm_w``
        from the same finishing kernel.  ``x (M, K/world)``, ``w (N, K/world)``; every rank calls it with the
        same shapes.  The call order must be the same on all ranks (buffers are taken from a ring by call count)."""
        X = self._X
        lib = X.load()
        M, K = x.shape
        N = w.shape[0]
        assert N <= self.n_max and M <= self.m_cap
        n_tiles = (N + 127) // 128
        if self.push_only == 0:
            # Every CTA of a launch waits for its peers on the other GPUs, so a launch must fit the chip in ONE
            # wave: taller inputs go in row slabs, one launch (and one buffer of the ring) per slab.
            slab = max(1, (2 * X.SM_COUNT) // n_tiles) * 128
            if M > slab:
                for m0 in range(0, M, slab):
                    m1 = min(M, m0 + slab)
                    self.gemm_allreduce(x[m0:m1], w, out[m0:m1], None if residual is None else residual[m0:m1], split,
                                        pdl, norm_w, None if norm_out is None else norm_out[m0:m1], eps)
                return out
        if split is None:
            tiles = n_tiles * ((M + 127) // 128)
            kb = (K + 63) // 64
            split = 1
            while split < 4 and tiles * (split + 1) <= X.SM_COUNT and kb // (split + 1) >= 2:
                split += 1
        t = self._turn % self.ring_mod
        self._turn += 1
        push = self._push_mode(N)
        rc = lib.js_gemm_bf16_allreduce(X._p(x), X._p(w), X._p(out), X._p(residual), M, N, K, x.stride(0), w.stride(0),
                                        out.stride(0), split, X._p(self.recv[t].ptrs_dev), X._p(self.flags[t].ptrs_dev),
                                        self.rank, self.world, self.m_cap, self.n_flags,
                                        X._p(X.status_word(x.device)), int(pdl), push, X._stream())
        X._check(rc, f"js_gemm_bf16_allreduce(M={M},N={N},K={K},split={split},mode={push})")
        self.launches += 1
        if push:
            self._finish(t, out, residual, M, N, split, pdl, push, norm_w, norm_out, eps)
        elif norm_w is not None:
            X.rmsnorm(out, norm_w, eps, out=norm_out, pdl=pdl)
            self.launches += 1
        return out

    def _push_mode(self, N: int) -> int:
        """The epilogue mode of this call: the two-shot form needs the columns to split evenly over the ranks."""
        if self.push_only == 3 and N % (8 * self.world):
            return 2
        return int(self.push_only)

    def _finish(self, t: int, out, residual, M: int, N: int, split: int, pdl: bool, push: int,
                norm_w=None, norm_out=None, eps: float = 1e-6) -> None:
        """Second kernel of the push-mode all-reduce: wait for every rank's tiles, sum in rank order, add the
        residual (and, in the cell modes, apply the following RMSNorm in the same pass)."""
        X = self._X
        lib = X.load()
        if push >= 2:
            lib.js_tp_finish_norm.restype = ctypes.c_int
            two = push == 3
            rc = lib.js_tp_finish_norm(ctypes.c_void_p(self.recv[t].local),
                                       X._p(self.gather[t].ptrs_dev) if two else ctypes.c_void_p(0),
                                       X._p(residual), X._p(out), out.stride(0), X._p(norm_w), X._p(norm_out),
                                       norm_out.stride(0) if norm_out is not None else 0, ctypes.c_float(eps), M, N,
                                       self.m_cap, self.world, self.rank, int(two), X._p(X.status_word(out.device)),
                                       int(pdl), X._stream())
            X._check(rc, "js_tp_finish_norm")
            self.launches += 1
            # cells are 8 bytes per two bf16 values: one shot sends the whole partial to every peer, two shot one
            # slice per peer in each of the two phases
            per_peer = M * N * 4
            self.bytes_pushed += (self.world - 1) * (2 * per_peer // self.world if two else per_peer)
            return
        lib.js_tp_allreduce_finish.restype = ctypes.c_int
        rc = lib.js_tp_allreduce_finish(ctypes.c_void_p(self.recv[t].local), ctypes.c_void_p(self.flags[t].local),
                                        X._p(residual), X._p(out), M, N, out.stride(0), self.m_cap, self.world, split,
                                        X._p(X.status_word(out.device)), int(pdl), X._stream())
        X._check(rc, "js_tp_allreduce_finish")
        self.launches += 1
        self.bytes_pushed += (self.world - 1) * M * N * 2
        if norm_w is not None:
            X.rmsnorm(out, norm_w, eps, out=norm_out, pdl=pdl)
            self.launches += 1

    def gemm_allreduce_nvfp4(self, act: dict, qw, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                             split: Optional[int] = None, pdl: bool = False):
        """NVFP4 twin of :meth:`gemm_allreduce`: ``act`` is this rank's quantised K-slice of the activations
        (``cuda_ext.quant_nvfp4``), ``qw`` this rank's K-slice of the 4-bit weight."""
        X = self._X
        lib = X.load()
        M = act.get("rows", act["M"])
        N, K = qw.shape
        assert N <= self.n_max and M <= self.m_cap and act["K"] == K
        qw.swizzled()
        if not hasattr(qw, "_w_scale"):
            qw._w_scale = float(qw.outer)
        if split is None:
            tiles = ((N + 127) // 128) * ((M + 127) // 128)
            split = 1
            while split < 4 and tiles * (split + 1) <= X.SM_COUNT and (K // 256) // (split + 1) >= 1:
                split += 1
        t = self._turn % self.ring_mod
        self._turn += 1
        push = self._push_mode(N)
        lib.js_gemm_nvfp4_allreduce.restype = ctypes.c_int
        rc = lib.js_gemm_nvfp4_allreduce(X._p(act["packed"]), X._p(act["sf"]), X._p(act["outer"]), X._p(qw.packed),
                                         X._p(qw.scales_swizzled), ctypes.c_float(qw._w_scale), X._p(out),
                                         X._p(residual), M, N, K, act["packed"].stride(0), qw.packed.stride(0),
                                         out.stride(0), split, X._p(self.recv[t].ptrs_dev),
                                         X._p(self.flags[t].ptrs_dev), self.rank, self.world, self.m_cap,
                                         self.n_flags, X._p(X.status_word(out.device)), int(pdl),
                                         push, X._stream())
        X._check(rc, f"js_gemm_nvfp4_allreduce(M={M},N={N},K={K},split={split})")
        self.launches += 1
        if push:
            self._finish(t, out, residual, M, N, split, pdl, push)
        return out

    def begin_sequence(self, calls_per_replay: Optional[int] = None) -> None:
        """Start a fresh, repeatable sequence of collectives (call before capturing a graph and
        before replaying a different one).  All ranks must call it at the same point; it
        synchronises them so no rank is still reading a buffer of the previous sequence."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._turn = 0
        self._am_turn = 0
        self._tk_turn = 0
        if calls_per_replay is not None:
            self.ring_mod = ring_mod_for(calls_per_replay)

    def gemm_allreduce_nccl(self, x, w, out, residual=None):
        """Unfused baseline twin: library GEMM, NCCL all-reduce, residual add."""
        import torch.distributed as dist
        y = torch.matmul(x, w.t())
        dist.all_reduce(y, group=self.group)
        if residual is not None:
            y = y + residual
        out.copy_(y)
        return out

    # ---- vocabulary-parallel greedy token ----------------------------------------------------
    def lm_head_argmax(self, h: torch.Tensor, w_local: torch.Tensor, vocab_offset: int, ws: dict,
                       out_idx: torch.Tensor, out_val: Optional[torch.Tensor] = None, pdl: bool = False):
        X = self._X
        lib = X.load()
        M = h.shape[0]
        assert M <= self.am_rows
        nt = X.n_tiles(w_local.shape[0])
        X.gemm(h, w_local, out=None, epi=X.EPI_ARGMAX, bn=128, split=1, pdl=pdl, part_val=ws["val"], part_idx=ws["idx"])
        t = self._am_turn % 2
        self._am_turn += 1
        rc = lib.js_tp_argmax_combine(X._p(ws["val"]), X._p(ws["idx"]), nt, M, int(vocab_offset),
                                      X._p(self.am_buf[t].ptrs_dev), X._p(self.am_flag[t].ptrs_dev), self.rank,
                                      self.world, self.am_rows, X._p(out_idx), X._p(out_val), X._p(X.status_word(h.device)),
                                      int(pdl), X._stream())
        X._check(rc, "js_tp_argmax_combine")
        self.launches += 2
        return out_idx

    def lm_head_topk_logprobs(self, h: torch.Tensor, w_local: torch.Tensor, vocab_offset: int, k: int, ws: dict,
                              out_tok: torch.Tensor, out_lp: torch.Tensor, pdl: bool = False):
        """Vocabulary-parallel top-``k`` tokens with full-vocabulary log-probabilities (the draft head's logits):
        the top-k GEMM epilogue over this rank's shard, then one kernel that merges the local tiles, exchanges the
        per-row records through peer memory and merges them identically on every rank."""
        X = self._X
        lib = X.load()
        M = h.shape[0]
        assert M <= self.tk_rows and 1 <= k <= 8
        nt = X.n_tiles(w_local.shape[0])
        X.gemm(h, w_local, out=None, epi=X.EPI_TOPK, bn=128, split=1, pdl=pdl, part_val=ws["val"], part_idx=ws["idx"],
               part_lse=ws["lse"])
        t = self._tk_turn % 2
        self._tk_turn += 1
        lib.js_tp_topk_combine.restype = ctypes.c_int
        rc = lib.js_tp_topk_combine(X._p(ws["val"]), X._p(ws["idx"]), X._p(ws["lse"]), nt, M, int(k), int(vocab_offset),
                                    X._p(self.tk_buf[t].ptrs_dev), self.rank, self.world, self.tk_rows, X._p(out_tok),
                                    X._p(out_lp), X._p(X.status_word(h.device)), int(pdl), X._stream())
        X._check(rc, "js_tp_topk_combine")
        self.launches += 2
        return out_tok, out_lp

    def reset_buffers(self) -> None:
        """Zero this rank's receive cells and counters (all ranks together): only needed after a call reported a
        peer timeout, which can leave unconsumed cells behind."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for b in self.recv + self.flags + self.gather + self.am_buf + self.am_flag + self.tk_buf:
            b.zero_local()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def close(self):
        for b in self.recv + self.flags + self.gather + self.am_buf + self.am_flag + self.tk_buf:
            b.close()
