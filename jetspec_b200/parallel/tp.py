"""Tensor parallelism for the verify forward.

Sharding plan (``world`` ranks, one process per GPU):

* QKV and gate/up projections are column-parallel (each rank owns ``Hq/world`` query heads,
  ``Hkv/world`` KV heads and ``I/world`` MLP channels, so attention and the KV pool are local);
* ``o_proj`` and ``down_proj`` are row-parallel: every rank multiplies its K-slice and the
  partial products are summed by a one-shot all-reduce that is FUSED into the GEMM epilogue —
  finished tiles are stored into all peers' buffers over NVLink from inside the kernel
  (``csrc/gemm_sm100.cu``, ``EPI_ALLREDUCE``);
* the LM head is vocabulary-parallel; local (value, token) maxima are combined by a peer-store
  kernel (``csrc/tp_kernels.cu``);
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
        # push mode (default): the GEMM only pushes its partial tiles and a finishing kernel reduces, so no GEMM CTA
        # ever waits for a peer; JETSPEC_TP_WAIT_IN_GEMM=1 selects the single-kernel variant that waits in its epilogue
        #   2 = low-latency cells (8 bytes = two bf16 outputs + a flag word, polled by the finishing kernel: no fence,
        #       no counter, one NVLink crossing), 1 = bf16 tiles + one release counter per CTA, 0 = wait inside the GEMM
        mode = os.environ.get("JETSPEC_TP_ALLREDUCE", "ll")
        self.push_only = {"ll": 2, "flags": 1, "wait": 0}[mode]
        if os.environ.get("JETSPEC_TP_WAIT_IN_GEMM", "0") == "1":
            self.push_only = 0
        self.recv = [SymmetricBuffer(self.world * self.m_cap * self.n_max * 4, group) for _ in range(self.RING)]
        self.flags = [SymmetricBuffer(self.n_flags * 4, group) for _ in range(self.RING)]
        self.am_buf = [SymmetricBuffer(self.world * 256 * 8, group) for _ in range(2)]
        self.am_flag = [SymmetricBuffer(64, group) for _ in range(2)]
        self._am_turn = 0
        self.launches = 0

    @classmethod
    def from_env(cls, **kw) -> "TensorParallel":
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl")
        return cls(None, **kw)

    # ---- fused row-parallel GEMM + all-reduce --------------------------------------------------
    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                       residual: Optional[torch.Tensor] = None, split: Optional[int] = None, pdl: bool = False):
        """``out = residual + all_reduce(x @ w.T)`` in ONE kernel per rank.  ``x (M, K/world)``,
        ``w (N, K/world)``; every rank calls it with the same shapes.  The call order must be the
        same on all ranks (buffers are taken from a ring by call count)."""
        X = self._X
        lib = X.load()
        M, K = x.shape
        N = w.shape[0]
        assert N <= self.n_max and M <= self.m_cap
        # Every CTA of a launch waits for its peers on the other GPUs, so a launch must fit the chip in ONE wave:
        # taller inputs go in row slabs, one launch (and one buffer of the ring) per slab.
        n_tiles = (N + 127) // 128
        slab = max(1, (2 * X.SM_COUNT) // n_tiles) * 128
        if M > slab:
            for m0 in range(0, M, slab):
                m1 = min(M, m0 + slab)
                self.gemm_allreduce(x[m0:m1], w, out[m0:m1], None if residual is None else residual[m0:m1], split, pdl)
            return out
        if split is None:
            tiles = ((N + 127) // 128) * ((M + 127) // 128)
            kb = (K + 63) // 64
            split = 1
            while split < 4 and tiles * (split + 1) <= X.SM_COUNT and kb // (split + 1) >= 2:
                split += 1
        t = self._turn % self.ring_mod
        self._turn += 1
        rc = lib.js_gemm_bf16_allreduce(X._p(x), X._p(w), X._p(out), X._p(residual), M, N, K, x.stride(0), w.stride(0),
                                        out.stride(0), split, X._p(self.recv[t].ptrs_dev), X._p(self.flags[t].ptrs_dev),
                                        self.rank, self.world, self.m_cap, self.n_flags,
                                        X._p(X.status_word(x.device)), int(pdl), int(self.push_only), X._stream())
        X._check(rc, f"js_gemm_bf16_allreduce(M={M},N={N},K={K},split={split})")
        self.launches += 1
        if self.push_only:
            self._finish(t, out, residual, M, N, split, pdl)
        return out

    def _finish(self, t: int, out, residual, M: int, N: int, split: int, pdl: bool) -> None:
        """Second kernel of the push-mode all-reduce: wait for every rank's tiles, sum in rank order, add the residual."""
        X = self._X
        lib = X.load()
        if self.push_only == 2:
            lib.js_tp_allreduce_finish_ll.restype = ctypes.c_int
            rc = lib.js_tp_allreduce_finish_ll(ctypes.c_void_p(self.recv[t].local), X._p(residual), X._p(out), M, N,
                                               out.stride(0), self.m_cap, self.world, X._p(X.status_word(out.device)),
                                               int(pdl), X._stream())
            X._check(rc, "js_tp_allreduce_finish_ll")
            self.launches += 1
            return
        lib.js_tp_allreduce_finish.restype = ctypes.c_int
        rc = lib.js_tp_allreduce_finish(ctypes.c_void_p(self.recv[t].local), ctypes.c_void_p(self.flags[t].local),
                                        X._p(residual), X._p(out), M, N, out.stride(0), self.m_cap, self.world, split,
                                        X._p(X.status_word(out.device)), int(pdl), X._stream())
        X._check(rc, "js_tp_allreduce_finish")
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
        lib.js_gemm_nvfp4_allreduce.restype = ctypes.c_int
        rc = lib.js_gemm_nvfp4_allreduce(X._p(act["packed"]), X._p(act["sf"]), X._p(act["outer"]), X._p(qw.packed),
                                         X._p(qw.scales_swizzled), ctypes.c_float(qw._w_scale), X._p(out),
                                         X._p(residual), M, N, K, act["packed"].stride(0), qw.packed.stride(0),
                                         out.stride(0), split, X._p(self.recv[t].ptrs_dev),
                                         X._p(self.flags[t].ptrs_dev), self.rank, self.world, self.m_cap,
                                         self.n_flags, X._p(X.status_word(out.device)), int(pdl),
                                         int(self.push_only), X._stream())
        X._check(rc, f"js_gemm_nvfp4_allreduce(M={M},N={N},K={K},split={split})")
        self.launches += 1
        if self.push_only:
            self._finish(t, out, residual, M, N, split, pdl)
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
        if calls_per_replay is not None:
            self.ring_mod = next(r for r in (4, 5, 3, 6) if calls_per_replay % r not in (1, 2))

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
        assert M <= 256
        nt = X.n_tiles(w_local.shape[0])
        X.gemm(h, w_local, out=None, epi=X.EPI_ARGMAX, bn=128, split=1, pdl=pdl, part_val=ws["val"], part_idx=ws["idx"])
        t = self._am_turn % 2
        self._am_turn += 1
        rc = lib.js_tp_argmax_combine(X._p(ws["val"]), X._p(ws["idx"]), nt, M, int(vocab_offset),
                                      X._p(self.am_buf[t].ptrs_dev), X._p(self.am_flag[t].ptrs_dev), self.rank,
                                      self.world, 256, X._p(out_idx), X._p(out_val), X._p(X.status_word(h.device)),
                                      int(pdl), X._stream())
        X._check(rc, "js_tp_argmax_combine")
        self.launches += 2
        return out_idx

    def close(self):
        for b in self.recv + self.flags + self.am_buf + self.am_flag:
            b.close()
