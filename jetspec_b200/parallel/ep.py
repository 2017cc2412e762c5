"""Expert parallelism for Qwen3-MoE layers.

Two plans live here.

:class:`TokenShardedEP` (the engine's plan): every rank owns its own tokens (its requests) and
``E / world`` experts.  A layer routes the local tokens, exchanges the per-expert counts, stores
every (token, choice) row straight into the owning expert rank's receive slab with peer stores
(``csrc/ep_kernels.cu``), runs the experts there as two grouped tcgen05 GEMMs, and the second
GEMM's epilogue returns each weighted output row to the token's owner only; the owner's finishing
kernel sums a token's ``top_k`` rows in choice order, adds the residual and applies the next
RMSNorm.  Bytes over NVLink per layer and rank: the all-to-all minimum (each row crosses once in
each direction) times two on the way back for the flag words.

:class:`ExpertParallel` (replicated residual): the residual stream is replicated on every rank (as
in the tensor-parallel plan), so *dispatch* needs no communication: each rank routes all tokens
(the router is tiny and replicated) and gathers the (token, choice) pairs whose expert it owns.  One grouped tcgen05 GEMM runs the
experts' gate/up projections with the SwiGLU epilogue; a second grouped GEMM runs the down
projections and its epilogue IS the *combine*: every output row is scaled by its routing weight
and stored straight into all ranks' pair buffers over NVLink, one counter per rank is bumped per
CTA, and a finishing kernel on each rank waits for the global count and sums the ``top_k`` rows of
every token in choice order (bit-identical replicas, no atomics).

Reference behaviour of the layer itself: ``jetspec/models/moe_fused.py:16-51`` (softmax top-k
routing, sort by expert, two grouped GEMMs, weighted un-sort).  The reference has no expert
parallelism; the measured baseline is :meth:`ExpertParallel.moe_layer_nccl` (library grouped math
+ NCCL all-reduce).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import reference as ref
from .symm import SymmetricBuffer


def interleave_experts(w_gate_up: torch.Tensor, bn: int = 128) -> torch.Tensor:
    """``(E, 2I, H)`` stacked ``[gate | up]`` → ``(E*2I, H)`` with every ``bn``-row tile holding
    ``bn/2`` gate rows then the ``bn/2`` up rows of the same outputs (the SwiGLU epilogue's layout)."""
    E, I2, H = w_gate_up.shape
    I, h = I2 // 2, bn // 2
    g = w_gate_up[:, :I].reshape(E, I // h, h, H)
    u = w_gate_up[:, I:].reshape(E, I // h, h, H)
    return torch.cat((g, u), dim=2).reshape(E * I2, H).contiguous()


def route_and_sort(router_logits: torch.Tensor, top_k: int, renorm: bool, first_expert: int, n_local: int):
    """Routing plus the static-shape permutation used by the grouped GEMMs.

    Returns ``(order, row_weight, group_off, counts_all)``: ``order (T*k,)`` lists pair indices
    ``t*k+j`` sorted by local expert (pairs of other ranks' experts last), ``row_weight`` their routing
    weights, ``group_off (n_local+1,)`` the row ranges of the local experts, ``counts_all (E,)`` the
    global per-expert pair counts (identical on every rank).
    """
    E = router_logits.shape[-1]
    if router_logits.is_cuda and E <= 256 and router_logits.shape[0] * top_k <= 16384:
        # router + permutation kernels (no host synchronisation, static shapes)
        from ..ops import cuda_ext as X
        order, row_w, group_off, counts_all = X.moe_route_sort(router_logits, top_k, renorm, first_expert, n_local)
        return order.long(), row_w, group_off, counts_all.long()
    wts, idx = ref.moe_route(router_logits, top_k, renorm)
    flat_e = idx.reshape(-1)
    local = flat_e - first_expert
    key = torch.where((local >= 0) & (local < n_local), local, torch.full_like(local, n_local))
    order = torch.argsort(key, stable=True)
    counts_local = torch.bincount(key, minlength=n_local + 1)[:n_local]
    group_off = torch.zeros(n_local + 1, dtype=torch.int32, device=router_logits.device)
    group_off[1:] = torch.cumsum(counts_local, 0).to(torch.int32)
    counts_all = torch.bincount(flat_e, minlength=E)
    return order, wts.reshape(-1)[order].float().contiguous(), group_off, counts_all


class ExpertParallel:
    RING = 3

    def __init__(self, group, num_experts: int, top_k: int, hidden: int, max_tokens: int):
        import torch.distributed as dist
        from ..ops import cuda_ext as X
        self._X = X
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert num_experts % self.world == 0
        self.E, self.k, self.H, self.max_tokens = num_experts, top_k, hidden, max_tokens
        self.n_local = num_experts // self.world
        self.first = self.rank * self.n_local
        self.pairs = [SymmetricBuffer(max_tokens * top_k * hidden * 2, group) for _ in range(self.RING)]
        self.cnt = [SymmetricBuffer(64, group) for _ in range(self.RING)]
        self.done = torch.zeros(self.RING, dtype=torch.int32, device="cuda")
        self._turn = 0
        self.launches = 0

    def shard(self, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        """This rank's experts as the two stacked kernel operands."""
        gu = interleave_experts(w_gate_up[self.first:self.first + self.n_local])
        dn = w_down[self.first:self.first + self.n_local]
        return gu, dn.reshape(self.n_local * dn.shape[1], dn.shape[2]).contiguous()

    def moe_layer(self, x: torch.Tensor, gate_w: torch.Tensor, gu_local: torch.Tensor, down_local: torch.Tensor,
                  renorm: bool, out: Optional[torch.Tensor] = None, router_logits: Optional[torch.Tensor] = None,
                  pdl: bool = False) -> torch.Tensor:
        """``out = x + MoE(x)`` with expert-parallel experts; ``x (T, H)`` replicated on every rank."""
        X = self._X
        lib = X.load()
        T, H = x.shape
        I = gu_local.shape[0] // (2 * self.n_local)
        assert T <= self.max_tokens and H == self.H
        if router_logits is None:
            router_logits = X.gemm(x, gate_w, epi=X.EPI_STORE_F32)
        order, row_w, group_off, counts_all = route_and_sort(router_logits, self.k, renorm, self.first, self.n_local)
        tok = torch.div(order, self.k, rounding_mode="floor")
        xs = x.index_select(0, tok)                                   # (T*k, H); rows past the local groups are unused
        h = torch.empty(T * self.k, I, dtype=x.dtype, device=x.device)
        st = X._p(X.status_word(x.device))
        X._check(lib.js_gemm_bf16_grouped(X._p(xs), X._p(gu_local), X._p(h), T * self.k, 2 * I, H, xs.stride(0),
                                          gu_local.stride(0), h.stride(0), X.EPI_SWIGLU, self.n_local, X._p(group_off),
                                          T, None, None, None, None, 1, st, int(pdl), X._stream()), "grouped gate/up")
        t = self._turn % self.RING
        self._turn += 1
        row_pair = order.to(torch.int32).contiguous()
        X._check(lib.js_gemm_bf16_grouped(X._p(h), X._p(down_local), None, T * self.k, H, I, h.stride(0),
                                          down_local.stride(0), H, 6, self.n_local, X._p(group_off), T, X._p(row_pair),
                                          X._p(row_w), X._p(self.pairs[t].ptrs_dev), X._p(self.cnt[t].ptrs_dev),
                                          self.world, st, int(pdl), X._stream()), "grouped down + combine")
        # every rank knows all experts' loads, hence how many CTAs of all ranks will report in
        expected = (torch.div(counts_all + 127, 128, rounding_mode="floor").sum() * (H // 128)).to(torch.int32).reshape(1)
        if out is None:
            out = torch.empty_like(x)
        import ctypes
        X._check(lib.js_ep_combine_finish(ctypes.c_void_p(self.pairs[t].local), ctypes.c_void_p(self.cnt[t].local),
                                          X._p(expected), X._p(self.done[t:t + 1]), X._p(x), X._p(out), T, self.k, H, st,
                                          int(pdl), X._stream()), "ep combine finish")
        self.launches += 3
        return out

    def moe_layer_grouped_nccl(self, x, gate_w, gu_local, down_local, renorm, router_logits=None):
        """Unfused twin on the SAME grouped GEMMs: local experts' outputs are stored, scattered into a dense fp32
        partial with their routing weights, summed over the ranks by an NCCL all-reduce, then the residual is added."""
        import torch.distributed as dist
        X = self._X
        lib = X.load()
        T, H = x.shape
        I = gu_local.shape[0] // (2 * self.n_local)
        if router_logits is None:
            router_logits = X.gemm(x, gate_w, epi=X.EPI_STORE_F32)
        order, row_w, group_off, _ = route_and_sort(router_logits, self.k, renorm, self.first, self.n_local)
        tok = torch.div(order, self.k, rounding_mode="floor")
        xs = x.index_select(0, tok)
        h = torch.empty(T * self.k, I, dtype=x.dtype, device=x.device)
        y = torch.zeros(T * self.k, H, dtype=x.dtype, device=x.device)
        st = X._p(X.status_word(x.device))
        X._check(lib.js_gemm_bf16_grouped(X._p(xs), X._p(gu_local), X._p(h), T * self.k, 2 * I, H, xs.stride(0),
                                          gu_local.stride(0), h.stride(0), X.EPI_SWIGLU, self.n_local, X._p(group_off),
                                          T, None, None, None, None, 1, st, 0, X._stream()), "grouped gate/up")
        X._check(lib.js_gemm_bf16_grouped(X._p(h), X._p(down_local), X._p(y), T * self.k, H, I, h.stride(0),
                                          down_local.stride(0), y.stride(0), X.EPI_STORE, self.n_local, X._p(group_off),
                                          T, None, None, None, None, 1, st, 0, X._stream()), "grouped down")
        n_mine = group_off[-1:].long()                       # rows past the local groups belong to other ranks
        valid = (torch.arange(T * self.k, device=x.device) < n_mine).float()[:, None]
        part = torch.zeros(T, H, dtype=torch.float32, device=x.device)
        part.index_add_(0, tok, y.float() * (row_w * valid[:, 0])[:, None])
        dist.all_reduce(part, group=self.group)
        return (x.float() + part).to(x.dtype)

    def moe_layer_nccl(self, x, gate_w, w_gate_up, w_down, renorm, router_logits=None):
        """Unfused baseline twin: this rank's experts through plain PyTorch, NCCL all-reduce, residual."""
        import torch.distributed as dist
        if router_logits is None:
            router_logits = torch.nn.functional.linear(x, gate_w)
        wts, idx = ref.moe_route(router_logits, self.k, renorm)
        part = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        flat_e, flat_w = idx.reshape(-1), wts.reshape(-1)
        flat_t = torch.arange(x.shape[0], device=x.device).repeat_interleave(self.k)
        for e in range(self.first, self.first + self.n_local):
            sel = (flat_e == e).nonzero(as_tuple=True)[0]
            if sel.numel():
                hh = ref.silu_mul(torch.nn.functional.linear(x[flat_t[sel]], w_gate_up[e]))
                part.index_add_(0, flat_t[sel], torch.nn.functional.linear(hh, w_down[e]).float() * flat_w[sel, None])
        dist.all_reduce(part, group=self.group)
        return (x.float() + part).to(x.dtype)

    def close(self):
        for b in self.pairs + self.cnt:
            b.close()


def slab_layout(counts, n_local: int):
    """Where the dispatch kernel puts rows (device-free statement of ``ep_dispatch_kernel``'s placement).

    ``counts[src][e]`` = number of (token, choice) pairs of source rank ``src`` routed to expert ``e``.  On the
    rank that owns expert ``e`` (``e // n_local``) the receive slab is ordered by expert, and inside an expert by
    source rank.  Returns ``(base, group_off)``: ``base[src][e]`` is the first slab row (on the owner of ``e``) of
    ``src``'s rows of expert ``e``; ``group_off[owner]`` the ``n_local + 1`` row offsets of that owner's experts,
    i.e. the row ranges its grouped GEMMs run over."""
    world, E = len(counts), len(counts[0])
    base = [[0] * E for _ in range(world)]
    group_off = [[0] * (n_local + 1) for _ in range(E // n_local)]
    for owner in range(E // n_local):
        run = 0
        for le in range(n_local):
            e = owner * n_local + le
            group_off[owner][le] = run
            for src in range(world):
                base[src][e] = run
                run += counts[src][e]
        group_off[owner][n_local] = run
    return base, group_off


class TokenShardedEP:
    """Expert parallelism over token-sharded ranks: peer-store dispatch, grouped expert GEMMs, combine in the
    down-projection epilogue (see the module docstring).  One instance serves every MoE layer of a model: the
    buffers re-arm themselves, and calls take the count / arrival buffers from a short ring by call count, so
    every rank must make the same sequence of calls (``idle_layer`` for a rank that has no tokens in a step)."""

    RING = 6

    def __init__(self, group, num_experts: int, top_k: int, hidden: int, max_tokens: int,
                 rows_factor: float = 2.0):
        import torch.distributed as dist
        from ..ops import cuda_ext as X
        from .tp import ring_mod_for
        self._X, self._ring_mod_for = X, ring_mod_for
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert num_experts % self.world == 0 and top_k <= 8 and hidden % 128 == 0
        self.E, self.k, self.H, self.max_tokens = int(num_experts), int(top_k), int(hidden), int(max_tokens)
        self.n_local = self.E // self.world
        self.first = self.rank * self.n_local
        # receive slab: worst case every pair of every rank lands here.  The grouped GEMMs are LAUNCHED for
        # `max_rows_per_expert` rows per expert (a few times the balanced load); an expert that receives more is
        # still finished: its CTAs walk on through its remaining row tiles, so skewed routing (identical tokens,
        # pad rows) costs time, never correctness
        self.slab_rows = self.world * self.max_tokens * self.k
        avg = self.slab_rows / self.E
        self.max_rows_per_expert = int(min(self.slab_rows, ((int(rows_factor * avg) + 127) // 128) * 128 or 128))
        dev = "cuda"
        self.slab = SymmetricBuffer(self.slab_rows * self.H * 2, group)
        self.meta = SymmetricBuffer(self.slab_rows * 8, group)
        self.roww = SymmetricBuffer(self.slab_rows * 4, group)
        self.cnt = [SymmetricBuffer(self.world * self.E * 8, group) for _ in range(self.RING)]
        self.arrive = [SymmetricBuffer(64, group) for _ in range(self.RING)]
        self.pairs = [SymmetricBuffer(self.max_tokens * self.k * self.H * 4, group) for _ in range(2)]
        i32 = dict(dtype=torch.int32, device=dev)
        self.hist, self.fill, self.done = torch.zeros(self.E, **i32), torch.zeros(self.E, **i32), torch.zeros(2, **i32)
        self.group_off = torch.zeros(self.n_local + 1, **i32)
        self.wts = torch.zeros(max(1, self.max_tokens), self.k, dtype=torch.float32, device=dev)
        self.idx = torch.zeros(max(1, self.max_tokens), self.k, **i32)
        self.logits = torch.zeros(max(1, self.max_tokens), self.E, dtype=torch.float32, device=dev)
        self.slab_t = self.slab.tensor(self.rank, (self.slab_rows, self.H), torch.bfloat16)
        self._act: dict = {}
        self._turn, self._pair_turn, self.ring_mod = 0, 0, 4
        self.launches = 0
        self.bytes_pushed = 0

    def shard(self, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        """This rank's experts as the two stacked kernel operands."""
        gu = interleave_experts(w_gate_up[self.first:self.first + self.n_local])
        dn = w_down[self.first:self.first + self.n_local]
        return gu, dn.reshape(self.n_local * dn.shape[1], dn.shape[2]).contiguous()

    def begin_sequence(self, calls_per_replay: Optional[int] = None) -> None:
        """Start a fresh, repeatable sequence of layer calls (before capturing a graph and before replaying a
        different one); all ranks call it at the same point."""
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._turn = self._pair_turn = 0
        if calls_per_replay is not None:
            self.ring_mod = self._ring_mod_for(calls_per_replay)

    def _exchange(self, h_norm: Optional[torch.Tensor], gate_w, renorm: bool, pdl: bool):
        """Route + count exchange + dispatch of this rank's tokens (none when ``h_norm`` is None)."""
        import ctypes
        X = self._X
        lib = X.load()
        T = 0 if h_norm is None else h_norm.shape[0]
        assert T <= self.max_tokens
        st = X._p(X.status_word("cuda"))
        t = self._turn % self.ring_mod
        self._turn += 1
        if T:
            X.gemm(h_norm, gate_w, out=self.logits[:T], epi=X.EPI_STORE_F32, pdl=pdl)
            self.launches += 1
        lib.js_ep_route_count.restype = ctypes.c_int
        X._check(lib.js_ep_route_count(X._p(self.logits), T, self.E, self.k, int(bool(renorm)), X._p(self.wts),
                                       X._p(self.idx), X._p(self.hist), X._p(self.done[0:1]),
                                       X._p(self.cnt[t].ptrs_dev), self.rank, self.world, int(pdl), X._stream()),
                 "js_ep_route_count")
        lib.js_ep_dispatch.restype = ctypes.c_int
        X._check(lib.js_ep_dispatch(X._p(h_norm), h_norm.stride(0) if T else self.H, X._p(self.wts), X._p(self.idx), T,
                                    self.H, self.k, self.E, self.n_local, self.rank, self.world, self.slab_rows,
                                    self.max_rows_per_expert, ctypes.c_void_p(self.cnt[t].local),
                                    X._p(self.slab.ptrs_dev), X._p(self.meta.ptrs_dev), X._p(self.roww.ptrs_dev),
                                    X._p(self.arrive[t].ptrs_dev), X._p(self.fill), X._p(self.done[1:2]),
                                    X._p(self.group_off), st, int(pdl), X._stream()), "js_ep_dispatch")
        self.launches += 2
        self.bytes_pushed += T * self.k * self.H * 2 * (self.world - 1) // self.world      # expected, balanced routing

    def _experts(self, gu_local: torch.Tensor, down_local: torch.Tensor, pairs_ptrs, pdl: bool) -> None:
        """This rank's experts over its receive slab; the down projection's epilogue sends the rows home."""
        import ctypes
        X = self._X
        lib = X.load()
        I = gu_local.shape[0] // (2 * self.n_local)
        if I not in self._act:
            self._act[I] = torch.zeros(self.slab_rows, I, dtype=torch.bfloat16, device="cuda")
        h = self._act[I]
        st = X._p(X.status_word("cuda"))
        # no programmatic early start for the first grouped GEMM: its CTAs read the row ranges (group_off) on
        # entry, and the dispatch kernel that writes them must have finished by then
        X._check(lib.js_gemm_bf16_grouped(X._p(self.slab_t), X._p(gu_local), X._p(h), self.slab_rows, 2 * I, self.H,
                                          self.H, gu_local.stride(0), h.stride(0), X.EPI_SWIGLU, self.n_local,
                                          X._p(self.group_off), self.max_rows_per_expert, None, None, None, None, 1,
                                          st, 0, X._stream()), "grouped gate/up")
        lib.js_gemm_bf16_grouped_ep.restype = ctypes.c_int
        X._check(lib.js_gemm_bf16_grouped_ep(X._p(h), X._p(down_local), self.slab_rows, self.H, I, h.stride(0),
                                             down_local.stride(0), self.n_local, X._p(self.group_off),
                                             self.max_rows_per_expert, ctypes.c_void_p(self.meta.local),
                                             ctypes.c_void_p(self.roww.local), pairs_ptrs, self.world, st, int(pdl),
                                             X._stream()), "grouped down + combine")
        self.launches += 2

    def moe_layer(self, x: torch.Tensor, h_norm: torch.Tensor, gate_w: torch.Tensor, gu_local: torch.Tensor,
                  down_local: torch.Tensor, renorm: bool, out: Optional[torch.Tensor] = None,
                  norm_w: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None, eps: float = 1e-6,
                  pdl: bool = False) -> torch.Tensor:
        """``out = x + MoE(h_norm)`` for this rank's ``T`` tokens (``x`` the residual rows, ``h_norm`` their
        normalised form); with ``norm_w`` also ``norm_out = rmsnorm(out) * norm_w`` from the same finishing kernel."""
        import ctypes
        X = self._X
        lib = X.load()
        T, H = h_norm.shape
        assert H == self.H
        pt = self._pair_turn % 2
        self._pair_turn += 1
        self._exchange(h_norm, gate_w, renorm, pdl)
        self._experts(gu_local, down_local, X._p(self.pairs[pt].ptrs_dev), pdl)
        if out is None:
            out = torch.empty_like(x)
        lib.js_ep_combine_finish_norm.restype = ctypes.c_int
        X._check(lib.js_ep_combine_finish_norm(ctypes.c_void_p(self.pairs[pt].local), X._p(x), X._p(out), out.stride(0),
                                               X._p(norm_w), X._p(norm_out),
                                               norm_out.stride(0) if norm_out is not None else 0, ctypes.c_float(eps),
                                               T, H, self.k, X._p(X.status_word("cuda")), int(pdl), X._stream()),
                 "js_ep_combine_finish_norm")
        self.launches += 1
        return out

    def idle_layer(self, gate_w, gu_local: torch.Tensor, down_local: torch.Tensor, renorm: bool = True,
                   pdl: bool = False) -> None:
        """Take part in a layer without tokens of one's own: publish zero counts, receive and run the other
        ranks' rows, send their results home."""
        X = self._X
        pt = self._pair_turn % 2
        self._pair_turn += 1
        self._exchange(None, gate_w, renorm, pdl)
        self._experts(gu_local, down_local, X._p(self.pairs[pt].ptrs_dev), pdl)

    def close(self):
        for b in [self.slab, self.meta, self.roww] + self.cnt + self.arrive + self.pairs:
            b.close()
