"""``JetSpecEngine``: paged-KV decode engine (AR, tree-speculative, continuous batching).

Public surface follows ``jetspec/inference_engine/engine.py:257-1521``:
``generate``, ``generate_tree``, ``generate_batch``, ``generate_tree_batch`` with the
same keyword arguments and return dictionaries.

Design (differs from the reference on purpose):

* one attention path — slot-addressed paged tree attention — instead of a ladder of
  six backends; the reference's backend names are accepted and all map onto it;
* KV commit is a permutation of the tree window's slot-map entries
  (:meth:`PagedKVPool.commit_path`), never a KV copy, and rejected slots are reused
  by the next round (the reference's no-gather path leaks them until reset,
  ``engine.py:815-822``);
* batched paths read the pool directly through ragged metadata (the reference
  rebuilds dense padded caches every step, ``engine.py:1309-1321``) and are driven
  by the scheduler, including finish-time admission and eviction/restore;
* on a CUDA device with bf16 weights the round (draft-head step, tree build,
  verify, accept, commit) runs as hand-written sm_100a kernels replayed from one
  CUDA graph per tree bucket (:mod:`jetspec_b200.engine.fast_round`); everywhere
  else the same steps run eagerly on the PyTorch reference ops.
"""
from __future__ import annotations

import math
import time
from typing import Optional, Sequence

import torch

from .. import ops
from ..core.llm import decode_text, resolve_eos
from ..models.qwen3 import Qwen3ForCausalLM, load_target
from ..runtime import PagedKVPool, Scheduler, SequenceRequest, build_attn_metadata
from ..sampling import SamplingParams, sample
from ..tree import (build_from_topk, get_algorithm, gpu_tree_accept, should_extend, splice_extension,
                    tree_accept)
from ..tree.accept import host_tree_accept
from ..utils.env import env_flag

TREE_BUCKETS = (16, 32, 64, 128, 192, 256)

_BACKEND_ALIASES = {
    "sm100", "sdpa", "triton_paged_tree", "triton_paged_tree_compiled", "triton_paged_tree_cudagraph",
    "triton_paged_tree_compiled_nogather", "triton_paged_tree_cudagraph_nogather",
}


def bucket_for_n(n: int) -> int:
    """Smallest tree bucket ``>= n``; beyond the largest, the next multiple of it."""
    for b in TREE_BUCKETS:
        if n <= b:
            return b
    step = TREE_BUCKETS[-1]
    return ((n + step - 1) // step) * step


class _OneNode:
    """A one-node tree (the last committed token) for autoregressive steps through the batched verify graph."""
    __slots__ = ("host", "num_nodes")

    def __init__(self, token: int):
        self.host = ([int(token)], [-1], [0])
        self.num_nodes = 1


def _round_session_capacity(prompt_len: int) -> int:
    return ((int(prompt_len) + 255) // 256) * 256


def maybe_extend_tree(tree, topk_tok, topk_lp, tree_drafter, committed, target_hidden, tree_width, extend_kwargs):
    """Gated extension below the rank-1 chain's leaf (one conditioned drafter pass).

    Fires only when the rank-1 chain is fully present in the tree and its mean top-2 gap
    clears ``gap_threshold``; otherwise the tree is returned unchanged
    (reference: ``_maybe_extend_tree``, ``jetspec/inference_engine/engine.py:109-146``).
    """
    cond_fn = getattr(tree_drafter, "propose_logits_conditioned", None)
    if cond_fn is None:
        return tree
    chain = [int(t) for t in topk_tok[:, 0].tolist()]
    parents, tokens = tree.parent_indices.tolist(), tree.token_ids.tolist()
    kids = [[] for _ in range(tree.num_nodes)]
    for i in range(1, tree.num_nodes):
        kids[parents[i]].append(i)
    node = 0
    for tok in chain:
        node = next((c for c in kids[node] if tokens[c] == tok), None)
        if node is None:
            return tree
    if not should_extend(topk_lp, [0] * len(chain), gap_threshold=float(extend_kwargs.get("gap_threshold", 1.0))):
        return tree
    cond = cond_fn(committed, topk_tok[:, 0], target_hidden=target_hidden)
    return splice_extension(tree, node, cond, ext_budget=int(extend_kwargs.get("ext_budget", len(chain))),
                            tree_width=tree_width, mode=extend_kwargs.get("mode", "chain"))


class JetSpecEngine:
    def __init__(self, model_name_or_path, device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                 block_size: int = 16, attn_implementation: str = "sdpa", attn_backend: str = "sm100",
                 fuse_gemms: bool = False, torch_compile: bool = False, fused_moe: bool = False, *,
                 tokenizer=None, num_pages: Optional[int] = None, max_seqs: int = 64,
                 max_seq_len: int = 8192, use_kernels: Optional[bool] = None, tensor_parallel=None,
                 expert_parallel=None):
        if attn_backend not in _BACKEND_ALIASES:
            raise ValueError(f"unknown attn_backend {attn_backend!r}; expected one of {sorted(_BACKEND_ALIASES)}")
        if isinstance(model_name_or_path, Qwen3ForCausalLM):
            self.model = model_name_or_path.to(device=device, dtype=dtype)
            self.tokenizer = tokenizer
        else:
            self.model, self.tokenizer = load_target(model_name_or_path, device=device, dtype=dtype)
            if tokenizer is not None:
                self.tokenizer = tokenizer
        self.device, self.dtype = device, dtype
        self.block_size = int(block_size)          # KV page size
        self.attn_backend = attn_backend
        self.resolved_attn_implementation = "sm100_paged_tree"
        self.fuse_gemms = bool(fuse_gemms) or env_flag("JETSPEC_FUSE_GEMMS")
        self.fused_moe_blocks = sum(1 for l in self.model.model.layers if hasattr(l.mlp, "w_gate_up"))
        self.eos_token_ids = resolve_eos(self.model, self.tokenizer)
        from ..core.model_runner import ModelRunner
        self.runner = ModelRunner(self.model)
        self.cfg = self.model.config
        self.tp = tensor_parallel      # jetspec_b200.parallel.TensorParallel or None
        # jetspec_b200.parallel.TokenShardedEP or None: every rank decodes its OWN request (one engine call per
        # rank, made together), the MoE layers' experts are sharded over the ranks
        self.ep = expert_parallel
        self._num_pages = num_pages
        self._max_seqs, self._max_seq_len = int(max_seqs), int(max_seq_len)
        self.pool: Optional[PagedKVPool] = None
        self._tree_session = None
        self._seq_counter = 0
        dev = torch.device(device)
        self.use_kernels = (dev.type == "cuda" and dtype == torch.bfloat16) if use_kernels is None else bool(use_kernels)
        self._fast = None
        self.last_stats: dict = {}

    # ------------------------------------------------------------------ pool
    def _ensure_pool(self, tokens_needed: int, seqs: int = 1) -> PagedKVPool:
        """Create (or grow, when nothing is resident) the KV pool."""
        need_pages = (tokens_needed + self.block_size - 1) // self.block_size + seqs
        want_pages = need_pages
        if self._num_pages is not None:
            want_pages = need_pages = int(self._num_pages)      # an explicit size is a hard size
        elif self.use_kernels:
            # captured graphs pin the pool: size it once for a full-length sequence
            want_pages = max(want_pages, (self._max_seq_len + self.block_size - 1) // self.block_size + seqs)
        max_len = max(self._max_seq_len, int(math.ceil(tokens_needed / max(1, seqs))) + self.block_size)
        if self.pool is not None:
            fits = self.pool.num_pages >= need_pages and self.pool.max_seq_len >= max_len \
                and self.pool.max_seqs >= seqs
            if fits:
                return self.pool
            if self.pool.resident():
                raise RuntimeError("cannot resize the KV pool while sequences are resident")
            if self.pool.frozen and self._tree_session is not None:
                # a session promised stable shapes: growing would silently drop its captured graphs
                raise RuntimeError("KV pool is frozen by live CUDA graphs and cannot grow; "
                                   "construct the engine with a larger num_pages / max_seq_len")
            # frozen but idle and outside a session: the graphs captured against the old pool are dropped with it
            # (self._fast below) and captured again on demand
        world = self.tp.world if getattr(self, "tp", None) is not None else 1
        self.pool = PagedKVPool(self.cfg.num_hidden_layers, self.cfg.num_key_value_heads // world, self.cfg.head_dim,
                                max(want_pages, 2), page_size=self.block_size,
                                max_seqs=max(self._max_seqs, seqs), max_seq_len=max_len,
                                device=self.device, dtype=self.dtype)
        self._fast = None
        return self.pool

    def _new_seq_id(self) -> int:
        self._seq_counter += 1
        return self._seq_counter

    def _ids(self, prompt) -> torch.Tensor:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer; pass token ids (1, T) instead")
            return self.tokenizer(prompt, return_tensors="pt").input_ids.to(self.device)
        return torch.as_tensor(prompt).reshape(1, -1).to(self.device)

    # --------------------------------------------------------------- forward
    @torch.inference_mode()
    def _forward(self, seq_ids, token_rows, past_lens, trees=None, taps=None, logits_rows=None):
        """One ragged forward.  ``token_rows[b]`` are the new tokens of sequence ``b``.

        Writes the new rows' K/V into the pool at ``slot_map[row, past + i]`` and attends
        through the slot map.  Returns ``(logits, tap_hidden, meta)``.
        """
        pool = self.pool
        meta = build_attn_metadata(pool, seq_ids, past_lens, trees=trees,
                                   num_query_nodes=None if trees is not None else [int(t.numel()) for t in token_rows],
                                   device=self.device)
        ids = torch.cat([t.reshape(-1) for t in token_rows]).to(self.device)
        scale = 1.0 / math.sqrt(self.cfg.head_dim)

        def attn(layer, q, k, v):
            kp, vp = pool.layer(layer)
            ops.kv_scatter(k, v, kp, vp, meta.slots)
            return ops.paged_tree_attention(q, kp, vp, pool.slot_map, meta.seq_rows, meta.cu_q, meta.past_lens,
                                            meta.mask_bits, scale, causal=meta.causal, max_q=meta.max_q)

        logits, hidden = self.model(ids, meta.positions.long(), attn, tap_layers=taps, logits_rows=logits_rows)
        return logits, hidden, meta

    def _prefill(self, seq_id: int, ids: torch.Tensor, taps=None, reserve: int = 0):
        """Causal prefill of one sequence; returns ``(last-row logits, tap hidden (T, taps*H))``."""
        T = ids.numel()
        self.pool.reserve(seq_id, T + reserve)
        logits, hidden, _ = self._forward([seq_id], [ids.reshape(-1)], [0], taps=taps,
                                          logits_rows=slice(T - 1, T))
        self.pool.state(seq_id).length = T
        return logits, hidden

    def _prefill_batch_member(self, seq_id: int, toks: torch.Tensor, taps, temperature: float):
        """Prefill one newly admitted request of a batch.  Returns ``(first token, tap hidden | None)``.  Under
        tensor parallelism the prompt runs through the sharded kernel path (the module forward holds full-size
        weights and cannot address the sharded KV pool)."""
        if self.tp is not None and temperature > 0.0:
            raise NotImplementedError("tensor-parallel batches decode greedily")
        kernel_path = self.tp is not None
        if not kernel_path and self.use_kernels and temperature <= 0.0 and self.cfg.head_dim == 128:
            from .fast_round import FastRound
            kernel_path = FastRound.get(self)._kernel_prefill_ok()      # the same prompt path as single requests
        if kernel_path:
            from .fast_round import FastRound
            T = int(toks.numel())
            have = self.pool.state(seq_id).capacity if self.pool.has(seq_id) else 0
            return FastRound.get(self)._prefill_kernels(seq_id, toks.reshape(1, -1), taps, max(T, have))
        logits, hidden, _ = self._forward([seq_id], [toks], [0], taps=taps,
                                          logits_rows=slice(toks.numel() - 1, toks.numel()))
        self.pool.state(seq_id).length = toks.numel()
        return int(sample(logits[-1], temperature)), hidden

    # ------------------------------------------------------------ AR decode
    @torch.inference_mode()
    def generate(self, prompt, sampling_params: SamplingParams = None) -> dict:
        """Autoregressive decode through the paged pool.  Returns ``{"token_ids","text"}``."""
        sp = sampling_params or SamplingParams()
        ids = self._ids(prompt)
        T = ids.shape[1]
        self._ensure_pool(T + sp.max_new_tokens + 1)
        sid = self._new_seq_id()
        try:
            if self.use_kernels:
                from .fast_round import FastRound
                return FastRound.get(self).generate_ar(sid, ids, sp)
            logits, _ = self._prefill(sid, ids, reserve=sp.max_new_tokens + 1)
            out = [int(sample(logits[-1], sp.temperature))]
            while len(out) < sp.max_new_tokens and out[-1] not in self.eos_token_ids:
                past = self.pool.state(sid).length
                logits, _, _ = self._forward([sid], [torch.tensor([out[-1]], device=self.device)], [past])
                self.pool.state(sid).length = past + 1
                out.append(int(sample(logits[-1], sp.temperature)))
            return {"token_ids": out, "text": decode_text(self.tokenizer, out)}
        finally:
            self.pool.free(sid)

    # ------------------------------------------------------------ tree decode
    def _session_check(self, session, session_prompt_capacity, prompt_len, tag):
        if not session:
            return
        cur = self._tree_session
        if cur is None:
            cap = _round_session_capacity(prompt_len) if session_prompt_capacity is None else int(session_prompt_capacity)
            if cap <= 0:
                raise ValueError(f"session_prompt_capacity must be positive; got {cap}")
            if prompt_len > cap:
                raise ValueError(f"tree session prompt_len mismatch: prompt_len={prompt_len} > session_prompt_capacity={cap}")
            self._tree_session = {"prompt_capacity": cap, "tag": tag}
            return
        problems = []
        cap = int(cur["prompt_capacity"])
        if session_prompt_capacity is not None and int(session_prompt_capacity) != cap:
            problems.append(f"session_prompt_capacity mismatch: expected {cap}, got {int(session_prompt_capacity)}")
        if prompt_len > cap:
            problems.append(f"prompt_len mismatch: prompt_len={prompt_len} > session_prompt_capacity={cap}")
        for k, v in tag.items():
            if cur["tag"].get(k) != v:
                problems.append(f"{k} mismatch: expected {cur['tag'].get(k)}, got {v}")
        if problems:
            raise ValueError("tree session mismatch: " + "; ".join(problems))

    def end_session(self) -> None:
        """Forget the session tag (captured graphs are kept while the pool is unchanged)."""
        self._tree_session = None

    @torch.inference_mode()
    def generate_tree(self, prompt, tree_drafter, block_size: int = 4, tree_width: int = 2, budget: int = 15,
                      algo: str = "accum_logp", algo_kwargs: Optional[dict] = None, target_layer_ids=None,
                      sampling_params: SamplingParams = None, return_stats: bool = False,
                      prompt_info: Optional[dict] = None, profile_table: Optional[dict] = None,
                      tree_diag: bool = False, session: bool = False,
                      session_prompt_capacity: Optional[int] = None, max_tree_depth: Optional[int] = None,
                      tree_depth: Optional[int] = None, extend_kwargs: Optional[dict] = None) -> dict:
        """Tree-speculative decode over the persistent paged pool.

        ``tree_depth`` sets ``block_size = tree_depth + 1`` (a ``block_size`` other than the
        default 4 must agree, else ``ValueError``).  ``session=True`` checks that successive
        calls keep the shapes the captured graphs and the pool were sized for.  Returns
        ``{"token_ids","text","tpf",["accept_lengths","tree_sizes","rounds"],["tree_nodes_per_depth"]}``.
        """
        sp = sampling_params or SamplingParams()
        committed = self._ids(prompt)
        if hasattr(tree_drafter, "reset_cache"):
            tree_drafter.reset_cache()
        if tree_depth is not None:
            tree_depth = int(tree_depth)
            if tree_depth < 1:
                raise ValueError(f"tree_depth must be >= 1; got {tree_depth}")
            if block_size != 4 and int(block_size) != tree_depth + 1:
                raise ValueError("block_size and tree_depth disagree: "
                                 f"block_size={block_size} implies tree_depth={int(block_size) - 1}, "
                                 f"but tree_depth={tree_depth}")
            block_size = tree_depth + 1
            if max_tree_depth is None:
                max_tree_depth = tree_depth
        max_depth = block_size - 1 if max_tree_depth is None else int(max_tree_depth)
        if max_depth < 0:
            raise ValueError(f"max_tree_depth must be >= 0; got {max_depth}")
        prompt_len = committed.shape[1]
        D = max(1, block_size - 1)
        ext_budget = int((extend_kwargs or {}).get("ext_budget", D)) if extend_kwargs else 0
        n_max = bucket_for_n(budget + ext_budget)
        taps = list(target_layer_ids) if (target_layer_ids is not None and block_size > 1) else None
        tag = {"block_size": int(block_size), "cache_block_size": self.block_size, "dtype": str(self.dtype),
               "need_hidden": taps is not None, "budget_bucket": n_max, "max_tree_depth": max_depth,
               "max_new_tokens": int(sp.max_new_tokens), "attn_backend": self.attn_backend}
        self._session_check(session, session_prompt_capacity, prompt_len, tag)
        cap_prompt = self._tree_session["prompt_capacity"] if (session and self._tree_session) else prompt_len
        total = cap_prompt + sp.max_new_tokens + max_depth + 1 + n_max
        self._ensure_pool(total)
        algo_obj = get_algorithm(algo, **(algo_kwargs or {}))
        sid = self._new_seq_id()
        try:
            graph_sampling = sp.temperature <= 0.0 or (self.tp is None and self.ep is None)
            if self.use_kernels and graph_sampling and not env_flag("JETSPEC_FORCE_EAGER_TREE"):
                from .fast_round import FastRound
                fast = FastRound.get(self)
                if fast.supports_tree(tree_drafter, algo_obj, block_size, tree_width, budget, extend_kwargs):
                    return fast.generate_tree(sid, committed, tree_drafter, algo_obj, block_size, tree_width, budget,
                                              taps, sp, return_stats, tree_diag, max_depth, prompt_info, profile_table,
                                              total, extend_kwargs=extend_kwargs)
            return self._generate_tree_eager(sid, committed, tree_drafter, algo_obj, algo, algo_kwargs, block_size,
                                             tree_width, budget, taps, sp, return_stats, prompt_info, profile_table,
                                             tree_diag, max_depth, extend_kwargs, total)
        finally:
            self.pool.free(sid)

    def _draft_and_build(self, tree_drafter, algo_obj, committed, target_hidden, D, block_size, tree_width, budget,
                         prompt_info, profile_table, extend_kwargs, root_token: Optional[int] = None,
                         host_only: bool = False):
        """One drafter call → tree.  Uses the drafter's direct top-k when it has one (and its host-only form,
        ``propose_topk_at``, when the proposal needs nothing from the device)."""
        root = int(committed[0, -1]) if root_token is None else int(root_token)
        topk_fn = getattr(tree_drafter, "propose_topk", None)
        at_fn = getattr(tree_drafter, "propose_topk_at", None)
        caps_fn = getattr(algo_obj, "caps_from_topk", None)
        if (topk_fn is not None or at_fn is not None) and caps_fn is not None and not extend_kwargs:
            if at_fn is not None:
                tok, lp = at_fn(int(committed.shape[-1]), D, tree_width)
            else:
                tok, lp = topk_fn(committed, D, tree_width, target_hidden=target_hidden)
            tree = build_from_topk(algo_obj.name, root, tok, lp, budget, "host" if host_only else self.device,
                                   algo_kwargs=_algo_init_kwargs(algo_obj), tree_width=tree_width,
                                   prompt_info=prompt_info, profile_table=profile_table)
            return tree
        draft_logits = tree_drafter.propose_logits(committed, D, target_hidden=target_hidden).to(self.device)
        tree = algo_obj.build(root_token=root, draft_logits=draft_logits, block_size=block_size,
                              tree_width=tree_width, budget=budget, device=self.device,
                              profile_table=profile_table, prompt_info=prompt_info)
        if extend_kwargs:
            lp = torch.log_softmax(draft_logits[0].float(), dim=-1)
            topk_lp, topk_tok = torch.topk(lp, tree_width, dim=-1)
            tree = maybe_extend_tree(tree, topk_tok, topk_lp, tree_drafter, committed, target_hidden,
                                     tree_width, extend_kwargs)
        return tree

    def _generate_tree_eager(self, sid, committed, tree_drafter, algo_obj, algo, algo_kwargs, block_size, tree_width,
                             budget, taps, sp, return_stats, prompt_info, profile_table, tree_diag, max_depth,
                             extend_kwargs, total):
        pool = self.pool
        D = max(1, block_size - 1)
        prompt_len = committed.shape[1]
        logits, hidden = self._prefill(sid, committed[0], taps=taps, reserve=total - prompt_len)
        hid_buf, hid_len = None, 0
        if hidden is not None:
            hid_buf = torch.empty(prompt_len + sp.max_new_tokens + max_depth + 2, hidden.shape[-1],
                                  dtype=hidden.dtype, device=self.device)
            hid_buf[:prompt_len] = hidden
            hid_len = prompt_len
        first = int(sample(logits[-1], sp.temperature))
        new_ids = [first]
        committed = torch.cat((committed, torch.tensor([[first]], device=self.device)), 1)
        accept_lengths, tree_sizes, rounds = [], [], 0
        depth_hist = torch.zeros(max_depth + 2, dtype=torch.long) if tree_diag else None
        done = first in self.eos_token_ids
        while len(new_ids) < sp.max_new_tokens and not done:
            th = hid_buf[:hid_len].unsqueeze(0) if hid_buf is not None else None
            tree = self._draft_and_build(tree_drafter, algo_obj, committed, th, D, block_size, tree_width, budget,
                                         prompt_info, profile_table, extend_kwargs)
            n = tree.num_nodes
            tree_max_depth = int(tree.depth.max())
            if tree_max_depth > max_depth:
                raise ValueError(f"tree depth {tree_max_depth} exceeds max_tree_depth {max_depth}; "
                                 "raise max_tree_depth when extending trees")
            if depth_hist is not None:
                depth_hist += torch.bincount(tree.depth.cpu(), minlength=depth_hist.numel())[: depth_hist.numel()]
            past = pool.state(sid).length
            logits, hidden, _ = self._forward([sid], [tree.token_ids], [past], trees=[tree], taps=taps)
            rounds += 1
            if sp.temperature <= 0.0:
                path, acc, corr = gpu_tree_accept(tree.token_ids, logits.argmax(-1), tree.parent_indices,
                                                  tree.depth, max_depth=max(tree_max_depth, 1))
                path_l, corr = path.tolist(), int(corr)
            else:
                path_l, acc, corr = tree_accept(tree, logits.unsqueeze(0), sp.temperature)
            pool.commit_path(sid, past, n, path_l)
            if hid_buf is not None:
                hid_buf[hid_len:hid_len + len(path_l)] = hidden[path_l]
                hid_len += len(path_l)
            block = tree.token_ids[path_l[1:]].tolist() + [corr]
            committed = torch.cat((committed, torch.tensor([block], device=self.device)), 1)
            accept_lengths.append(acc + 1)
            tree_sizes.append(n)
            for t in block:
                new_ids.append(int(t))
                if int(t) in self.eos_token_ids:
                    done = True
                    break
        new_ids = new_ids[: sp.max_new_tokens]
        out = {"token_ids": new_ids, "text": decode_text(self.tokenizer, new_ids),
               "tpf": (len(new_ids) / rounds if rounds else 0.0)}
        if return_stats:
            out.update(accept_lengths=accept_lengths, tree_sizes=tree_sizes, rounds=rounds)
        if depth_hist is not None:
            out["tree_nodes_per_depth"] = depth_hist.tolist()
        return out

    # ------------------------------------------------------------ batching
    def _make_scheduler(self, n_requests: int, max_batch_size: Optional[int]) -> Scheduler:
        return Scheduler(self.pool, max_batch_size=max_batch_size or min(n_requests, self.pool.max_seqs),
                         prefill_batch_size=max_batch_size or min(n_requests, self.pool.max_seqs))

    def _ensure_room(self, sched: Scheduler, req: SequenceRequest, tokens: int) -> bool:
        """Make sure ``req`` has ``tokens`` mapped positions, evicting + re-queueing other running
        sequences when the pool is short.  False when ``req`` itself had to yield."""
        pool = self.pool
        while not pool.allocate_slots(req.seq_id, tokens, allow_evict=False):
            others = [r for r in sched.running.values() if r.seq_id != req.seq_id and pool.has(r.seq_id)]
            if not others:
                raise RuntimeError(f"KV pool too small for a single sequence of {tokens} tokens")
            victim = sched._pick_victim(others)
            sched.evict_sequence(victim.seq_id)
            sched.restore_sequence(victim.seq_id)
        return True

    @torch.inference_mode()
    def generate_batch(self, prompts: list, sampling_params: SamplingParams = None,
                       max_batch_size: Optional[int] = None) -> list:
        """Continuous-batching AR decode.  Returns ``[{"token_ids","text"}, …]`` in prompt order.

        Requests are queued with the scheduler; each iteration prefills newly admitted
        requests, runs ONE ragged decode forward over all running sequences, and retires
        finished ones so that waiting requests take their pages.
        """
        sp = sampling_params or SamplingParams()
        id_rows = [self._ids(p)[0] for p in prompts]
        longest = max(int(r.numel()) for r in id_rows) + sp.max_new_tokens + 1
        if self.pool is None or self._num_pages is None:
            self._ensure_pool(sum(int(r.numel()) + sp.max_new_tokens + 1 for r in id_rows), seqs=len(prompts))
        if self.pool.max_seq_len < longest:
            self._ensure_pool(longest * len(prompts), seqs=len(prompts))
        sched = self._make_scheduler(len(prompts), max_batch_size)
        reqs = {}
        for i, row in enumerate(id_rows):
            r = SequenceRequest(seq_id=self._new_seq_id(), input_ids=row.tolist(), max_new_tokens=sp.max_new_tokens,
                                temperature=sp.temperature, reserve_tokens=1)
            reqs[r.seq_id] = i
            sched.admit_request(r)
        results = [None] * len(prompts)
        self.last_stats = {"steps": 0, "evictions": 0, "max_batch": 0}
        while sched.has_work:
            out = sched.step()
            self.last_stats["evictions"] += len(out.evicted)
            for v in out.evicted:
                sched.restore_sequence(v.seq_id)
            for req in out.admitted:
                toks = torch.tensor(req.input_ids, device=self.device)
                first, _ = self._prefill_batch_member(req.seq_id, toks, None, sp.temperature)
                self._record_token(sched, req, first, results, reqs)
            running = [r for r in sched.running.values() if not r.is_prefill]
            if not running:
                if not out.admitted and sched.waiting_queue and not sched.running:
                    raise RuntimeError("scheduler stalled: a waiting request does not fit in an empty pool")
                continue
            ready = []
            for r in running:
                if r.seq_id in sched.running and self._ensure_room(sched, r, self.pool.state(r.seq_id).length + 1):
                    ready.append(r)
            ready = [r for r in ready if r.seq_id in sched.running]
            if not ready:
                continue
            self.last_stats["steps"] += 1
            self.last_stats["max_batch"] = max(self.last_stats["max_batch"], len(ready))
            past = [self.pool.state(r.seq_id).length for r in ready]
            if self.use_kernels and sp.temperature <= 0.0 and self.cfg.head_dim == 128 \
                    and (env_flag("JETSPEC_BATCH_GRAPH", True) or self.tp is not None):
                # one graph replay per decode step: every sequence contributes a one-node "tree"
                from .fast_round import FastRound
                nodes = [_OneNode(r.input_ids[-1]) for r in ready]
                greedy, _ = FastRound.get(self).batch_verify([r.seq_id for r in ready], nodes, past, 1)
                nxt = [g[0] for g in greedy]
            else:
                toks = [torch.tensor(r.input_ids[-1:], device=self.device) for r in ready]
                logits, _, _ = self._forward([r.seq_id for r in ready], toks, past)
                nxt = sample(logits, sp.temperature).tolist()
            for r, p, t in zip(ready, past, nxt):
                self.pool.state(r.seq_id).length = p + 1
                self.pool.touch(r.seq_id)
                self._record_token(sched, r, int(t), results, reqs)
        return results

    def _record_token(self, sched, req, tok, results, reqs):
        sched.mark_decode_step(req.seq_id, tok)
        if tok in self.eos_token_ids or len(req.output_tokens) >= req.max_new_tokens:
            ids = req.output_tokens[: req.max_new_tokens]
            results[reqs[req.seq_id]] = {"token_ids": ids, "text": decode_text(self.tokenizer, ids)}
            sched.mark_finished(req.seq_id)

    @torch.inference_mode()
    def generate_tree_batch(self, prompts: list, tree_drafter, block_size: int = 4, tree_width: int = 2,
                            budget: int = 15, algo: str = "accum_logp", algo_kwargs: Optional[dict] = None,
                            sampling_params: SamplingParams = None, target_layer_ids=None,
                            max_batch_size: Optional[int] = None, return_stats: bool = False) -> list:
        """Batched tree-speculative decode: every round verifies all live sequences' trees in ONE
        ragged forward through the paged pool.  ``tree_drafter`` may be one stateless drafter, a
        list with one drafter per prompt, or a stateful drafter offering ``clone()``.
        Returns ``[{"token_ids","text","tpf"}, …]`` in prompt order.
        """
        sp = sampling_params or SamplingParams()
        id_rows = [self._ids(p)[0] for p in prompts]
        D = max(1, block_size - 1)
        n_max = bucket_for_n(budget)
        taps = list(target_layer_ids) if (target_layer_ids is not None and block_size > 1) else None
        per_seq = lambda r: int(r.numel()) + sp.max_new_tokens + D + 1 + n_max
        if self.pool is None or self._num_pages is None:
            self._ensure_pool(sum(per_seq(r) for r in id_rows), seqs=len(prompts))
        if self.pool.max_seq_len < max(per_seq(r) for r in id_rows):
            self._ensure_pool(max(per_seq(r) for r in id_rows) * len(prompts), seqs=len(prompts))
        algo_obj = get_algorithm(algo, **(algo_kwargs or {}))
        if isinstance(tree_drafter, (list, tuple)):
            drafters = list(tree_drafter)
        elif hasattr(tree_drafter, "clone"):
            drafters = [tree_drafter.clone() for _ in prompts]
        else:
            drafters = [tree_drafter] * len(prompts)
        for d in drafters:
            if hasattr(d, "reset_cache"):
                d.reset_cache()
        sched = self._make_scheduler(len(prompts), max_batch_size)
        state, reqs = {}, {}
        batch_graph = env_flag("JETSPEC_BATCH_GRAPH", True)     # graph-replayed verify forward for the whole batch
        # when the graph path is certain to take every tree, trees are built as host lists only (no device tensors)
        if self.tp is not None:
            batch_graph = True         # the sharded stack exists on the kernel path only
        graph_ok = bool(batch_graph and self.use_kernels and sp.temperature <= 0.0 and self.cfg.head_dim == 128
                        and n_max <= 256)
        for i, row in enumerate(id_rows):
            r = SequenceRequest(seq_id=self._new_seq_id(), input_ids=row.tolist(), max_new_tokens=sp.max_new_tokens,
                                temperature=sp.temperature, use_tree=True, tree_drafter=drafters[i],
                                reserve_tokens=n_max + 1)
            reqs[r.seq_id] = i
            sched.admit_request(r)
        results = [None] * len(prompts)

        def finish(req, st):
            ids = req.output_tokens[: sp.max_new_tokens]
            res = {"token_ids": ids, "text": decode_text(self.tokenizer, ids),
                   "tpf": (len(ids) / st["rounds"] if st["rounds"] else 0.0)}
            if return_stats:
                res.update(accept_lengths=st["acc"], rounds=st["rounds"])
            results[reqs[req.seq_id]] = res
            sched.mark_finished(req.seq_id)

        while sched.has_work:
            out = sched.step()
            for v in out.evicted:
                sched.restore_sequence(v.seq_id)
            for req in out.admitted:
                toks = torch.tensor(req.input_ids, device=self.device)
                first, hidden = self._prefill_batch_member(req.seq_id, toks, taps, sp.temperature)
                prior = state.get(req.seq_id, {"rounds": 0, "acc": []})
                state[req.seq_id] = {"committed": torch.cat((toks, torch.tensor([first], device=self.device))),
                                     "hidden": hidden, "rounds": prior["rounds"], "acc": prior["acc"]}
                if hasattr(req.tree_drafter, "reset_cache"):
                    req.tree_drafter.reset_cache()
                req.output_tokens.append(first)
                req.is_prefill = False
                if first in self.eos_token_ids or len(req.output_tokens) >= sp.max_new_tokens:
                    finish(req, state[req.seq_id])
            live = [r for r in sched.running.values() if not r.is_prefill]
            if not live:
                if not out.admitted and sched.waiting_queue and not sched.running:
                    raise RuntimeError("scheduler stalled: a waiting request does not fit in an empty pool")
                continue
            ready = []
            for r in live:
                if r.seq_id in sched.running:
                    self._ensure_room(sched, r, self.pool.state(r.seq_id).length + n_max + 1)
                    ready.append(r)
            live = [r for r in ready if r.seq_id in sched.running]
            if not live:
                continue
            trees = []
            for r in live:
                st = state[r.seq_id]
                th = st["hidden"].unsqueeze(0) if st["hidden"] is not None else None
                trees.append(self._draft_and_build(r.tree_drafter, algo_obj, st["committed"].unsqueeze(0), th, D,
                                                   block_size, tree_width, budget, None, None, None,
                                                   root_token=r.output_tokens[-1], host_only=graph_ok))
            past = [self.pool.state(r.seq_id).length for r in live]
            graph_verify = False
            if self.use_kernels and sp.temperature <= 0.0 and batch_graph:
                from .fast_round import FastRound
                fast = FastRound.get(self)
                graph_verify = fast.supports_batch_verify(trees, taps)
            if self.tp is not None and not graph_verify:
                raise NotImplementedError("tensor-parallel batches need trees the graph path covers "
                                          "(greedy, head_dim 128, at most 256 nodes, host-built trees)")
            if graph_verify:
                # the whole verify forward of all live trees is one graph replay; the logits are never written
                greedy_seq, hidden = fast.batch_verify([r.seq_id for r in live], trees, past, n_max, taps)
                nb = hidden.shape[0] // len(live) if hidden is not None else 0
                cu = [b * nb for b in range(len(live) + 1)]
                logits, host_accept, greedy_all = None, True, None
            else:
                logits, hidden, meta = self._forward([r.seq_id for r in live], [t.token_ids for t in trees], past,
                                                     trees=trees, taps=taps)
                cu = meta.cu_q.tolist()
                # greedy: ONE argmax over the whole ragged batch and one device read; acceptance itself runs on
                # the host lists the builder left on each tree (no per-sequence launches or synchronisations)
                host_accept = sp.temperature <= 0.0 and all(t.host is not None for t in trees)
                greedy_all = logits.argmax(-1).tolist() if host_accept else None
            for b, (r, tree) in enumerate(zip(live, trees)):
                st = state[r.seq_id]
                lg = logits[cu[b]:cu[b + 1]] if logits is not None else None
                if graph_verify:
                    h_tok, h_par, h_dep = tree.host
                    path_l, acc, corr = host_tree_accept(h_tok, h_par, h_dep, greedy_seq[b])
                elif host_accept:
                    h_tok, h_par, h_dep = tree.host
                    path_l, acc, corr = host_tree_accept(h_tok, h_par, h_dep, greedy_all[cu[b]:cu[b + 1]])
                elif sp.temperature <= 0.0:
                    path, acc, corr = gpu_tree_accept(tree.token_ids, lg.argmax(-1), tree.parent_indices, tree.depth,
                                                      max_depth=max(int(tree.depth.max()), 1))
                    path_l, corr = path.tolist(), int(corr)
                else:
                    path_l, acc, corr = tree_accept(tree, lg.unsqueeze(0), sp.temperature)
                self.pool.commit_path(r.seq_id, past[b], tree.num_nodes, path_l)
                if st["hidden"] is not None:
                    st["hidden"] = torch.cat((st["hidden"], hidden[cu[b]:cu[b] + tree.num_nodes][path_l]), 0)
                if tree.host is not None:
                    block = [tree.host[0][i] for i in path_l[1:]] + [corr]
                else:
                    block = tree.token_ids[path_l[1:]].tolist() + [corr]
                st["committed"] = torch.cat((st["committed"], torch.tensor(block, device=self.device)))
                st["rounds"] += 1
                st["acc"].append(acc + 1)
                stop = False
                for t in block:
                    r.output_tokens.append(int(t))
                    if int(t) in self.eos_token_ids:
                        stop = True
                        break
                r.input_ids = [r.output_tokens[-1]]
                if stop or len(r.output_tokens) >= sp.max_new_tokens:
                    finish(r, st)
        return results


def _algo_init_kwargs(algo_obj) -> dict:
    """Constructor knobs of an algorithm instance, for re-instantiation by name."""
    keys = ("beta", "g_0", "tau", "gap_high", "gap_low", "templates", "force_baseline", "gap_threshold",
            "open_ended_template")
    return {k: getattr(algo_obj, k) for k in keys if hasattr(algo_obj, k)}
