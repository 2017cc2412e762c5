"""Kernel path of the engine: a whole decode round replayed from one CUDA graph.

A round is ``draft-head step → tree build → verify forward → accept → commit``.  On a
B200 with bf16 weights every step is a hand-written sm_100a kernel launched with
programmatic dependent launch, all captured once per tree bucket; the host stages
at most a few hundred bytes (scripted drafter candidates / fan-out caps), replays
the graph and reads one small result record — one host synchronisation per round,
as in the reference's production path (``jetspec/inference_engine/engine.py:881-1164``)
but with the drafter, the tree builder and the commit inside the same graph.

Per-sequence device state (int32 words, see ``csrc/tree_kernels.cu``):
``[past, draft_ctx, new_ctx_rows, done, generated, n_nodes, rounds]``.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import numpy as np
import torch

from ..core.llm import decode_text
from ..drafters.head import DraftHeadTreeDrafter
from ..models.qwen3 import MLP
from ..parallel.tp import stack_rows
from ..ops import cuda_ext as X
from ..ops import reference as ref
from ..sampling import SamplingParams, sample
from ..tree.builder import topk_rows

ST_PAST, ST_CTX, ST_NEW, ST_DONE, ST_GEN, ST_NNODES, ST_ROUNDS = range(7)
_PDL = os.environ.get("JETSPEC_PDL", "1") != "0"
# Off by default: measured slower (5.68 -> 6.5 ms/round at best).  The decoder GEMMs at 128 rows are bound by
# their per-launch latency chain, not by HBM: with L2-resident weights they run no faster (o_proj 12.3 us cold,
# 14.7 us hot), and the prefetch requests compete with the GEMMs' own loads.
_L2_PREFETCH = os.environ.get("JETSPEC_L2_PREFETCH", "0") == "1"


def _i32(n, device, fill=0):
    return torch.full((n,), fill, dtype=torch.int32, device=device)


def local_dims(cfg, world: int = 1):
    """The per-rank view of a model's geometry under tensor parallelism."""
    import types
    return types.SimpleNamespace(
        num_attention_heads=cfg.num_attention_heads // world, num_key_value_heads=cfg.num_key_value_heads // world,
        head_dim=cfg.head_dim, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size // world,
        rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, vocab_size=cfg.vocab_size,
        num_hidden_layers=cfg.num_hidden_layers)


def kernel_layer_weights(layers, cfg=None, tp=None, ep=None) -> list:
    """Kernel-ready per-layer weights: fused QKV (and K|V alone), tile-interleaved gate/up; with
    tensor parallelism, this rank's shards of them; with expert parallelism, this rank's experts."""
    out = []
    if tp is not None:
        from ..parallel.tp import shard_attention, shard_mlp
        for layer in layers:
            if not isinstance(layer.mlp, MLP) or layer.self_attn.q_proj.bias is not None:
                raise NotImplementedError("the tensor-parallel graph path covers dense, bias-free layers")
            d = {"ln1": layer.input_layernorm.weight, "ln2": layer.post_attention_layernorm.weight}
            d.update(shard_attention(layer, cfg, tp.rank, tp.world))
            m = shard_mlp(layer.mlp, tp.rank, tp.world, lambda g, u: X.interleave_gate_up(g, u, 128))
            d.update({"gu": m["gu"], "down": m["down"]})
            out.append(d)
        return _finish_layer_weights(out)
    for layer in layers:
        a = layer.self_attn
        if a.q_proj.bias is not None:
            raise NotImplementedError("the graph path covers bias-free attention projections")
        d = {
            "ln1": layer.input_layernorm.weight, "ln2": layer.post_attention_layernorm.weight,
            "qkv": stack_rows([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight]),
            "kv": stack_rows([a.k_proj.weight, a.v_proj.weight]),
            "qn": a.q_norm.weight, "kn": a.k_norm.weight, "o": a.o_proj.weight,
        }
        if isinstance(layer.mlp, MLP):
            g = layer.mlp.gate_proj.weight
            d["gu_bn"] = X.gu_tile(g.shape[0]) if isinstance(g, torch.Tensor) else 128   # the NVFP4 kernel has 128-column tiles
            d["gu"] = X.interleave_gate_up(g, layer.mlp.up_proj.weight, d["gu_bn"])
            d["down"] = layer.mlp.down_proj.weight
        else:   # sparse MoE: router + permutation kernels and two grouped GEMMs, all static-shape (no host read)
            m = layer.mlp
            if ep is not None:
                gu_l, dn_l = ep.shard(m.w_gate_up, m.w_down)
                d["moe"] = (m.gate.weight, gu_l, dn_l, int(m.top_k), bool(m.norm_topk_prob))
                d["moe_ep"] = True
            else:
                d["moe"] = (m.gate.weight, m.w_gate_up, m.w_down, int(m.top_k), bool(m.norm_topk_prob))
        out.append(d)
    return _finish_layer_weights(out)


def _finish_layer_weights(out: list) -> list:
    """NVFP4 layers: build the tile-ordered block scales and read the per-tensor scales once, up front."""
    for d in out:
        d["fp4"] = not isinstance(d["qkv"], torch.Tensor)
        if d["fp4"]:
            for k in ("qkv", "kv", "o", "gu", "down"):
                if k in d:
                    d[k].swizzled()
                    d[k]._w_scale = float(d[k].outer)
    return out


_WIDE_GU_ROWS = 1024


def _gu_wide(L: dict) -> torch.Tensor:
    """The layer's gate/up weight re-interleaved for 256-column tiles (128 gate + 128 up rows per tile)."""
    if "gu256" not in L:
        w, h = L["gu"], L.get("gu_bn", 128) // 2
        I2, H = w.shape
        v = w.view(I2 // (2 * h), 2, h, H)
        L["gu256"] = X.interleave_gate_up(v[:, 0].reshape(I2 // 2, H), v[:, 1].reshape(I2 // 2, H), 256)
    return L["gu256"]


class _Stack:
    """Static activation buffers of one decoder stack for a fixed row count ``T``."""

    def __init__(self, cfg, T: int, device, max_keys: int):
        H, I = cfg.hidden_size, cfg.intermediate_size
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        bf = dict(dtype=torch.bfloat16, device=device)
        self.T = T
        self.x = torch.zeros(T, H, **bf)
        self.h = torch.zeros(T, H, **bf)
        self.qkv = torch.zeros(T, (Hq + 2 * Hkv) * D, **bf)
        self.q = torch.zeros(T, Hq, D, **bf)
        self.attn = torch.zeros(T, Hq * D, **bf)
        self.act = torch.zeros(T, I, **bf)
        self._q4: dict = {}
        self.splits = X.attn_splits_for(T, Hq, Hkv, max_keys)
        self.attn_ws = None
        if self.splits > 1:
            self.attn_ws = {"o": torch.zeros(self.splits, T, Hq, D, dtype=torch.float32, device=device),
                            "ml": torch.zeros(self.splits, T, Hq, 2, dtype=torch.float32, device=device)}


def _q4(st: _Stack, K: int) -> dict:
    """The stack's NVFP4 staging buffers for activations of width ``K`` (allocated on first use)."""
    if K not in st._q4:
        st._q4[K] = X.nvfp4_act_buffers(st.T, K, st.x.device)
    return st._q4[K]


def _decoder_layer_fp4(cfg, L, st, attend, pdl, tp) -> int:
    """One decoder layer on NVFP4 weights: every GEMM input is quantised on the fly (the two norms are fused
    into their quantisation kernels) and multiplied on the block-scaled tensor-core path."""
    eps = cfg.rms_norm_eps
    h4 = X.quant_nvfp4(st.x, _q4(st, st.x.shape[1]), norm_w=L["ln1"], eps=eps, pdl=pdl)
    X.gemm_nvfp4(h4, L["qkv"], out=st.qkv, pdl=pdl)
    attend()
    a4 = X.quant_nvfp4(st.attn, _q4(st, st.attn.shape[1]), pdl=pdl)
    if tp is None:
        X.gemm_nvfp4(a4, L["o"], out=st.x, residual=st.x, pdl=pdl)
    else:
        tp.gemm_allreduce_nvfp4(a4, L["o"], st.x, residual=st.x, pdl=pdl)
    h4 = X.quant_nvfp4(st.x, _q4(st, st.x.shape[1]), norm_w=L["ln2"], eps=eps, pdl=pdl)
    X.gemm_nvfp4(h4, L["gu"], out=st.act, epi=X.EPI_SWIGLU, pdl=pdl)
    m4 = X.quant_nvfp4(st.act, _q4(st, st.act.shape[1]), pdl=pdl)
    if tp is None:
        X.gemm_nvfp4(m4, L["down"], out=st.x, residual=st.x, pdl=pdl)
    else:
        tp.gemm_allreduce_nvfp4(m4, L["down"], st.x, residual=st.x, pdl=pdl)
    return 8


class WeightPrefetcher:
    """Pulls the NEXT GEMM's weights into L2 on a side stream while the current kernels run.

    A decode round is a chain of short dependent kernels; while attention, the norms and every GEMM's
    prologue and epilogue run, HBM is idle.  ``ahead(w)`` is called right before a kernel is launched on
    the main stream: the side stream waits for everything launched so far, then issues L2 prefetches for
    ``w`` (at most ``cap`` bytes, so a prefetch never evicts what was prefetched before it and is still
    unread).  Works eagerly and inside CUDA-graph capture (the fork/join become graph edges).
    """

    def __init__(self, device, cap_bytes: int = 72 << 20, ctas: int = 8):
        self.side = torch.cuda.Stream(device)
        self.cap, self.ctas = int(cap_bytes), int(ctas)
        self.launches = 0

    def ahead(self, w) -> None:
        if not isinstance(w, torch.Tensor):
            w = w.packed                                   # NVFP4: the codes are the bulk of the bytes
        main = torch.cuda.current_stream()
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            X.l2_prefetch(w, self.cap, self.ctas)
        self.launches += 1

    def join(self) -> None:
        torch.cuda.current_stream().wait_stream(self.side)


def decoder_layers(cfg, layers, st: _Stack, k_pools, v_pools, slot_map, seq_rows, cu_q, past_lens, positions, slots,
                   mask_bits, causal: bool, freq, taps=None, tap_ids=None, pdl=True, tp=None, prefetch=None,
                   then_prefetch=None, final_norm=None, ep=None) -> int:
    """Launch the kernels of ``len(layers)`` decoder layers on ``st.x`` (in place).  Returns the launch count.

    ``final_norm = (weight, out)`` also applies the model's last RMSNorm to the stack's output.  Under tensor
    parallelism every row-parallel GEMM's all-reduce finishes inside the kernel that also computes the NEXT
    RMSNorm (the following layer's input norm, or ``final_norm``), so a layer launches no separate norm kernels."""
    Hq, Hkv, D, H = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size
    scale, eps = 1.0 / math.sqrt(D), cfg.rms_norm_eps
    last = len(layers) - 1
    n = 0
    # the split merge is a second launch unless the tcgen05 kernel does it inside a cluster
    in_kernel = (X.attn_impl(Hq, Hkv, 0 if mask_bits is None else mask_bits.shape[1]) == "tc"
                 and X.attn_merges_in_cluster(st.T, Hq, Hkv, st.splits))
    merge_launch = 1 if st.splits > 1 and not in_kernel else 0
    fuse_norm = tp is not None and tp.push_only >= 2     # the all-reduce tail computes the following norm
    h_ready = False                                      # st.h already holds this layer's normalised input
    for li, L in enumerate(layers):
        def attend(li=li, L=L):
            X.qkv_post(st.qkv, L["qn"], L["kn"], positions, slots, freq, st.q, k_pools[li], v_pools[li], Hq, Hkv, eps,
                       pdl=pdl)
            X.paged_tree_attention(st.q, k_pools[li], v_pools[li], slot_map, seq_rows, cu_q, past_lens, mask_bits,
                                   scale, causal, st.T, out=st.attn, splits=st.splits, ws=st.attn_ws, pdl=pdl)
        if L.get("fp4"):
            h_ready = False
            n += _decoder_layer_fp4(cfg, L, st, attend, pdl, tp) + 2 + merge_launch
            if taps is not None and li != last:
                for j, t in enumerate(tap_ids):
                    if t == li:
                        X.gather_rows(st.x, None, taps, dst_col0=j * H, pdl=pdl)
                        n += 1
            continue
        pf = prefetch
        if not h_ready:
            X.rmsnorm(st.x, L["ln1"], eps, out=st.h, pdl=pdl)
            n += 1
        h_ready = False
        if pf is not None:
            pf.ahead(L["o"])                   # o_proj's weights arrive while qkv, the KV scatter and attention run
        X.gemm(st.h, L["qkv"], out=st.qkv, pdl=pdl)
        attend()
        if pf is not None and "gu" in L:
            pf.ahead(L["gu"])
        if tp is None:
            X.gemm(st.attn, L["o"], out=st.x, residual=st.x, pdl=pdl)
            X.rmsnorm(st.x, L["ln2"], eps, out=st.h, pdl=pdl)
        else:   # row-parallel: GEMM fused with the all-reduce over NVLink peer memory, finished together with ln2
            tp.gemm_allreduce(st.attn, L["o"], st.x, residual=st.x, pdl=pdl, norm_w=L["ln2"], norm_out=st.h, eps=eps)
        if "moe" in L and L.get("moe_ep"):
            # expert-parallel layer: this rank's rows travel to the experts' owners and back inside the kernels;
            # the finishing kernel of the combine also computes the next RMSNorm
            gate_w, gu_l, dn_l, top_k, renorm = L["moe"]
            nw, nout = None, None
            if li != last and not layers[li + 1].get("fp4"):
                nw, nout, h_ready = layers[li + 1]["ln1"], st.h, True
            elif li == last and final_norm is not None:
                nw, nout = final_norm
                final_norm = None
            ep.moe_layer(st.x, st.h, gate_w, gu_l, dn_l, renorm, out=st.x, norm_w=nw, norm_out=nout, eps=eps, pdl=pdl)
            n += 5 + merge_launch + 6          # + router GEMM, route + counts, dispatch, two grouped GEMMs, finish
            if taps is not None and li != last:
                for j, t in enumerate(tap_ids):
                    if t == li:
                        X.gather_rows(st.x, None, taps, dst_col0=j * H, pdl=pdl)
                        n += 1
            continue
        if "moe" in L:
            gate_w, w_gu, w_dn, top_k, renorm = L["moe"]
            X.moe_forward(st.h, gate_w, w_gu, w_dn, top_k, renorm, residual=st.x)     # st.x += MoE(st.h), in the combine kernel
            n += 5 + merge_launch + 8          # + router GEMM, route, sort, row gather, two grouped GEMMs, invert, combine (+ residual)
            if taps is not None and li != last:
                for j, t in enumerate(tap_ids):
                    if t == li:
                        X.gather_rows(st.x, None, taps, dst_col0=j * H, pdl=pdl)
                        n += 1
            continue
        if pf is not None:
            pf.ahead(L["down"])
        if st.T >= _WIDE_GU_ROWS and tp is None:
            # many row tiles (batched verify, long prefill): compute bound, 128x256 tiles measured 24 % faster at
            # 2048 rows (519 -> 396 us); the 256-interleaved copy of the weight is made on first use
            X.gemm(st.h, _gu_wide(L), out=st.act, epi=X.EPI_SWIGLU, bn=256, split=1, deep=0, pdl=pdl)
        else:
            X.gemm(st.h, L["gu"], out=st.act, epi=X.EPI_SWIGLU, bn=L.get("gu_bn"), pdl=pdl)
        if pf is not None:
            nxt = layers[li + 1]["qkv"] if li != last else then_prefetch
            if nxt is not None:
                pf.ahead(nxt)
        if tp is None:
            X.gemm(st.act, L["down"], out=st.x, residual=st.x, pdl=pdl)
        else:
            nw, nout = None, None
            if fuse_norm and li != last and not layers[li + 1].get("fp4"):
                nw, nout, h_ready = layers[li + 1]["ln1"], st.h, True
            elif fuse_norm and li == last and final_norm is not None:
                nw, nout = final_norm
                final_norm = None                      # done by the all-reduce tail
            tp.gemm_allreduce(st.act, L["down"], st.x, residual=st.x, pdl=pdl, norm_w=nw, norm_out=nout, eps=eps)
        n += 7 + merge_launch + (0 if tp is None else 1 if fuse_norm else 2)
        if taps is not None and li != last:
            for j, t in enumerate(tap_ids):
                if t == li:
                    X.gather_rows(st.x, None, taps, dst_col0=j * H, pdl=pdl)
                    n += 1
    if final_norm is not None:
        X.rmsnorm(st.x, final_norm[0], eps, out=final_norm[1], pdl=pdl)
        n += 1
    if prefetch is not None:
        prefetch.join()
    return n


class FastRound:
    """Graph-captured decode rounds for one engine (single sequence, greedy)."""

    @classmethod
    def get(cls, engine) -> "FastRound":
        if engine._fast is None:
            engine._fast = cls(engine)
        return engine._fast

    def __init__(self, engine):
        self.eng = engine
        self.cfg = engine.cfg
        self.device = torch.device(engine.device)
        X.load()
        m = engine.model
        self.embed_w, self.lm_head_w, self.final_norm = m.model.embed_tokens.weight, m.lm_head.weight, m.model.norm.weight
        self.tp = getattr(engine, "tp", None)
        self.ep = getattr(engine, "ep", None)
        if self.tp is not None and self.ep is not None:
            raise NotImplementedError("tensor parallelism and expert parallelism are separate plans here")
        world = self.tp.world if self.tp is not None else 1
        self.lcfg = local_dims(self.cfg, world)
        self.layers = kernel_layer_weights(m.model.layers, self.cfg, self.tp, self.ep)
        if self.tp is not None:
            from ..parallel.tp import shard_rows
            self.vocab_local = self.cfg.vocab_size // world
            self.lm_head_w = shard_rows(m.lm_head.weight, self.tp.rank, world)
        self.freq = X.inv_freq(self.cfg.head_dim, self.cfg.rope_theta, self.device)
        self.prefetcher = WeightPrefetcher(self.device) if _L2_PREFETCH else None
        self.graphs: dict = {}
        self.draft_cache: dict = {}
        self.launches_per_round = 0
        self.timing = False            # when set, each graph replay is bracketed by CUDA events
        self.last_device_ms = 0.0      # summed device time of the last call's rounds
        self.last_prefill_ms = 0.0     # device time of the last call's prompt phase (target prefill + head context)
        self._prefill_events: list = []
        self.last_rounds = 0
        self._tp_graph_key = None

    # ------------------------------------------------------------------ support matrix
    def supports_tree(self, drafter, algo_obj, block_size, tree_width, budget, extend_kwargs=None) -> bool:
        cfg = self.cfg
        if cfg.head_dim != 128 or budget > 256 or tree_width > 8 or block_size - 1 > 48:
            return False
        if extend_kwargs:
            # the gated extension stays on the graph path for a draft head that runs inside the round, in chain mode
            head, scripted, host = self._split_drafter(drafter)
            ext_budget = int(extend_kwargs.get("ext_budget", max(1, block_size - 1)))
            if (head is None or scripted is not None or host is not None or extend_kwargs.get("mode", "chain") != "chain"
                    or self.tp is not None or self.ep is not None or ext_budget < 1 or ext_budget > block_size - 1
                    or block_size - 1 + ext_budget > 48 or budget + ext_budget > 256
                    or getattr(head.head, "hidden_dim_adapter", None) is not None):
                return False
        return hasattr(algo_obj, "caps_from_topk")

    @staticmethod
    def _split_drafter(drafter):
        """``(head drafter | None, scripted host drafter | None, other host drafter | None)``.

        Drafter protocol of the graph path (no class checks): a drafter whose proposal needs nothing from the
        device sets ``host_scripted = True`` (and may offer ``propose_topk_at(context_len, depth, width)``); a
        wrapper that runs a real drafter for its cost and substitutes a scripted one's candidates exposes them as
        ``.real`` and ``.oracle``."""
        scripted = getattr(drafter, "oracle", None)
        if scripted is not None and hasattr(drafter, "real"):
            real = drafter.real if isinstance(drafter.real, DraftHeadTreeDrafter) else None
            return real, scripted, (None if real is not None else drafter.real)
        if getattr(drafter, "host_scripted", False):
            return None, drafter, None
        if isinstance(drafter, DraftHeadTreeDrafter):
            return drafter, None, None
        return None, None, drafter

    # ------------------------------------------------------------------ buffers + capture
    def _round(self, NB: int, D: int, K: int, budget: int, head: Optional[DraftHeadTreeDrafter], staged: bool,
               tap_ids, max_new: int, remote=None, temperature: float = 0.0, ext=None):
        pool = self.eng.pool
        tap_ids = list(tap_ids) if (tap_ids and (head is not None or remote is not None)) else None
        temperature = float(temperature) if temperature > 0.0 else 0.0
        ext = (int(ext[0]), float(ext[1])) if ext else None       # (extension budget, gap threshold)
        key = (NB, D, K, budget, id(head) if head is not None else 0, staged, tuple(tap_ids or ()), id(pool),
               id(remote) if remote is not None else 0, temperature, ext)
        if key in self.graphs:
            return self.graphs[key]
        if pool.resident():
            raise RuntimeError("a decode graph must be captured before any sequence is resident in the pool")
        cfg, dev = self.cfg, self.device
        H = cfg.hidden_size
        words = max(1, (NB + 31) // 32)
        Dn, Kn = max(1, D), max(1, K)
        r = {"NB": NB, "D": D, "K": K, "W": words, "budget": budget, "head": head, "staged": staged,
             "max_new": 1 << 30, "tap_ids": tap_ids, "remote": remote}
        r["state"] = _i32(8, dev)
        r["committed"] = _i32(pool.max_seq_len + 64, dev)
        for name in ("tokens", "parents", "depth", "positions", "slots", "greedy"):
            r[name] = _i32(NB, dev)
        r["mask"] = _i32(NB * words, dev).view(NB, words)
        r["topk_tok"] = _i32(Dn * Kn, dev).view(Dn, Kn)
        r["topk_lp"] = torch.zeros(Dn, Kn, dtype=torch.float32, device=dev)
        r["caps"] = _i32(Dn, dev, fill=K)
        # the algorithm's per-request caps plan (see CapScheduleAlgorithm.device_caps_plan): mode, two doubles and
        # three cap lists, evaluated on the device each round when the top-k comes from an in-graph head
        r["plan_i"], r["plan_t"] = _i32(1, dev), _i32(3 * Dn, dev, fill=K)
        r["plan_f"] = torch.zeros(2, dtype=torch.float64, device=dev)
        r["path_idx"] = _i32(64, dev)
        r["result"] = _i32(64, dev)
        r["result_host"] = torch.zeros(64, dtype=torch.int32).pin_memory()
        r["stage_tok"] = torch.zeros(Dn, Kn, dtype=torch.int32).pin_memory()
        r["stage_lp"] = torch.zeros(Dn, Kn, dtype=torch.float32).pin_memory()
        r["stage_caps"] = torch.full((Dn,), K, dtype=torch.int32).pin_memory()
        r["cu_q"] = torch.tensor([0, NB], dtype=torch.int32, device=dev)
        r["seq_rows"] = _i32(1, dev)
        eos = sorted(self.eng.eos_token_ids)
        r["eos"] = torch.tensor(eos or [-1], dtype=torch.int32, device=dev)
        r["n_eos"] = len(eos)
        r["stack"] = _Stack(self.lcfg, NB, dev, pool.max_seq_len)
        r["xn"] = torch.zeros(NB, H, dtype=torch.bfloat16, device=dev)
        nt = X.n_tiles(self.lm_head_w.shape[0])
        r["am_ws"] = {"val": torch.zeros(NB, nt, dtype=torch.float32, device=dev),
                      "idx": torch.zeros(NB, nt, dtype=torch.int32, device=dev)}
        r["am_val"] = torch.zeros(NB, dtype=torch.float32, device=dev)
        r["temperature"] = temperature
        r["ext"] = ext
        if ext is not None:
            # gated chain extension: the round is captured as three graphs (draft + build + gate | conditioned draft
            # pass + splice | verify + accept) with one extra host read of the gate between the first two
            r["gate"] = _i32(4, dev)
            r["gate_host"] = torch.zeros(4, dtype=torch.int32).pin_memory()
            r["ext_tok"] = _i32(max(1, Dn), dev)
            r["ext_val"] = torch.zeros(max(1, Dn), dtype=torch.float32, device=dev)
        if temperature > 0.0:
            # sampling keeps the round in the graph: the LM head writes fp32 logits for the NB nodes, one kernel
            # draws a token per node (inverse CDF, uniforms from the graph-registered generator), and acceptance
            # walks the tree against the SAMPLED tokens (reference: the graphed verify with the accept swapped,
            # jetspec/inference_engine/engine.py:1084-1109)
            r["logits"] = torch.zeros(NB, self.lm_head_w.shape[0], dtype=torch.float32, device=dev)
            r["uniform"] = torch.zeros(NB, dtype=torch.float32, device=dev)
            r["sampled"] = torch.zeros(NB, dtype=torch.int64, device=dev)
        r["taps"] = torch.zeros(NB, len(tap_ids) * H, dtype=torch.bfloat16, device=dev) if tap_ids else None
        if remote is not None:
            # the layer-epilogue copies write the tapped rows straight into the drafter GPU's buffer
            assert remote.nodes == NB and remote.tap_width == len(tap_ids) * H
            r["taps"] = remote.taps_on_drafter
        if head is not None:
            self._draft_buffers(r, head)
        # run every kernel once outside capture (module load, function attributes), then capture
        par = self.tp if self.tp is not None else self.ep      # whichever runs collectives inside the round
        if par is not None:
            par.begin_sequence()
        r["launches"] = self._launch_round(r, pdl=False, use_remote=False)   # no handshakes while warming up
        torch.cuda.synchronize()
        X.status_word(dev).zero_()
        if par is not None:
            par.begin_sequence(par._turn)     # cycle length that is safe across replays
            r["ring_mod"] = par.ring_mod
        if ext is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_round(r, pdl=_PDL)
            r["graph"] = g
        else:
            for part in ("a", "x", "b"):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._launch_round(r, pdl=_PDL, part=part)
                r["graph_" + part] = g
        pool.frozen = True
        self.graphs[key] = r
        self.launches_per_round = r["launches"]
        return r

    def _draft_buffers(self, r, head: DraftHeadTreeDrafter):
        dev = self.device
        hm = head.head
        hc = hm.config
        if hm.hidden_dim_adapter is not None:
            raise NotImplementedError("heads with a hidden_dim_adapter use the eager path")
        bs = head.block_size
        cap = self.eng.pool.max_seq_len + 2 * bs + 64
        dkey = (id(head), cap)
        if dkey not in self.draft_cache:
            layers = kernel_layer_weights(hm.layers)
            Hkv, Dh = hc.num_key_value_heads, hc.head_dim
            self.draft_cache[dkey] = {
                "layers": layers,
                "k": [torch.zeros(Hkv, cap, Dh, dtype=torch.bfloat16, device=dev) for _ in layers],
                "v": [torch.zeros(Hkv, cap, Dh, dtype=torch.bfloat16, device=dev) for _ in layers],
                "slot_map": torch.arange(cap, dtype=torch.int32, device=dev).view(1, cap), "cap": cap}
        d = dict(self.draft_cache[dkey])
        H, ntap, Dd, K = hc.hidden_size, len(head.target_layer_ids), bs - 1, max(1, r["K"])
        bf = dict(dtype=torch.bfloat16, device=dev)
        d["bs"] = bs
        d["block_ids"], d["block_pos"], d["ctx_pos"], d["n_new"] = _i32(bs, dev), _i32(bs, dev), _i32(bs, dev), _i32(1, dev)
        d["ctx_in"] = torch.zeros(bs, ntap * H, **bf)
        d["ctx_h"], d["ctx_n"], d["hn"] = torch.zeros(bs, H, **bf), torch.zeros(bs, H, **bf), torch.zeros(bs, H, **bf)
        d["kv"] = torch.zeros(bs, 2 * hc.num_key_value_heads * hc.head_dim, **bf)
        d["stack"] = _Stack(hc, bs, dev, d["cap"])
        d["cu_q"] = torch.tensor([0, bs], dtype=torch.int32, device=dev)
        d["seq_rows"] = _i32(1, dev)
        d["full_mask"] = torch.full((bs, max(1, (bs + 31) // 32)), -1, dtype=torch.int32, device=dev)
        nt = X.n_tiles(self._draft_lm_head(head).shape[0])
        d["tk_ws"] = {"val": torch.zeros(Dd, nt, 8, dtype=torch.float32, device=dev),
                      "idx": torch.zeros(Dd, nt, 8, dtype=torch.int32, device=dev),
                      "lse": torch.zeros(Dd, nt, 2, dtype=torch.float32, device=dev)}
        d["topk_tok"] = _i32(Dd * K, dev).view(Dd, K)
        d["topk_lp"] = torch.zeros(Dd, K, dtype=torch.float32, device=dev)
        d["freq"] = X.inv_freq(hc.head_dim, hc.rope_theta, dev)
        nt_full = X.n_tiles(head._fwd.lm_head_w.shape[0])
        d["ext_ws"] = {"val": torch.zeros(Dd, nt_full, dtype=torch.float32, device=dev),
                       "idx": torch.zeros(Dd, nt_full, dtype=torch.int32, device=dev)}
        r["draft"] = d

    @staticmethod
    def _stage_caps_plan(r, plan: dict, D: int, K: int) -> None:
        """Upload one request's caps plan (mode, parameters, up to three cap lists) for the in-graph caps kernel."""
        mode = {"static": 0, "sigmoid": 1, "gap_select": 2}[plan["mode"]]
        rows = {0: [plan.get("caps")], 1: [], 2: [plan.get("above"), plan.get("below"), plan.get("between")]}[mode]
        t = torch.full((3, max(1, D)), K, dtype=torch.int32)
        for i, row in enumerate(rows):
            t[i, :D] = torch.tensor([int(c) for c in row[:D]], dtype=torch.int32)
        ab = {0: (0.0, 0.0), 1: (plan.get("beta", 0.0), plan.get("g_0", 0.0)), 2: (plan.get("hi", 0.0), plan.get("lo", 0.0))}[mode]
        r["plan_i"].copy_(torch.tensor([mode], dtype=torch.int32))
        r["plan_f"].copy_(torch.tensor(ab, dtype=torch.float64))
        r["plan_t"].copy_(t.reshape(-1))

    def _draft_lm_head(self, head) -> torch.Tensor:
        """The vocabulary matrix the draft head scores against: the target's (its shard under tensor parallelism)."""
        w = head._fwd.lm_head_w
        if self.tp is None:
            return w
        if w.data_ptr() == self.eng.model.lm_head.weight.data_ptr():
            return self.lm_head_w
        key = ("draft_lm_head", id(head))
        if key not in self.draft_cache:
            from ..parallel.tp import shard_rows
            self.draft_cache[key] = shard_rows(w, self.tp.rank, self.tp.world)
        return self.draft_cache[key]

    def _launch_draft(self, r, pdl) -> int:
        head, d = r["head"], r["draft"]
        hm, hc = head.head, head.head.config
        lib, p, s = X.load(), X._p, X._stream
        bs, eps, Hkv = d["bs"], hc.rms_norm_eps, hc.num_key_value_heads
        X._check(lib.js_draft_prep(p(r["state"]), p(r["committed"]), int(hm.mask_token_id), bs, bs, bs,
                                   p(d["block_ids"]), p(d["block_pos"]), p(d["ctx_pos"]), p(d["n_new"]), int(pdl), s()),
                 "js_draft_prep")
        # context update: tap rows of the previously accepted path -> fc -> norm -> per-layer K/V
        X.gather_rows(r["taps"], r["path_idx"], d["ctx_in"], n_valid=d["n_new"], rows=bs, pdl=pdl)
        X.gemm(d["ctx_in"], hm.fc.weight, out=d["ctx_h"], pdl=pdl)
        X.rmsnorm(d["ctx_h"], hm.hidden_norm.weight, eps, out=d["ctx_n"], pdl=pdl)
        n = 4
        for li, L in enumerate(d["layers"]):
            X.gemm(d["ctx_n"], L["kv"], out=d["kv"], pdl=pdl)
            X.qkv_post(d["kv"], None, L["kn"], d["ctx_pos"], d["ctx_pos"], d["freq"], None, d["k"][li], d["v"][li],
                       0, Hkv, eps, n_valid=d["n_new"], pdl=pdl)
            n += 2
        # block forward over [anchor, mask, mask, ...]
        st = d["stack"]
        X.embed(d["block_ids"], head._fwd.embed_w, out=st.x, pdl=pdl)
        causal = hm.resolve_causal_head("auto")
        n += 1 + decoder_layers(hc, d["layers"], st, d["k"], d["v"], d["slot_map"], d["seq_rows"], d["cu_q"],
                                r["state"][ST_CTX:ST_CTX + 1], d["block_pos"], d["block_pos"],
                                None if causal else d["full_mask"], causal, d["freq"], pdl=pdl)
        X.rmsnorm(st.x, hm.norm.weight, eps, out=d["hn"], pdl=pdl)
        rows = d["hn"][:bs - 1] if head.draft_shift else d["hn"][1:bs]
        if r.get("no_topk"):                   # the caller wants the hidden rows only (dense-logits contract)
            return n + 1
        if self.tp is None:
            X.lm_head_topk_logprobs(rows, head._fwd.lm_head_w, max(1, r["K"]), ws=d["tk_ws"], pdl=pdl,
                                    out_tok=d["topk_tok"], out_lp=d["topk_lp"])
        else:   # vocabulary-parallel: each rank scores its shard, the per-row records are merged through peer memory
            self.tp.lm_head_topk_logprobs(rows, self._draft_lm_head(head), self.tp.rank * self.vocab_local,
                                          max(1, r["K"]), d["tk_ws"], d["topk_tok"], d["topk_lp"], pdl=pdl)
        return n + 3

    def _launch_round(self, r, pdl: bool, use_remote: bool = True, part: str = "all") -> int:
        """Launch the kernels of one round.  ``part``: ``"all"`` (one graph), or for rounds with the gated tree
        extension ``"a"`` (draft, caps, tree build, extension gate), ``"x"`` (path-conditioned draft pass + splice)
        and ``"b"`` (verify forward, acceptance, commit)."""
        lib, p, s = X.load(), X._p, X._stream
        pool, cfg = self.eng.pool, self.cfg
        NB, D, K = r["NB"], r["D"], r["K"]
        status = X.status_word(self.device)
        n = 0
        if part == "all" and r.get("ext") is not None:      # the warm-up run of an extension round: every part once
            return sum(self._launch_round(r, pdl, use_remote, q) for q in ("a", "x", "b"))
        if part == "x":
            return self._launch_extension(r, pdl)
        if part == "b":
            return self._launch_verify(r, pdl, use_remote)
        if r["head"] is not None and D > 0:
            n += self._launch_draft(r, pdl)
            if not r["staged"]:
                r["topk_tok"].copy_(r["draft"]["topk_tok"][:D])
                r["topk_lp"].copy_(r["draft"]["topk_lp"][:D])
                lib.js_caps_from_topk.restype = ctypes.c_int
                X._check(lib.js_caps_from_topk(p(r["topk_lp"]), D, max(1, K), p(r["plan_i"]), p(r["plan_f"]),
                                               p(r["plan_t"]), p(r["caps"]), int(pdl), s()), "js_caps_from_topk")
                n += 1
        remote = r.get("remote") if use_remote else None
        if remote is not None and D > 0:
            remote.target_wait_topk(pdl)
            r["topk_tok"].copy_(remote.topk_on_target[0])
            r["topk_lp"].copy_(remote.topk_on_target[1].view(torch.float32))
            n += 1
        if r["staged"] and D > 0:
            r["topk_tok"].copy_(r["stage_tok"], non_blocking=True)
            r["topk_lp"].copy_(r["stage_lp"], non_blocking=True)
            r["caps"].copy_(r["stage_caps"], non_blocking=True)
        X._check(lib.js_tree_build(p(r["topk_tok"]), p(r["topk_lp"]), p(r["caps"]), D, max(1, K), r["budget"], NB,
                                   r["W"], p(r["committed"]), p(r["state"]), p(pool.slot_map), p(r["seq_rows"]),
                                   pool.max_seq_len, p(r["tokens"]), p(r["parents"]), p(r["depth"]), p(r["positions"]),
                                   p(r["slots"]), p(r["mask"]), p(status), int(pdl), s()), "js_tree_build")
        if part == "a":
            ext_budget, gap = r["ext"]
            lib.js_tree_ext_gate.restype = ctypes.c_int
            X._check(lib.js_tree_ext_gate(p(r["tokens"]), p(r["parents"]), p(r["state"]), p(r["topk_tok"]), p(r["topk_lp"]),
                                          D, max(1, K), ctypes.c_float(gap), ext_budget, NB, p(r["gate"]), int(pdl), s()),
                     "js_tree_ext_gate")
            r["gate_host"].copy_(r["gate"], non_blocking=True)
            return n + 2
        return n + 1 + self._launch_verify(r, pdl, use_remote)

    def _launch_extension(self, r, pdl: bool) -> int:
        """The path-conditioned draft pass (the block reads [anchor, rank-1 chain tokens]) and the splice of its
        first ``ext`` argmax tokens as a chain below the leaf the gate found (reference: ``_maybe_extend_tree``,
        ``jetspec/inference_engine/engine.py:109-146``, chain mode of ``jetspec/tree/_core/extend.py:100-129``)."""
        lib, p, s = X.load(), X._p, X._stream
        head, d = r["head"], r["draft"]
        hm, hc = head.head, head.head.config
        bs, D, K, NB = d["bs"], r["D"], max(1, r["K"]), r["NB"]
        ext_budget = r["ext"][0]
        lib.js_draft_prep_fill.restype = ctypes.c_int
        X._check(lib.js_draft_prep_fill(p(r["state"]), p(r["committed"]), int(hm.mask_token_id), bs, bs, bs,
                                        p(d["block_ids"]), p(d["block_pos"]), p(d["ctx_pos"]), p(d["n_new"]),
                                        p(r["topk_tok"]), K, D, int(pdl), s()), "js_draft_prep_fill")
        st = d["stack"]
        X.embed(d["block_ids"], head._fwd.embed_w, out=st.x, pdl=pdl)
        causal = hm.resolve_causal_head("auto")
        n = 2 + decoder_layers(hc, d["layers"], st, d["k"], d["v"], d["slot_map"], d["seq_rows"], d["cu_q"],
                               r["state"][ST_CTX:ST_CTX + 1], d["block_pos"], d["block_pos"],
                               None if causal else d["full_mask"], causal, d["freq"], pdl=pdl)
        X.rmsnorm(st.x, hm.norm.weight, hc.rms_norm_eps, out=d["hn"], pdl=pdl)
        rows = d["hn"][:bs - 1] if head.draft_shift else d["hn"][1:bs]
        X.lm_head_argmax(rows[:ext_budget], head._fwd.lm_head_w, pdl=pdl, out_idx=r["ext_tok"][:ext_budget],
                         out_val=r["ext_val"][:ext_budget], ws=d["ext_ws"])
        lib.js_tree_ext_splice.restype = ctypes.c_int
        X._check(lib.js_tree_ext_splice(p(r["tokens"]), p(r["parents"]), p(r["depth"]), p(r["positions"]), p(r["mask"]),
                                        p(r["state"]), p(r["gate"]), p(r["ext_tok"]), ext_budget, NB, r["W"],
                                        p(X.status_word(self.device)), int(pdl), s()), "js_tree_ext_splice")
        return n + 4

    def _launch_verify(self, r, pdl: bool, use_remote: bool = True) -> int:
        """Verify forward over the round's tree, greedy (or sampled) tokens, acceptance and commit."""
        lib, p, s = X.load(), X._p, X._stream
        pool, cfg = self.eng.pool, self.cfg
        NB = r["NB"]
        status = X.status_word(self.device)
        remote = r.get("remote") if use_remote else None
        n = 0
        st = r["stack"]
        pf = self.prefetcher
        if pf is not None:
            pf.ahead(self.layers[0]["qkv"])       # the first projection's weights arrive during the tree build
        X.embed(r["tokens"], self.embed_w, out=st.x, pdl=pdl)
        n += 1 + decoder_layers(self.lcfg, self.layers, st, pool.k_pool, pool.v_pool, pool.slot_map, r["seq_rows"],
                                r["cu_q"], r["state"][ST_PAST:ST_PAST + 1], r["positions"], r["slots"], r["mask"],
                                False, self.freq, taps=r["taps"], tap_ids=r["tap_ids"], pdl=pdl, tp=self.tp,
                                prefetch=pf, then_prefetch=self.lm_head_w, final_norm=(self.final_norm, r["xn"]),
                                ep=self.ep)
        last = cfg.num_hidden_layers - 1
        if r["taps"] is not None:
            for j, t in enumerate(r["tap_ids"]):
                if t == last:
                    X.gather_rows(r["xn"], None, r["taps"], dst_col0=j * cfg.hidden_size, pdl=pdl)
                    n += 1
        if r.get("temperature", 0.0) > 0.0:
            X.gemm(r["xn"], self.lm_head_w, out=r["logits"], epi=X.EPI_STORE_F32, bn=128, split=1, pdl=pdl)
            r["uniform"].uniform_()
            lib.js_sample_temperature.restype = ctypes.c_int
            X._check(lib.js_sample_temperature(p(r["logits"]), 0, NB, r["logits"].shape[1], r["logits"].stride(0),
                                               ctypes.c_float(r["temperature"]), p(r["uniform"]), p(r["sampled"]), s()),
                     "js_sample_temperature")
            r["greedy"].copy_(r["sampled"])
            n += 1
        elif self.tp is None:
            X.lm_head_argmax(r["xn"], self.lm_head_w, ws=r["am_ws"], pdl=pdl, out_idx=r["greedy"], out_val=r["am_val"])
        else:
            self.tp.lm_head_argmax(r["xn"], self.lm_head_w, self.tp.rank * self.vocab_local, r["am_ws"], r["greedy"],
                                   r["am_val"], pdl=pdl)
        X._check(lib.js_tree_accept_commit(p(r["tokens"]), p(r["parents"]), p(r["depth"]), p(r["greedy"]), NB,
                                           p(r["state"]), p(pool.slot_map), p(r["seq_rows"]), pool.max_seq_len,
                                           p(r["committed"]), r["committed"].numel(), p(r["eos"]), r["n_eos"],
                                           r["max_new"], p(r["path_idx"]), p(r["result"]), p(status), int(pdl), s()),
                 "js_tree_accept_commit")
        if remote is not None:
            remote.target_push_header(r["state"], r["committed"], r["path_idx"], pdl)
            n += 4
        r["result_host"].copy_(r["result"], non_blocking=True)
        return n + 3

    # ------------------------------------------------------------------ batched verify (continuous batching)
    def supports_batch_verify(self, trees, tap_ids) -> bool:
        cfg = self.cfg
        if cfg.head_dim != 128 or not trees:
            return False
        return all(t.host is not None and t.num_nodes <= 256 for t in trees)

    def batch_verify(self, seq_ids, trees, past, nb: int, tap_ids=None):
        """The verify forward of ``B`` trees (one per live sequence) as ONE graph replay: embedding, the decoder
        stack on ``B x NB`` rows through the paged pool, final norm and the vocabulary argmax.  The host stages
        tokens, positions, ancestor bits, slot-map rows and committed lengths in one pinned buffer; one copy in, one
        copy out.  Returns ``(greedy, hidden)``: per sequence the target's argmax at every node (host lists) and,
        with ``tap_ids``, the tapped hidden rows ``(B*NB, taps*H)`` on the device (row ``b*NB + i`` = node ``i``).

        A graph is captured per ``(B, NB)``; the first call of a shape runs the kernels once eagerly with the real
        inputs (idempotent: the same KV rows are written again by the replay)."""
        import numpy as np
        from ..tree.ancestor import ancestor_bits_np
        pool, cfg, dev = self.eng.pool, self.cfg, self.device
        B = len(seq_ids)
        NB = int(nb)                      # the tree bucket the caller reserved KV room for
        if max(t.num_nodes for t in trees) > NB:
            raise ValueError("a tree is larger than the reserved bucket")
        W = max(1, (NB + 31) // 32)
        tap_ids = list(tap_ids) if tap_ids else None
        key = ("batch", B, NB, tuple(tap_ids or ()), id(pool))
        r = self.graphs.get(key)
        fresh = r is None
        if self.tp is not None and B * NB > self.tp.m_cap:
            raise RuntimeError(f"batched verify of {B} x {NB} rows exceeds the tensor-parallel buffers "
                               f"(m_cap={self.tp.m_cap}); construct TensorParallel with a larger m_cap")
        if fresh:
            H, T = cfg.hidden_size, B * NB
            n_in = T * (2 + W) + 2 * B
            r = {"B": B, "NB": NB, "W": W, "tap_ids": tap_ids}
            r["inp"] = _i32(n_in, dev)
            r["inp_host"] = torch.zeros(n_in, dtype=torch.int32).pin_memory()
            r["tokens"], r["positions"] = r["inp"][:T], r["inp"][T:2 * T]
            r["mask"] = r["inp"][2 * T:2 * T + T * W].view(T, W)
            r["seq_rows"] = r["inp"][2 * T + T * W:2 * T + T * W + B]
            r["past"] = r["inp"][2 * T + T * W + B:]
            r["slots"] = _i32(T, dev)
            r["cu_q"] = (torch.arange(B + 1, dtype=torch.int32, device=dev) * NB).contiguous()
            r["ar"] = torch.arange(NB, dtype=torch.long, device=dev)
            r["greedy"] = _i32(T, dev)
            r["greedy_host"] = torch.zeros(T, dtype=torch.int32).pin_memory()
            r["stack"] = _Stack(self.lcfg, T, dev, pool.max_seq_len)
            r["xn"] = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
            nt = X.n_tiles(self.lm_head_w.shape[0])
            r["am_ws"] = {"val": torch.zeros(T, nt, dtype=torch.float32, device=dev),
                          "idx": torch.zeros(T, nt, dtype=torch.int32, device=dev)}
            r["am_val"] = torch.zeros(T, dtype=torch.float32, device=dev)
            r["taps"] = torch.zeros(T, len(tap_ids) * H, dtype=torch.bfloat16, device=dev) if tap_ids else None
        NB, W, T = r["NB"], r["W"], B * r["NB"]
        h = r["inp_host"].numpy()
        tok, pos = h[:T].reshape(B, NB), h[T:2 * T].reshape(B, NB)
        bits = h[2 * T:2 * T + T * W].reshape(B, NB, W)
        rows, pst = h[2 * T + T * W:2 * T + T * W + B], h[2 * T + T * W + B:]
        pad_bits = np.zeros((NB, W), dtype=np.uint32)                   # a pad row sees only itself
        idx = np.arange(NB)
        pad_bits[idx, idx >> 5] = np.uint32(1) << (idx & 31).astype(np.uint32)
        pad_bits = pad_bits.view(np.int32)
        for b, (sid, t) in enumerate(zip(seq_ids, trees)):
            n = t.num_nodes
            t_tok, t_par, t_dep = t.host
            p0 = int(past[b])
            if p0 + NB > pool.max_seq_len:
                raise RuntimeError("tree window exceeds the sequence capacity of the pool")
            tok[b, :n] = t_tok
            tok[b, n:] = 0
            pos[b, :n] = np.asarray(t_dep, dtype=np.int32) + p0
            pos[b, n:] = p0 + max(t_dep)
            bits[b] = pad_bits
            bits[b, :n, :max(1, (n + 31) // 32)] = ancestor_bits_np(t_par, n, max(1, (n + 31) // 32)).view(np.int32)
            rows[b] = pool.state(sid).row
            pst[b] = p0
        r["inp"].copy_(r["inp_host"], non_blocking=True)
        if fresh:
            if self.tp is not None:
                self.tp.begin_sequence()
            self._launch_batch_verify(r, pdl=False)
            torch.cuda.synchronize()
            X.check_status(dev)
            if self.tp is not None:
                self.tp.begin_sequence(self.tp._turn)     # cycle length that is safe across replays
                r["ring_mod"] = self.tp.ring_mod
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_batch_verify(r, pdl=_PDL)
            r["graph"] = g
            pool.frozen = True
            self.graphs[key] = r
            self._tp_graph_key = None
        if self.tp is not None and getattr(self, "_tp_graph_key", None) != key:
            # the graph's collectives restart their buffer cycle: every rank must have left the previous sequence
            # of collectives (eager prefill, another graph) before the first replay of this one
            self.tp.begin_sequence()
            self.tp.ring_mod = r["ring_mod"]
            self._tp_graph_key = key
        r["graph"].replay()
        torch.cuda.current_stream().synchronize()
        g_all = r["greedy_host"].numpy().reshape(B, NB)
        greedy = [g_all[b, :t.num_nodes].tolist() for b, t in enumerate(trees)]
        return greedy, r["taps"]

    def _launch_batch_verify(self, r, pdl: bool) -> None:
        pool, cfg = self.eng.pool, self.cfg
        st = r["stack"]
        # KV slots of every sequence's tree window: slot_map[row_b, past_b + i]
        win = r["past"].long()[:, None] + r["ar"][None, :]
        r["slots"].copy_(pool.slot_map[r["seq_rows"].long()].gather(1, win).reshape(-1))
        X.embed(r["tokens"], self.embed_w, out=st.x, pdl=False)
        decoder_layers(self.lcfg, self.layers, st, pool.k_pool, pool.v_pool, pool.slot_map, r["seq_rows"], r["cu_q"],
                       r["past"], r["positions"], r["slots"], r["mask"], False, self.freq, taps=r["taps"],
                       tap_ids=r["tap_ids"], pdl=pdl, tp=self.tp, final_norm=(self.final_norm, r["xn"]))
        last = cfg.num_hidden_layers - 1
        if r["taps"] is not None:
            for j, t in enumerate(r["tap_ids"]):
                if t == last:
                    X.gather_rows(r["xn"], None, r["taps"], dst_col0=j * cfg.hidden_size, pdl=pdl)
        if self.tp is None:
            X.lm_head_argmax(r["xn"], self.lm_head_w, ws=r["am_ws"], pdl=pdl, out_idx=r["greedy"], out_val=r["am_val"])
        else:
            self.tp.lm_head_argmax(r["xn"], self.lm_head_w, self.tp.rank * self.vocab_local, r["am_ws"], r["greedy"],
                                   r["am_val"], pdl=pdl)
        r["greedy_host"].copy_(r["greedy"], non_blocking=True)

    # ------------------------------------------------------------------ sequence setup
    def _begin(self, r, sid: int, ids: torch.Tensor, taps, total: int, temperature: float = 0.0) -> int:
        """Prefill through the eager kernel path and initialise the round's device state."""
        eng, pool = self.eng, self.eng.pool
        T = ids.shape[1]
        remote = r.get("remote")
        if remote is not None:
            remote.reset()
        ev = None
        if self.timing:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if self._kernel_prefill_ok() and temperature <= 0.0:
            first, hidden = self._prefill_kernels(sid, ids, taps, total)
        else:     # the module path returns the last row's logits, which a sampled first token needs
            logits, hidden = eng._prefill(sid, ids[0], taps=taps, reserve=total - T)
            first = int(sample(logits[-1], temperature)) if temperature > 0.0 else int(logits[-1].float().argmax())
        r["seq_rows"].fill_(pool.state(sid).row)
        state = torch.zeros(8, dtype=torch.int32)
        state[ST_PAST], state[ST_GEN] = T, 1
        committed = torch.zeros(r["committed"].numel(), dtype=torch.int32)
        committed[:T] = ids[0].to(torch.int32).cpu()
        committed[T] = first
        r["committed"].copy_(committed)
        head = r["head"]
        if head is not None:
            state[ST_CTX] = self._draft_prompt_context(r, hidden)
        if ev is not None:
            ev[1].record()
            self._prefill_events.append(ev)
        r["state"].copy_(state)
        torch.cuda.synchronize()
        if remote is not None:
            import torch.distributed as dist
            hid = hidden.to(torch.bfloat16).contiguous()
            dist.send(torch.tensor([hid.shape[0], hid.shape[1]], dtype=torch.int64, device=self.device),
                      dst=remote.draft_rank, group=remote.group)
            dist.send(hid, dst=remote.draft_rank, group=remote.group)
            remote.target_push_raw_header(0, first, 0)
        par = self.tp if self.tp is not None else self.ep
        if par is not None:
            par.begin_sequence()          # the graph's collectives restart their buffer cycle here
            par.ring_mod = r.get("ring_mod", par.ring_mod)
        return first

    def _all_max(self, v: int) -> int:
        """Maximum of a host integer over the expert-parallel group."""
        import torch.distributed as dist
        t = torch.tensor([int(v)], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.ep.group)
        return int(t.item())

    def _all_done(self, mine_done: bool) -> bool:
        """True once every rank of the expert-parallel group has finished its own request."""
        import torch.distributed as dist
        t = torch.tensor([1 if mine_done else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.ep.group)
        return bool(int(t.item()))

    def _kernel_prefill_ok(self) -> bool:
        """The prompt runs through the same kernels as the rounds (fused QKV, in-kernel KV scatter, SwiGLU epilogue)
        whenever the layers are ones :func:`decoder_layers` covers; ``JETSPEC_EAGER_PREFILL=1`` keeps the module path."""
        return self.tp is not None or self.ep is not None or os.environ.get("JETSPEC_EAGER_PREFILL", "0") != "1"

    def _draft_prompt_context(self, r, hidden: torch.Tensor, start: int = 0) -> int:
        """Fill the draft head's context K/V for rows ``start ..`` of the tapped hidden states (the prompt), with
        the same kernels the in-graph context update uses (fc GEMM, RMSNorm, fused K|V GEMM, per-head norm + RoPE +
        scatter), in row chunks.  Returns the number of context rows."""
        d, hm = r["draft"], r["head"].head
        hc = hm.config
        n, Hkv, eps = hidden.shape[0], hc.num_key_value_heads, hc.rms_norm_eps
        hid = hidden.to(torch.bfloat16)
        for s0 in range(start, n, 512):
            rows = hid[s0:s0 + 512].contiguous()
            m = rows.shape[0]
            ctx = X.rmsnorm(X.gemm(rows, hm.fc.weight), hm.hidden_norm.weight, eps)
            pos = torch.arange(s0, s0 + m, dtype=torch.int32, device=self.device)
            for li, L in enumerate(d["layers"]):
                kv = X.gemm(ctx, L["kv"])
                X.qkv_post(kv, None, L["kn"], pos, pos, d["freq"], None, d["k"][li], d["v"][li], 0, Hkv, eps)
        return n

    def _prefill_kernels(self, sid: int, ids: torch.Tensor, taps, total: int):
        """Causal prefill on the kernel path in chunks (the tensor-parallel route: sharded weights,
        fused GEMM+all-reduce).  Returns ``(first greedy token, tapped hidden (T, taps*H) or None)``."""
        pool, dev, cfg = self.eng.pool, self.device, self.cfg
        T, H = ids.shape[1], cfg.hidden_size
        pool.reserve(sid, total)
        row = pool.state(sid).row
        chunk = 512 if self.tp is None else min(512, self.tp.m_cap)
        if self.ep is not None:
            chunk = min(chunk, self.ep.max_tokens)
        # Line the ranks up on the host before the first exchange of the request: graph capture and host-side set-up
        # take a different time on every rank (seconds apart with eight processes sharing the host), while the
        # kernels' waits on peers are bounded at about a second.  Under expert parallelism the same exchange tells
        # every rank how many prompt chunks the longest prompt has: it must be known BEFORE the chunks run, because
        # a rank with a shorter prompt has to keep serving the others' rows (`idle_layer`) right after its own.
        chunks_all = None
        if self.ep is not None:
            chunks_all = self._all_max((T + chunk - 1) // chunk)
        elif self.tp is not None:
            import torch.distributed as dist
            dist.barrier(group=self.tp.group)
        tap_ids = list(taps) if taps else None
        hidden = torch.empty(T, len(tap_ids) * H, dtype=torch.bfloat16, device=dev) if tap_ids else None
        seq_rows = torch.tensor([row], dtype=torch.int32, device=dev)
        ids32 = ids[0].to(device=dev, dtype=torch.int32)
        last = cfg.num_hidden_layers - 1
        xn = None
        for s0 in range(0, T, chunk):
            n = min(chunk, T - s0)
            st = _Stack(self.lcfg, n, dev, pool.max_seq_len)
            pos = torch.arange(s0, s0 + n, dtype=torch.int32, device=dev)
            slots = pool.slot_map[row, s0:s0 + n].contiguous()
            cu_q = torch.tensor([0, n], dtype=torch.int32, device=dev)
            past = torch.tensor([s0], dtype=torch.int32, device=dev)
            tapbuf = hidden[s0:s0 + n] if hidden is not None else None
            X.embed(ids32[s0:s0 + n].contiguous(), self.embed_w, out=st.x)
            xn = torch.empty_like(st.x)
            decoder_layers(self.lcfg, self.layers, st, pool.k_pool, pool.v_pool, pool.slot_map, seq_rows, cu_q, past,
                           pos, slots, None, True, self.freq, taps=tapbuf, tap_ids=tap_ids, pdl=False, tp=self.tp,
                           final_norm=(self.final_norm, xn), ep=self.ep)
            if tap_ids:
                for j, t in enumerate(tap_ids):
                    if t == last:
                        hidden[s0:s0 + n, j * H:(j + 1) * H] = xn
        if self.ep is not None:
            # every rank takes part in every expert-parallel layer call: ranks with shorter prompts sit the
            # remaining chunks out (their experts still serve the others' rows)
            mine = (T + chunk - 1) // chunk
            for _ in range(chunks_all - mine):
                for L in self.layers:
                    if L.get("moe_ep"):
                        gate_w, gu_l, dn_l, _, renorm = L["moe"]
                        self.ep.idle_layer(gate_w, gu_l, dn_l, renorm)
        h_last = xn[-1:].contiguous()
        out_idx = torch.empty(1, dtype=torch.int32, device=dev)
        nt = X.n_tiles(self.lm_head_w.shape[0])
        ws = {"val": torch.empty(1, nt, dtype=torch.float32, device=dev), "idx": torch.empty(1, nt, dtype=torch.int32, device=dev)}
        if self.tp is None:
            X.lm_head_argmax(h_last, self.lm_head_w, ws=ws, out_idx=out_idx)
        else:
            self.tp.lm_head_argmax(h_last, self.lm_head_w, self.tp.rank * self.vocab_local, ws, out_idx)
        pool.state(sid).length = T
        self._tp_graph_key = None          # eager collectives ran: a batched-verify graph must re-synchronise first
        return int(out_idx.item()), hidden

    # ------------------------------------------------------------------ public entry points
    @torch.inference_mode()
    def generate_tree(self, sid, committed, tree_drafter, algo_obj, block_size, tree_width, budget, taps, sp,
                      return_stats, tree_diag, max_depth, prompt_info, profile_table, total, extend_kwargs=None):
        from .engine import bucket_for_n
        eng = self.eng
        ext = None
        if extend_kwargs:
            ext = (int(extend_kwargs.get("ext_budget", max(1, block_size - 1))),
                   float(extend_kwargs.get("gap_threshold", 1.0)))
        D, K = max(1, block_size - 1), int(tree_width)
        NB = bucket_for_n(budget + (ext[0] if ext else 0))
        from .disagg import RemoteDraftHead
        remote = None
        if isinstance(tree_drafter, RemoteDraftHead):
            remote, head, oracle, host_drafter = tree_drafter.channel, None, tree_drafter.oracle, None
            taps = list(tree_drafter.target_layer_ids)
        else:
            head, oracle, host_drafter = self._split_drafter(tree_drafter)
        staged = oracle is not None or host_drafter is not None
        plan = None
        if head is not None and not staged:
            plan_fn = getattr(algo_obj, "device_caps_plan", None)
            plan = plan_fn(D, K, prompt_info=prompt_info, profile_table=profile_table) if plan_fn is not None else None
        if (host_drafter is not None and taps is not None) or (head is not None and not staged and plan is None):
            # a host drafter that conditions on hidden states, or an algorithm whose caps have no device form,
            # take the eager path
            return eng._generate_tree_eager(sid, committed, tree_drafter, algo_obj, algo_obj.name, None, block_size,
                                            tree_width, budget, taps, sp, return_stats, prompt_info, profile_table,
                                            tree_diag, max_depth, extend_kwargs, total)
        if head is not None:
            taps = list(head.target_layer_ids) if taps is None else taps
            if head.block_size != block_size:
                raise ValueError(f"draft head block_size {head.block_size} != block_size {block_size}")
        if ext is not None and D + ext[0] > max_depth:
            raise ValueError(f"tree depth {D + ext[0]} exceeds max_tree_depth {max_depth}; "
                             "raise max_tree_depth when extending trees")
        r = self._round(NB, D, K, budget, head, staged, taps, sp.max_new_tokens, remote=remote,
                        temperature=sp.temperature, ext=ext)
        if plan is not None:
            self._stage_caps_plan(r, plan, D, K)
        first = self._begin(r, sid, committed, taps if (head is not None or remote is not None) else None, total,
                            temperature=sp.temperature)
        new_ids = [first]
        ctx_ids = committed[0].tolist() + [first]
        accept_lengths, tree_sizes, rounds = [], [], 0
        depth_hist = [0] * (max_depth + 2) if tree_diag else None
        done = first in eng.eos_token_ids
        res = r["result_host"].numpy()
        stage_tok, stage_lp, stage_caps = r["stage_tok"].numpy(), r["stage_lp"].numpy(), r["stage_caps"].numpy()
        src = oracle if oracle is not None else host_drafter
        stream = torch.cuda.current_stream()
        events = []
        frozen = None                      # expert parallelism: device state a finished rank keeps replaying from
        final_len = None
        extended = 0
        while True:
            active = len(new_ids) < sp.max_new_tokens and not done
            if not active:
                if self.ep is None:
                    break
                # this rank's request is over but others' are not: keep taking part in every layer's exchange by
                # replaying the round from a fixed state (its own results are discarded, nothing advances)
                if frozen is None:
                    frozen, final_len = r["state"].clone(), int(res[4]) if rounds else None
                r["state"].copy_(frozen)
            if not active:
                pass
            elif staged and oracle is not None and hasattr(oracle, "propose_topk_at"):
                tok_l, lp_l = oracle.propose_topk_at(len(ctx_ids), D, K)      # the script needs the position only
                stage_tok[:] = np.asarray(tok_l, dtype=np.int32)
                stage_lp[:] = np.asarray(lp_l, dtype=np.float32)
                stage_caps[:] = np.asarray(algo_obj.caps_from_topk(lp_l, K, prompt_info=prompt_info,
                                                                   profile_table=profile_table), dtype=np.int32)
            elif staged:
                ctx_t = torch.tensor([ctx_ids], dtype=torch.long, device="cpu" if oracle is not None else eng.device)
                if hasattr(src, "propose_topk"):
                    tok, lp = src.propose_topk(ctx_t, D, K)
                    tok_l, lp_l = tok.tolist(), lp.tolist()
                else:
                    tok_l, lp_l = topk_rows(src.propose_logits(ctx_t, D), K)
                stage_tok[:] = np.asarray(tok_l, dtype=np.int32)
                stage_lp[:] = np.asarray(lp_l, dtype=np.float32)
                stage_caps[:] = np.asarray(algo_obj.caps_from_topk(lp_l, K, prompt_info=prompt_info,
                                                                   profile_table=profile_table), dtype=np.int32)
            if self.timing:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            if ext is None:
                r["graph"].replay()
            else:         # draft + build + gate, one host read, then (if the gate fired) the conditioned pass + splice
                r["graph_a"].replay()
                stream.synchronize()
                if int(r["gate_host"][0]) != 0:
                    r["graph_x"].replay()
                    extended += 1
                r["graph_b"].replay()
            if self.timing:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record(stream)
                events.append((e0, e1))
            stream.synchronize()
            if active:
                rounds += 1
                acc, n_nodes = int(res[0]), int(res[3])
                if int(res[6]) != 0:
                    X.check_status(self.device)
                block = res[8:8 + acc + 1].tolist()
                accept_lengths.append(acc + 1)
                tree_sizes.append(n_nodes)
                if depth_hist is not None:
                    for dpt in r["depth"][:n_nodes].tolist():
                        depth_hist[dpt] += 1
                for t in block:
                    new_ids.append(int(t))
                    ctx_ids.append(int(t))
                    if int(t) in eng.eos_token_ids:
                        done = True
                        break
                if final_len is None and (len(new_ids) >= sp.max_new_tokens or done):
                    final_len = int(res[4])
            if self.ep is not None and self._all_done(len(new_ids) >= sp.max_new_tokens or done):
                break
        if self.ep is not None:
            X.check_status(self.device)
        if rounds:
            eng.pool.state(sid).length = final_len if final_len is not None else int(res[4])
        if remote is not None:
            remote.target_push_raw_header(0, 0, 1)      # tell the drafter GPU this request is over
            torch.cuda.synchronize()
        self.last_rounds = rounds
        self.last_device_ms = float(sum(a.elapsed_time(b) for a, b in events)) if events else 0.0
        if self._prefill_events:
            torch.cuda.synchronize()
            self.last_prefill_ms = float(sum(a.elapsed_time(b) for a, b in self._prefill_events))
            self._prefill_events = []
        new_ids = new_ids[: sp.max_new_tokens]
        out = {"token_ids": new_ids, "text": decode_text(eng.tokenizer, new_ids),
               "tpf": (len(new_ids) / rounds if rounds else 0.0)}
        if return_stats:
            out.update(accept_lengths=accept_lengths, tree_sizes=tree_sizes, rounds=rounds)
            if ext is not None:
                out["extended_rounds"] = extended
        if depth_hist is not None:
            out["tree_nodes_per_depth"] = depth_hist
        return out

    @torch.inference_mode()
    def generate_ar(self, sid, ids, sp: SamplingParams):
        """Autoregressive decode = rounds with a one-node tree (budget 1, no drafter)."""
        eng = self.eng
        if sp.temperature > 0.0 or self.cfg.head_dim != 128:
            logits, _ = eng._prefill(sid, ids[0], reserve=sp.max_new_tokens + 1)
            out = [int(sample(logits[-1], sp.temperature))]
            while len(out) < sp.max_new_tokens and out[-1] not in eng.eos_token_ids:
                past = eng.pool.state(sid).length
                logits, _, _ = eng._forward([sid], [torch.tensor([out[-1]], device=eng.device)], [past])
                eng.pool.state(sid).length = past + 1
                out.append(int(sample(logits[-1], sp.temperature)))
            return {"token_ids": out, "text": decode_text(eng.tokenizer, out)}
        T = ids.shape[1]
        r = self._round(1, 0, 1, 1, None, False, None, sp.max_new_tokens)
        first = self._begin(r, sid, ids, None, T + sp.max_new_tokens + 2)
        out = [first]
        res = r["result_host"].numpy()
        stream = torch.cuda.current_stream()
        frozen = None
        while True:
            active = len(out) < sp.max_new_tokens and out[-1] not in eng.eos_token_ids
            if not active:
                if self.ep is None:
                    break
                if frozen is None:               # keep serving the other ranks' rows from a state that never advances
                    frozen = r["state"].clone()
                r["state"].copy_(frozen)
            r["graph"].replay()
            stream.synchronize()
            if active:
                if int(res[6]) != 0:
                    X.check_status(self.device)
                out.append(int(res[8]))
            if self.ep is not None and self._all_done(len(out) >= sp.max_new_tokens or out[-1] in eng.eos_token_ids):
                break
        return {"token_ids": out, "text": decode_text(eng.tokenizer, out)}
