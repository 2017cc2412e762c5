"""Qwen3 dense and Qwen3-MoE decoders, written directly on the framework's ops.

The module tree mirrors the Hugging Face parameter names
(``model.layers.N.self_attn.q_proj.weight`` … ``lm_head.weight``) so a stock
safetensors checkpoint loads without renaming; those are the module paths the
reference relies on (``jetspec/inference_engine/compiled_verify_stack.py:106-117``).
The forward pass is token-major (one row per token of a ragged batch) and takes an
*attention backend*: a callable that owns KV placement and masking.  The same
decoder therefore serves the contiguous-cache reference engine, the paged engine
and prefill.

MoE expert weights are held stacked, ``(E, 2I, H)`` and ``(E, H, I)``, which is
what the grouped GEMM consumes (reference stacks them the same way at patch time:
``jetspec/models/moe_fused.py:89-106``).
"""
from __future__ import annotations

import json
import os
from typing import Callable, Optional, Sequence

import torch
import torch.nn as nn

from .. import ops
from .config import Qwen3Config


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class Attention(nn.Module):
    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        H, D = cfg.hidden_size, cfg.head_dim
        b = cfg.attention_bias
        self.q_proj = nn.Linear(H, cfg.num_attention_heads * D, bias=b)
        self.k_proj = nn.Linear(H, cfg.num_key_value_heads * D, bias=b)
        self.v_proj = nn.Linear(H, cfg.num_key_value_heads * D, bias=b)
        self.o_proj = nn.Linear(cfg.num_attention_heads * D, H, bias=b)
        self.q_norm = RMSNorm(D, cfg.rms_norm_eps)
        self.k_norm = RMSNorm(D, cfg.rms_norm_eps)


class MLP(nn.Module):
    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        gu = torch.cat((ops.linear(x, self.gate_proj.weight), ops.linear(x, self.up_proj.weight)), dim=-1)
        return ops.linear(ops.silu_mul(gu), self.down_proj.weight)


class SparseMoE(nn.Module):
    """Top-k routed experts with stacked weights."""

    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.num_experts = E
        self.top_k = cfg.num_experts_per_tok
        self.norm_topk_prob = cfg.norm_topk_prob
        self.gate = nn.Linear(H, E, bias=False)
        self.w_gate_up = nn.Parameter(torch.empty(E, 2 * I, H))
        self.w_down = nn.Parameter(torch.empty(E, H, I))

    def forward(self, x, router_logits: Optional[torch.Tensor] = None):
        return ops.moe_forward(x, self.gate.weight, self.w_gate_up, self.w_down,
                               self.top_k, self.norm_topk_prob, router_logits)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config, layer_idx: int):
        super().__init__()
        self.self_attn = Attention(cfg)
        self.mlp = SparseMoE(cfg) if cfg.layer_is_moe(layer_idx) else MLP(cfg.hidden_size, cfg.intermediate_size)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class Qwen3Model(nn.Module):
    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList(DecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


AttnBackend = Callable[[int, torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


class Qwen3ForCausalLM(nn.Module):
    """Decoder-only LM.  ``forward`` is token-major and cache-agnostic."""

    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.config = cfg
        self.model = Qwen3Model(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    # -- construction ---------------------------------------------------------
    @classmethod
    def random_init(cls, cfg: Qwen3Config, seed: int = 0, dtype=torch.float32, device="cpu",
                    std: float = 0.02, init: str = "normal") -> "Qwen3ForCausalLM":
        """Synthetic weights.

        ``init="normal"``: every matrix N(0, std), norm scales 1.

        ``init="stable"``: a residual-dominant variant for benchmarks whose drafter is scripted
        from the target's own greedy continuation.  A deep N(0, 0.02) network has near-tied
        logits (top-1/top-2 gap of a few percent) that flip with the last bf16 bit, so its
        greedy continuation differs between any two kernels or KV layouts and no script
        survives.  Here the embedding is N(0, 1), the output projections (``o_proj``,
        ``down_proj``) are N(0, std / sqrt(2 L)) as in scaled-init schemes, and the LM head is
        the embedding table shifted by one row, so the greedy next token of ``t`` is ``t + 1``
        with a wide margin.  Shapes, dtypes and therefore all kernel work are unchanged.
        """
        with torch.device("meta"):
            m = cls(cfg)
        m = m.to_empty(device=device).to(dtype)
        g = torch.Generator(device="cpu").manual_seed(seed)
        out_scale = 1.0 / (2.0 * cfg.num_hidden_layers) ** 0.5
        with torch.no_grad():
            for name, p in m.named_parameters():
                if name.endswith("norm.weight") or "layernorm" in name:
                    p.fill_(1.0)
                elif init == "stable" and name.endswith("embed_tokens.weight"):
                    _fill_normal_(p, 1.0, g)
                elif init == "stable" and (name.endswith("o_proj.weight") or name.endswith("down_proj.weight")
                                           or name.endswith("w_down")):
                    _fill_normal_(p, std * out_scale, g)
                else:
                    _fill_normal_(p, std, g)
            if init == "stable":
                m.lm_head.weight.copy_(torch.roll(m.model.embed_tokens.weight, 1, dims=0))
        return m.eval()

    @classmethod
    def from_pretrained(cls, path: str, dtype=torch.bfloat16, device="cpu") -> "Qwen3ForCausalLM":
        from .loader import load_state_into
        cfg = Qwen3Config.from_pretrained(path)
        with torch.device("meta"):
            m = cls(cfg)
        m = m.to_empty(device=device).to(dtype)
        load_state_into(m, path, remap=_moe_key_remap(cfg))
        if cfg.tie_word_embeddings:
            m.lm_head.weight = m.model.embed_tokens.weight
        return m.eval()

    def save_pretrained(self, path: str) -> None:
        from .loader import save_state
        self.config.save_pretrained(path)
        sd = {}
        for k, v in self.state_dict().items():
            if k.endswith("mlp.w_gate_up"):
                base = k[: -len("w_gate_up")]
                I = v.shape[1] // 2
                for e in range(v.shape[0]):
                    sd[f"{base}experts.{e}.gate_proj.weight"] = v[e, :I]
                    sd[f"{base}experts.{e}.up_proj.weight"] = v[e, I:]
            elif k.endswith("mlp.w_down"):
                base = k[: -len("w_down")]
                for e in range(v.shape[0]):
                    sd[f"{base}experts.{e}.down_proj.weight"] = v[e]
            else:
                sd[k] = v
        if self.config.tie_word_embeddings:
            sd.pop("lm_head.weight", None)
        save_state(sd, path)

    # -- forward ----------------------------------------------------------------
    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, attn: AttnBackend,
                tap_layers: Optional[Sequence[int]] = None, logits_rows=None,
                router_logits_fn=None, return_hidden: bool = False):
        """Run the decoder on ``input_ids (T,)`` at ``positions (T,)``.

        ``attn(layer, q, k, v)`` receives post-norm, post-RoPE ``q (T,Hq,D)``,
        ``k, v (T,Hkv,D)`` and returns ``(T, Hq*D)``.  ``tap_layers`` selects the
        residual streams concatenated into the draft head's conditioning feature:
        the stream after layer L, except that the last layer is tapped after the
        final norm (reference: ``compiled_verify_stack.py:131-137,262-271``).
        ``logits_rows``: ``None`` → all rows, or an index tensor / slice of rows.
        Returns ``(logits, taps or None)`` (``hidden`` appended when requested).
        """
        cfg = self.config
        x = self.model.embed_tokens(input_ids)
        tap_ids = list(tap_layers) if tap_layers is not None else None
        tapped = {}
        last = cfg.num_hidden_layers - 1
        for li, layer in enumerate(self.model.layers):
            a = layer.self_attn
            h = layer.input_layernorm(x)
            qkv = torch.cat((ops.linear(h, a.q_proj.weight, a.q_proj.bias),
                             ops.linear(h, a.k_proj.weight, a.k_proj.bias),
                             ops.linear(h, a.v_proj.weight, a.v_proj.bias)), dim=-1)
            q, k, v = ops.qkv_postprocess(qkv, a.q_norm.weight, a.k_norm.weight, positions,
                                          cfg.num_attention_heads, cfg.num_key_value_heads,
                                          cfg.head_dim, cfg.rope_theta, cfg.rms_norm_eps)
            o = attn(li, q, k, v)
            x = x + ops.linear(o, a.o_proj.weight, a.o_proj.bias)
            h = layer.post_attention_layernorm(x)
            if isinstance(layer.mlp, SparseMoE):
                rl = router_logits_fn(li, h) if router_logits_fn is not None else None
                x = x + layer.mlp(h, rl)
            else:
                x = x + layer.mlp(h)
            if tap_ids is not None and li in tap_ids and li != last:
                tapped[li] = x
        xn = self.model.norm(x)
        if tap_ids is not None and last in tap_ids:
            tapped[last] = xn
        tap_cat = torch.cat([tapped[i] for i in tap_ids], dim=-1) if tap_ids else None
        rows = xn if logits_rows is None else xn[logits_rows]
        logits = ops.linear(rows, self.lm_head.weight)
        if return_hidden:
            return logits, tap_cat, xn
        return logits, tap_cat

    # -- fused views for the kernel path ---------------------------------------
    def fused_weights(self):
        """Per-layer ``[q|k|v]`` and ``[gate|up]`` weights concatenated along the
        output dim, built once (reference equivalent: ``_cat_linear_params``,
        ``compiled_verify_stack.py:59-75``)."""
        if getattr(self, "_fused", None) is None:
            fused = []
            for layer in self.model.layers:
                a = layer.self_attn
                d = {"qkv": torch.cat((a.q_proj.weight, a.k_proj.weight, a.v_proj.weight), 0).contiguous()}
                if isinstance(layer.mlp, MLP):
                    d["gate_up"] = torch.cat((layer.mlp.gate_proj.weight, layer.mlp.up_proj.weight), 0).contiguous()
                fused.append(d)
            self._fused = fused
        return self._fused


def _fill_normal_(p: torch.Tensor, std: float, g: torch.Generator, chunk: int = 1 << 24) -> None:
    """Seeded normal fill.  Small tensors are drawn on the host (identical on every device);
    tensors above 4M elements that live on a GPU are drawn there with a generator seeded from
    the host stream, which keeps multi-billion-parameter synthetic models quick to build."""
    flat = p.view(-1)
    n = flat.numel()
    if p.is_cuda and n > (1 << 22):
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=g))
        dg = torch.Generator(device=p.device).manual_seed(seed)
        for s in range(0, n, chunk):
            e = min(n, s + chunk)
            flat[s:e] = (torch.randn(e - s, generator=dg, dtype=torch.float32, device=p.device) * std).to(p.dtype)
        return
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        flat[s:e] = (torch.randn(e - s, generator=g, dtype=torch.float32) * std).to(p.dtype).to(p.device)


def _moe_key_remap(cfg: Qwen3Config):
    """Map per-expert checkpoint keys onto the stacked expert parameters."""
    if not cfg.is_moe:
        return None
    I = cfg.moe_intermediate_size

    def remap(key: str):
        # model.layers.N.mlp.experts.E.{gate,up,down}_proj.weight
        parts = key.split(".")
        if "experts" not in parts:
            return key, None
        i = parts.index("experts")
        base = ".".join(parts[:i])
        e = int(parts[i + 1])
        proj = parts[i + 2]
        if proj == "gate_proj":
            return base + ".w_gate_up", (e, slice(0, I))
        if proj == "up_proj":
            return base + ".w_gate_up", (e, slice(I, 2 * I))
        if proj == "down_proj":
            return base + ".w_down", (e,)
        return key, None

    return remap


def load_target(model_name_or_path, device="cuda", dtype=torch.bfloat16, attn_implementation: str = "auto",
                **_unused):
    """Load a target LM and its tokenizer from a local Hugging Face directory.

    Counterpart of the reference's ``load_target`` (``jetspec/models/qwen3.py:38-71``).
    ``attn_implementation`` is accepted for signature compatibility; attention is
    always this framework's own backend.  The tokenizer is ``None`` when the
    directory has no tokenizer files (token-id prompts still work).
    """
    model = Qwen3ForCausalLM.from_pretrained(model_name_or_path, dtype=dtype, device=device)
    return model, load_tokenizer(model_name_or_path)


def load_tokenizer(path: str):
    has_tok = any(os.path.exists(os.path.join(path, f))
                  for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json"))
    if not has_tok:
        return None
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(path)
