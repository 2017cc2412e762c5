"""Causal-parallel draft head.

A small decoder that predicts ``block_size - 1`` future tokens in ONE forward.
Its queries come from a block of *noise* embeddings ``[anchor, mask, mask, …]``;
its keys and values come from ``[ctx ; block]`` where ``ctx`` is the target
model's tapped hidden states pushed through ``fc`` + ``hidden_norm``.  The head
owns no embedding table and no LM head: it borrows the target's.

Behavioural reference: ``jetspec/models/draft_head.py:113-381`` (module layout,
parameter names, block-causal rule ``key_pos <= cached + ctx + q_idx``) and
``jetspec/draft_head_adapter.py:75-130`` (how a drafting step drives it).
Checkpoint keys are identical, so published heads load unchanged:
``layers.{i}.self_attn.{q,k,v,o}_proj.weight``, ``…{q,k}_norm.weight``,
``layers.{i}.mlp.{gate,up,down}_proj.weight``, the two layer norms,
``norm.weight``, ``fc.weight``, ``hidden_norm.weight`` and the optional
``hidden_dim_adapter.proj.weight``.

What differs from the reference is the execution model: the context K/V of every
layer is kept in a persistent per-sequence cache and only rows for newly
accepted tokens are projected each round, so a draft step costs O(new tokens),
not O(context).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from .config import Qwen3Config
from .qwen3 import RMSNorm, MLP, Attention, _fill_normal_


def build_target_layer_ids(num_target_layers: int, num_draft_layers: int) -> list[int]:
    """Evenly spaced tap layers between layer 1 and layer ``L-3``.

    Same rule as the reference (``jetspec/models/draft_head.py:41-50``).
    """
    if num_draft_layers == 1:
        return [num_target_layers // 2]
    start, end = 1, num_target_layers - 3
    span = end - start
    return [int(round(start + (i * span) / (num_draft_layers - 1))) for i in range(num_draft_layers)]


def extract_context_feature(hidden_states, layer_ids) -> torch.Tensor:
    """Concatenate ``hidden_states[L+1]`` for each tap layer (index 0 is the embedding output)."""
    return torch.cat([hidden_states[i + 1] for i in layer_ids], dim=-1)


class HiddenDimAdapter(nn.Module):
    """One shared projection applied to every tap slice when the head was trained
    against a target of a different hidden size."""

    def __init__(self, in_dim: int, out_dim: int):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.proj = nn.Linear(in_dim, out_dim, bias=False)

    def forward(self, x):
        lead, total = x.shape[:-1], x.shape[-1]
        L = total // self.in_dim
        return ops.linear(x.reshape(-1, self.in_dim), self.proj.weight).reshape(*lead, L * self.out_dim)


class DraftLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.self_attn = Attention(cfg)
        self.mlp = MLP(cfg.hidden_size, cfg.intermediate_size)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class DraftKVCache:
    """Per-sequence context K/V of every draft layer, grown geometrically."""

    def __init__(self, cfg: Qwen3Config, device, dtype, capacity: int = 1024):
        self.cfg = cfg
        self.device, self.dtype = device, dtype
        self.length = 0
        self.capacity = 0
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        self._grow(capacity)

    def _grow(self, cap: int) -> None:
        L, Hkv, D = self.cfg.num_hidden_layers, self.cfg.num_key_value_heads, self.cfg.head_dim
        nk = [torch.zeros(cap, Hkv, D, dtype=self.dtype, device=self.device) for _ in range(L)]
        nv = [torch.zeros(cap, Hkv, D, dtype=self.dtype, device=self.device) for _ in range(L)]
        for i in range(len(self.k)):
            nk[i][: self.length] = self.k[i][: self.length]
            nv[i][: self.length] = self.v[i][: self.length]
        self.k, self.v, self.capacity = nk, nv, cap

    def ensure(self, n: int) -> None:
        if n > self.capacity:
            self._grow(max(n, 2 * self.capacity))

    def reset(self) -> None:
        self.length = 0


class DraftHeadModel(nn.Module):
    """The draft head (``DFlashDraftModel`` in the reference)."""

    def __init__(self, cfg: Qwen3Config):
        super().__init__()
        self.config = cfg
        d = cfg.dflash_config or {}
        self.causal_head = bool(d.get("causal_head", False))
        self.layers = nn.ModuleList(DraftLayer(cfg) for _ in range(cfg.num_hidden_layers))
        self.target_layer_ids = list(d.get("target_layer_ids") or build_target_layer_ids(
            cfg.num_target_layers or cfg.num_hidden_layers, cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        th = d.get("target_hidden_size", cfg.hidden_size)
        self.hidden_dim_adapter = HiddenDimAdapter(th, cfg.hidden_size) if th != cfg.hidden_size else None
        self.fc = nn.Linear(len(self.target_layer_ids) * cfg.hidden_size, cfg.hidden_size, bias=False)
        self.hidden_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.block_size = cfg.block_size
        self.mask_token_id = d.get("mask_token_id", None)

    def resolve_causal_head(self, head_type: str = "auto") -> bool:
        if head_type == "auto":
            return bool(self.causal_head)
        if head_type == "bidirectional":
            return False
        if head_type == "causal":
            return True
        raise ValueError(f"Unsupported head_type={head_type!r}. Expected one of: auto, bidirectional, causal.")

    # -- construction ---------------------------------------------------------
    @classmethod
    def random_init(cls, cfg: Qwen3Config, seed: int = 1, dtype=torch.float32, device="cpu", std: float = 0.02):
        with torch.device("meta"):
            m = cls(cfg)
        m = m.to_empty(device=device).to(dtype)
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in m.named_parameters():
                if name.endswith("norm.weight") or "layernorm" in name:
                    p.fill_(1.0)
                else:
                    _fill_normal_(p, std, g)
        return m.eval()

    def save_pretrained(self, path: str) -> None:
        from .loader import save_state
        self.config.save_pretrained(path)
        save_state(dict(self.state_dict()), path)

    # -- forward ----------------------------------------------------------------
    def project_target_hidden(self, target_hidden: torch.Tensor) -> torch.Tensor:
        """``hidden_norm(fc(adapter(target_hidden)))`` on rows ``(n, taps*H)``."""
        x = target_hidden
        if self.hidden_dim_adapter is not None:
            x = self.hidden_dim_adapter(x)
        return self.hidden_norm(ops.linear(x, self.fc.weight))

    def new_cache(self, device=None, dtype=None, capacity: int = 1024) -> DraftKVCache:
        p = self.fc.weight
        return DraftKVCache(self.config, device or p.device, dtype or p.dtype, capacity)

    @torch.inference_mode()
    def append_context(self, cache: DraftKVCache, target_hidden_new: torch.Tensor) -> None:
        """Project rows for newly committed positions and append their K/V to ``cache``.

        Row ``i`` of ``target_hidden_new`` belongs to absolute position
        ``cache.length + i`` (the rotary position of that context key).
        """
        n = target_hidden_new.shape[0]
        if n == 0:
            return
        cfg = self.config
        cache.ensure(cache.length + n)
        ctx = self.project_target_hidden(target_hidden_new.to(self.fc.weight.dtype))
        pos = torch.arange(cache.length, cache.length + n, device=ctx.device)
        cos, sin = ref.rope_cos_sin(pos, cfg.head_dim, cfg.rope_theta)
        for li, layer in enumerate(self.layers):
            a = layer.self_attn
            k = ops.linear(ctx, a.k_proj.weight, a.k_proj.bias).view(n, cfg.num_key_value_heads, cfg.head_dim)
            v = ops.linear(ctx, a.v_proj.weight, a.v_proj.bias).view(n, cfg.num_key_value_heads, cfg.head_dim)
            k = ref.apply_rope(ref.rmsnorm(k, a.k_norm.weight, cfg.rms_norm_eps), cos, sin)
            cache.k[li][cache.length:cache.length + n] = k
            cache.v[li][cache.length:cache.length + n] = v
        cache.length += n

    @torch.inference_mode()
    def forward_block(self, noise_embedding: torch.Tensor, cache: DraftKVCache,
                      causal: Optional[bool] = None) -> torch.Tensor:
        """Run the block ``noise_embedding (bs, H)`` against the cached context.

        Block row ``i`` sits at rotary position ``cache.length + i``.  With a causal
        head, row ``i`` sees the whole context plus block rows ``<= i``; a
        bidirectional head sees the whole block.  Returns ``norm(hidden) (bs, H)``;
        the block's own K/V are not kept.
        """
        cfg = self.config
        causal = self.resolve_causal_head("auto") if causal is None else causal
        bs = noise_embedding.shape[0]
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        g = Hq // Hkv
        ctx_len = cache.length
        pos = torch.arange(ctx_len, ctx_len + bs, device=noise_embedding.device)
        cos, sin = ref.rope_cos_sin(pos, D, cfg.rope_theta)
        scale = 1.0 / math.sqrt(D)
        x = noise_embedding
        vis = torch.ones(bs, ctx_len + bs, dtype=torch.bool, device=x.device)
        if causal:
            vis[:, ctx_len:] = torch.tril(torch.ones(bs, bs, dtype=torch.bool, device=x.device))
        for li, layer in enumerate(self.layers):
            a = layer.self_attn
            h = layer.input_layernorm(x)
            q = ops.linear(h, a.q_proj.weight, a.q_proj.bias).view(bs, Hq, D)
            k = ops.linear(h, a.k_proj.weight, a.k_proj.bias).view(bs, Hkv, D)
            v = ops.linear(h, a.v_proj.weight, a.v_proj.bias).view(bs, Hkv, D)
            q = ref.apply_rope(ref.rmsnorm(q, a.q_norm.weight, cfg.rms_norm_eps), cos, sin)
            k = ref.apply_rope(ref.rmsnorm(k, a.k_norm.weight, cfg.rms_norm_eps), cos, sin)
            K = torch.cat((cache.k[li][:ctx_len], k), 0).float()  # (L, Hkv, D)
            V = torch.cat((cache.v[li][:ctx_len], v), 0).float()
            qf = q.float().view(bs, Hkv, g, D)
            s = torch.einsum("nhgd,lhd->hgnl", qf, K) * scale
            s = s.masked_fill(~vis[None, None], float("-inf"))
            p = torch.softmax(s, -1)
            o = torch.einsum("hgnl,lhd->nhgd", p, V).reshape(bs, Hq * D).to(x.dtype)
            x = x + ops.linear(o, a.o_proj.weight, a.o_proj.bias)
            x = x + layer.mlp(layer.post_attention_layernorm(x))
        return self.norm(x)


def load_draft_head(repo_or_path: str, device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                    attn_implementation: str = "sdpa") -> DraftHeadModel:
    """Load a trained draft head from a local directory.

    ``"path::subfolder"`` selects a sub-directory, as the reference does for
    multi-cell repos (``jetspec/models/draft_head.py:384-402``).
    ``attn_implementation`` is accepted for signature compatibility only.
    """
    import os
    from .loader import load_state_into
    repo, _, sub = repo_or_path.partition("::")
    path = os.path.join(repo, sub) if sub else repo
    cfg = Qwen3Config.from_pretrained(path)
    with torch.device("meta"):
        head = DraftHeadModel(cfg)
    head = head.to_empty(device=device).to(dtype)
    load_state_into(head, path, strict=True)
    return head.eval()
