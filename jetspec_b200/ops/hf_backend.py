"""Attention backend for Hugging Face models: plugs the paged tree attention into ``transformers``'
``AttentionInterface`` so a stock ``Qwen3ForCausalLM`` can verify token trees against this framework's KV pool.

Counterpart of the reference's ``jetspec/inference_engine/paged_attn_backend.py:27-92``.  A forward that wants the
paged kernel passes a :class:`PagedHandle` through the model's attention kwargs (``paged_handle=...``); the backend
scatters the new K/V rows into the slot-addressed pool and runs :func:`jetspec_b200.ops.paged_tree_attention`.
Without a handle the call falls back to PyTorch SDPA, so the same model object still serves plain dense forwards.

    from jetspec_b200.ops.hf_backend import register_hf_backend, PagedHandle
    register_hf_backend()                                   # once
    model = AutoModelForCausalLM.from_pretrained(path, attn_implementation="jetspec_paged_tree_attn")
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

BACKEND_NAME = "jetspec_paged_tree_attn"


@dataclass
class PagedHandle:
    """What one forward needs to address the pool: per-layer pools ``(L, Hkv, S, D)``, the slot map, the ragged
    batch description (see :func:`jetspec_b200.ops.reference.paged_tree_attention`) and where the new rows go."""
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    slot_map: torch.Tensor
    seq_rows: torch.Tensor
    cu_q: torch.Tensor
    past_lens: torch.Tensor
    new_slots: torch.Tensor                    # (T,) pool slot of every query token's own K/V row
    mask_bits: Optional[torch.Tensor] = None   # packed ancestor bits; None = causal inside the window
    causal: bool = True


def paged_tree_attention_forward(module, query, key, value, attention_mask, scaling=None, dropout=0.0, **kwargs):
    """``AttentionInterface`` entry: ``query (B, Hq, T, D)``, ``key/value (B, Hkv, T, D)`` -> ``(B, T, Hq, D), None``."""
    from . import kv_scatter, paged_tree_attention
    handle: Optional[PagedHandle] = kwargs.get("paged_handle")
    D = query.shape[-1]
    scale = float(scaling) if scaling is not None else D ** -0.5
    if handle is None:          # dense fallback
        g = query.shape[1] // key.shape[1]
        k, v = key.repeat_interleave(g, 1), value.repeat_interleave(g, 1)
        out = torch.nn.functional.scaled_dot_product_attention(query, k, v, attn_mask=attention_mask, scale=scale,
                                                               is_causal=attention_mask is None and query.shape[2] > 1)
        return out.transpose(1, 2).contiguous(), None
    if query.shape[0] != 1:
        raise ValueError("the paged path takes all sequences packed along the token axis (batch dimension 1)")
    li = int(getattr(module, "layer_idx", 0))
    q = query[0].transpose(0, 1).contiguous()                   # (T, Hq, D)
    k_new, v_new = key[0].transpose(0, 1), value[0].transpose(0, 1)
    kv_scatter(k_new, v_new, handle.k_pool[li], handle.v_pool[li], handle.new_slots)
    out = paged_tree_attention(q, handle.k_pool[li], handle.v_pool[li], handle.slot_map, handle.seq_rows, handle.cu_q,
                               handle.past_lens, handle.mask_bits, scale, handle.causal)
    return out.view(1, q.shape[0], q.shape[1], D), None


def register_hf_backend(name: str = BACKEND_NAME) -> str:
    """Register the backend with ``transformers`` (idempotent); returns the name to pass as ``attn_implementation``."""
    from transformers import AttentionInterface
    AttentionInterface.register(name, paged_tree_attention_forward)
    return name
