"""Model configuration read from a Hugging Face ``config.json``.

Only the fields the decoder actually uses are kept.  The draft head adds
``block_size``, ``num_target_layers`` and ``dflash_config`` on top of the Qwen3
fields (reference: ``jetspec/models/draft_head.py:317-337``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Optional


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: Optional[int] = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    sliding_window: Optional[int] = None
    layer_types: Optional[list] = None
    eos_token_id: Any = None
    # mixture-of-experts (Qwen3-MoE); num_experts == 0 means a dense model
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: list = field(default_factory=list)
    # draft-head extras
    block_size: Optional[int] = None
    num_target_layers: Optional[int] = None
    dflash_config: Optional[dict] = None
    model_type: str = "qwen3"

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.layer_types is None:
            self.layer_types = ["full_attention"] * self.num_hidden_layers

    # -- derived sizes ------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, layer_idx: int) -> bool:
        if not self.is_moe or layer_idx in self.mlp_only_layers:
            return False
        return (layer_idx + 1) % max(1, self.decoder_sparse_step) == 0

    # -- io -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        names = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in names}
        rope = d.get("rope_parameters") or {}
        if "rope_theta" not in kw and "rope_theta" in rope:
            kw["rope_theta"] = rope["rope_theta"]
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str, subfolder: str = "") -> "Qwen3Config":
        p = os.path.join(path, subfolder, "config.json") if subfolder else os.path.join(path, "config.json")
        with open(p) as f:
            d = json.load(f)
        cfg = cls.from_dict(d)
        gen = os.path.join(os.path.dirname(p), "generation_config.json")
        if os.path.exists(gen):
            with open(gen) as f:
                g = json.load(f)
            if g.get("eos_token_id") is not None:
                cfg.eos_token_id = _merge_eos(cfg.eos_token_id, g["eos_token_id"])
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = ["Qwen3MoeForCausalLM" if self.is_moe else "Qwen3ForCausalLM"]
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)


def _as_list(x) -> list:
    if x is None:
        return []
    if isinstance(x, (list, tuple)):
        return [int(v) for v in x]
    return [int(x)]


def _merge_eos(a, b) -> list:
    out = []
    for v in _as_list(a) + _as_list(b):
        if v not in out:
            out.append(v)
    return out


# Geometry presets used by the tests and the benchmarks (random-init weights).
def tiny_config(**over) -> Qwen3Config:
    """2 layers, hidden 256, 4 q / 2 kv heads, head_dim 64, SwiGLU 512, vocab 1024."""
    kw = dict(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6,
              rms_norm_eps=1e-6, max_position_embeddings=4096)
    kw.update(over)
    return Qwen3Config(**kw)


def qwen3_8b_config(**over) -> Qwen3Config:
    kw = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
              num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1e6)
    kw.update(over)
    return Qwen3Config(**kw)


def qwen3_30b_a3b_config(**over) -> Qwen3Config:
    kw = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=48,
              num_attention_heads=32, num_key_value_heads=4, head_dim=128, rope_theta=1e6,
              num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
              norm_topk_prob=True, model_type="qwen3_moe")
    kw.update(over)
    return Qwen3Config(**kw)


def draft_head_config(target: Qwen3Config, num_layers: int = 1, block_size: int = 16,
                      target_layer_ids: Optional[list] = None, mask_token_id: Optional[int] = None,
                      num_taps: int = 5, causal_head: bool = True) -> Qwen3Config:
    """Config of a causal-parallel draft head attached to ``target``."""
    from .draft_head import build_target_layer_ids
    ids = target_layer_ids or build_target_layer_ids(target.num_hidden_layers, num_taps)
    return Qwen3Config(
        vocab_size=target.vocab_size, hidden_size=target.hidden_size,
        intermediate_size=target.intermediate_size, num_hidden_layers=num_layers,
        num_attention_heads=target.num_attention_heads, num_key_value_heads=target.num_key_value_heads,
        head_dim=target.head_dim, rms_norm_eps=target.rms_norm_eps, rope_theta=target.rope_theta,
        block_size=block_size, num_target_layers=target.num_hidden_layers,
        dflash_config={"causal_head": causal_head, "target_layer_ids": list(ids),
                       "target_hidden_size": target.hidden_size,
                       "mask_token_id": target.vocab_size - 1 if mask_token_id is None else mask_token_id},
    )
