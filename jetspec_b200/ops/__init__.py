"""Op front-end: one function per op, routed to the sm_100a kernel or the reference.

Routing rule: a CUDA bf16 tensor goes to the hand-written kernel in the compiled
extension (and raises if the extension is not loadable — no silent fallback on a
GPU); CPU tensors, and non-bf16 CUDA tensors used by oracle tests, go to the plain
PyTorch implementation in :mod:`jetspec_b200.ops.reference`.  The reference's own seam of this kind is its
``torch.library`` op around the Triton kernel (``jetspec/inference_engine/paged_tree_attn_op.py:29-79``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import reference as ref
from .reference import (pack_ancestor_bits, unpack_ancestor_bits, rope_cos_sin, apply_rope,
                        moe_route)


def sample(logits, temperature: float = 0.0, generator=None):
    """argmax at temperature 0, else one draw per row from ``softmax(logits / T)``; CUDA tensors use the
    sampling kernel (the generator must then be a CUDA generator or None)."""
    if temperature >= 1e-5 and logits.is_cuda and (generator is None or generator.device.type == "cuda"):
        return _ext().sample_temperature(logits, temperature, generator)
    return ref.sample(logits, temperature, generator)


def _kern(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _ext():
    from . import cuda_ext
    return cuda_ext


def rmsnorm(x, weight, eps: float = 1e-6):
    if _kern(x) and x.shape[-1] % 8 == 0:
        return _ext().rmsnorm(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def add_rmsnorm(residual, x, weight, eps: float = 1e-6):
    return ref.add_rmsnorm(residual, x, weight, eps)


def linear(x, w, bias: Optional[torch.Tensor] = None):
    if not isinstance(w, torch.Tensor):            # an NVFP4Tensor: 4-bit weights, activations quantised per row
        from ..models.nvfp4 import nvfp4_linear_reference
        if _kern(x) and x.dim() == 2 and w.shape[1] % 256 == 0:
            return _ext().gemm_nvfp4(x.contiguous(), w.swizzled())
        return nvfp4_linear_reference(x, w).to(x.dtype)
    if _kern(x) and bias is None and x.dim() == 2 and w.dtype == torch.bfloat16:
        from . import cuda_ext
        if cuda_ext.gemm_supported(x.shape[0], w.shape[0], x.shape[1]):
            return cuda_ext.gemm(x, w)
    return ref.linear(x, w, bias)


def silu_mul(gate_up):
    if _kern(gate_up) and gate_up.dim() == 2 and gate_up.shape[-1] % 16 == 0:
        return _ext().silu_mul(gate_up)
    return ref.silu_mul(gate_up)


def qkv_postprocess(qkv, q_norm_w, k_norm_w, positions, num_q_heads, num_kv_heads, head_dim, theta, eps):
    if _kern(qkv) and head_dim == 128:
        ext = _ext()
        T = qkv.shape[0]
        q = torch.empty(T, num_q_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
        k = torch.empty(num_kv_heads, T, head_dim, dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
        rows = torch.arange(T, dtype=torch.int32, device=qkv.device)
        ext.qkv_post(qkv, q_norm_w, k_norm_w, positions.to(torch.int32), rows,
                     ext.inv_freq(head_dim, theta, qkv.device), q, k, v, num_q_heads, num_kv_heads, float(eps))
        return q, k.transpose(0, 1), v.transpose(0, 1)
    return ref.qkv_postprocess(qkv, q_norm_w, k_norm_w, positions, num_q_heads, num_kv_heads,
                               head_dim, theta, eps)


def kv_scatter(k, v, k_pool, v_pool, slots):
    return ref.kv_scatter(k, v, k_pool, v_pool, slots)


def paged_tree_attention(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens, mask_bits, scale,
                         causal: bool = False, max_q: Optional[int] = None):
    if _kern(q) and q.shape[-1] == 128:
        return _ext().paged_tree_attention(q.contiguous(), k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens,
                                           mask_bits, float(scale), bool(causal),
                                           int(max_q if max_q is not None else q.shape[0]))
    return ref.paged_tree_attention(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens,
                                    mask_bits, scale, causal)


def lm_head_argmax(h, w):
    if _kern(h):
        from . import cuda_ext
        return cuda_ext.lm_head_argmax(h, w)
    return ref.lm_head_argmax(h, w)


def lm_head_topk_logprobs(h, w, k: int):
    if _kern(h):
        from . import cuda_ext
        return cuda_ext.lm_head_topk_logprobs(h, w, k)
    return ref.lm_head_topk_logprobs(h, w, k)


def moe_forward(x, gate_w, w_gate_up, w_down, top_k, renorm, router_logits=None):
    if _kern(x):
        from . import cuda_ext
        return cuda_ext.moe_forward(x, gate_w, w_gate_up, w_down, top_k, renorm, router_logits)
    return ref.moe_forward(x, gate_w, w_gate_up, w_down, top_k, renorm, router_logits)


__all__ = [
    "rmsnorm", "add_rmsnorm", "linear", "silu_mul", "qkv_postprocess", "kv_scatter",
    "paged_tree_attention", "lm_head_argmax", "lm_head_topk_logprobs", "moe_forward",
    "pack_ancestor_bits", "unpack_ancestor_bits", "rope_cos_sin", "apply_rope", "moe_route", "sample",
]
