"""``torch.library`` op boundary for the kernels a traced or exported program must see as opaque calls.

Counterpart of the reference's ``jetspec::paged_tree_attn`` custom op
(``jetspec/inference_engine/paged_tree_attn_op.py:28-79``): the op has a real implementation (the dispatcher of
:mod:`jetspec_b200.ops`: sm_100a kernel for CUDA bf16, PyTorch oracle otherwise) and a fake implementation that
only produces shapes, so ``torch.compile(fullgraph=True)`` / ``torch.export`` keep it as one node.  The engine's
own hot path does not go through here (it launches the kernels directly inside its CUDA graph); this is the seam
for users who embed the ops in their own compiled programs.

    import jetspec_b200.ops.library        # registers torch.ops.jetspec_b200.*
    out = torch.ops.jetspec_b200.paged_tree_attn(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past, bits, scale, False)
"""
from __future__ import annotations

from typing import Optional

import torch

NAMESPACE = "jetspec_b200"


@torch.library.custom_op(f"{NAMESPACE}::paged_tree_attn", mutates_args=())
def paged_tree_attn(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, slot_map: torch.Tensor,
                    seq_rows: torch.Tensor, cu_q: torch.Tensor, past_lens: torch.Tensor,
                    mask_bits: Optional[torch.Tensor], scale: float, causal: bool) -> torch.Tensor:
    from . import paged_tree_attention
    out = paged_tree_attention(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens, mask_bits, scale, causal)
    return out.reshape(q.shape[0], q.shape[1] * q.shape[2]).clone()


@paged_tree_attn.register_fake
def _(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens, mask_bits, scale, causal):
    return q.new_empty(q.shape[0], q.shape[1] * q.shape[2])


@torch.library.custom_op(f"{NAMESPACE}::linear_bf16", mutates_args=())
def linear_bf16(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x (M, K) @ w (N, K)^T`` on the tcgen05 GEMM for CUDA bf16 operands, ``F.linear`` otherwise."""
    from . import linear
    return linear(x, w).clone()


@linear_bf16.register_fake
def _(x, w):
    return x.new_empty(x.shape[0], w.shape[0])


@torch.library.custom_op(f"{NAMESPACE}::lm_head_argmax", mutates_args=())
def lm_head_argmax(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Greedy token per row of ``h (M, K)`` against the vocabulary matrix ``w (V, K)``; the logits are never stored."""
    from . import lm_head_argmax as impl
    out = impl(h, w)
    idx = out[0] if isinstance(out, tuple) else out
    return idx.to(torch.int64).clone()


@lm_head_argmax.register_fake
def _(h, w):
    return h.new_empty(h.shape[0], dtype=torch.int64)
