"""Plain PyTorch implementations of every op the engine uses.

These run on any device and dtype and are the numerical oracle for the sm_100a
kernels (each kernel test compares against the function of the same name here,
evaluated in fp32).  They are also the only implementation used on CPU.

Shapes use T = number of token rows in the (ragged) batch, H = hidden size,
Hq/Hkv = query / key-value heads, D = head_dim, S = KV slots in the pool.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# norms, rotary, activations
# --------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Qwen3 RMSNorm over the last dim; fp32 math, result in ``x.dtype``."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def add_rmsnorm(residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """``residual += x`` then RMSNorm; returns ``(new_residual, normed)``."""
    r = (residual.float() + x.float()).to(residual.dtype)
    return r, rmsnorm(r, weight, eps)


def rope_inv_freq(head_dim: int, theta: float, device=None) -> torch.Tensor:
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    return 1.0 / (theta ** (idx / head_dim))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    """fp32 ``cos, sin`` of shape ``(T, D/2)`` for integer positions."""
    inv = rope_inv_freq(head_dim, theta, positions.device)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``x (T, heads, D)`` with ``cos/sin (T, D/2)``."""
    xf = x.float()
    half = xf.shape[-1] // 2
    x1, x2 = xf[..., :half], xf[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """SwiGLU on a fused ``[gate | up]`` row: ``silu(gate) * up``."""
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x (M, K) @ w (N, K)^T``; the weight layout of ``nn.Linear``."""
    return F.linear(x, w, bias)


def qkv_postprocess(qkv: torch.Tensor, q_norm_w: torch.Tensor, k_norm_w: torch.Tensor,
                    positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                    theta: float, eps: float):
    """Split a fused QKV row, per-head RMSNorm on q and k, then RoPE.

    Returns ``q (T, Hq, D)``, ``k (T, Hkv, D)``, ``v (T, Hkv, D)``.  The norm comes
    before the rotation, as in Qwen3 (reference: ``compiled_verify_stack.py:226-233``).
    """
    T = qkv.shape[0]
    qs, ks = num_q_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :qs].reshape(T, num_q_heads, head_dim)
    k = qkv[:, qs:qs + ks].reshape(T, num_kv_heads, head_dim)
    v = qkv[:, qs + ks:].reshape(T, num_kv_heads, head_dim)
    q = rmsnorm(q, q_norm_w, eps)
    k = rmsnorm(k, k_norm_w, eps)
    cos, sin = rope_cos_sin(positions, head_dim, theta)
    return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v.contiguous()


# --------------------------------------------------------------------------
# paged tree attention
# --------------------------------------------------------------------------
def pack_ancestor_bits(ancestor: torch.Tensor, words: int) -> torch.Tensor:
    """Pack a bool ``(n, n)`` ancestor matrix into ``(n, words)`` int32 bit rows.

    Bit ``j`` of row ``i`` is set when tree key ``j`` is visible to query ``i``.
    """
    n = ancestor.shape[0]
    out = torch.zeros(n, words, dtype=torch.int64, device=ancestor.device)
    a = ancestor.to(torch.int64)
    for w in range(min(words, (n + 31) // 32)):
        chunk = a[:, w * 32:(w + 1) * 32]
        sh = torch.arange(chunk.shape[1], device=a.device, dtype=torch.int64)
        out[:, w] = (chunk << sh).sum(-1)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def unpack_ancestor_bits(bits: torch.Tensor, n: int) -> torch.Tensor:
    """Inverse of :func:`pack_ancestor_bits` for the first ``n`` columns."""
    b = bits.to(torch.int64) & 0xFFFFFFFF
    cols = torch.arange(n, device=bits.device)
    return ((b[:, cols // 32] >> (cols % 32)) & 1).bool()


def paged_tree_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         slot_map: torch.Tensor, seq_rows: torch.Tensor, cu_q: torch.Tensor,
                         past_lens: torch.Tensor, mask_bits: Optional[torch.Tensor],
                         scale: float, causal: bool = False) -> torch.Tensor:
    """Ragged multi-sequence attention over a slot-addressed KV pool.

    ``q (T, Hq, D)`` holds the query rows of all sequences back to back;
    sequence ``b`` owns rows ``cu_q[b]:cu_q[b+1]`` (n_b rows).  Its keys are the
    logical positions ``0 .. past_lens[b]+n_b-1`` whose KV rows live at
    ``k_pool[:, slot_map[seq_rows[b], pos]]``.  Every position below
    ``past_lens[b]`` is visible to every query; position ``past_lens[b]+j`` is
    visible to query ``i`` when bit ``j`` of ``mask_bits[cu_q[b]+i]`` is set, or,
    with ``causal=True``, when ``j <= i``.  ``k_pool/v_pool`` are ``(Hkv, S, D)``.
    Softmax is evaluated in fp32.  Returns ``(T, Hq*D)`` in ``q.dtype``.
    """
    T, Hq, D = q.shape
    Hkv = k_pool.shape[0]
    g = Hq // Hkv
    out = torch.empty(T, Hq * D, dtype=q.dtype, device=q.device)
    cu = cu_q.tolist()
    pl = past_lens.tolist()
    rows = seq_rows.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        n = e - s
        if n == 0:
            continue
        past = pl[b]
        L = past + n
        slots = slot_map[rows[b], :L].long()
        k = k_pool[:, slots].float()  # (Hkv, L, D)
        v = v_pool[:, slots].float()
        qb = q[s:e].float().view(n, Hkv, g, D).permute(1, 2, 0, 3)  # (Hkv, g, n, D)
        scores = torch.einsum("hgnd,hld->hgnl", qb, k) * scale
        vis = torch.ones(n, L, dtype=torch.bool, device=q.device)
        if causal:
            vis[:, past:] = torch.tril(torch.ones(n, n, dtype=torch.bool, device=q.device))
        else:
            vis[:, past:] = unpack_ancestor_bits(mask_bits[s:e], n)
        scores = scores.masked_fill(~vis[None, None], float("-inf"))
        p = torch.softmax(scores, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)  # a fully masked row yields zeros
        o = torch.einsum("hgnl,hld->hgnd", p, v)  # (Hkv, g, n, D)
        out[s:e] = o.permute(2, 0, 1, 3).reshape(n, Hq * D).to(q.dtype)
    return out


def kv_scatter(k: torch.Tensor, v: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
               slots: torch.Tensor) -> None:
    """Write ``k, v (T, Hkv, D)`` into ``(Hkv, S, D)`` pools at ``slots (T,)``."""
    idx = slots.long()
    k_pool[:, idx] = k.transpose(0, 1).to(k_pool.dtype)
    v_pool[:, idx] = v.transpose(0, 1).to(v_pool.dtype)


# --------------------------------------------------------------------------
# vocabulary heads
# --------------------------------------------------------------------------
def lm_head_argmax(h: torch.Tensor, w: torch.Tensor):
    """Greedy token per row without keeping the logits: ``(argmax (T,), max (T,))``."""
    logits = F.linear(h, w).float()
    val, idx = logits.max(dim=-1)
    return idx, val


def lm_head_topk_logprobs(h: torch.Tensor, w: torch.Tensor, k: int):
    """Per-row top-``k`` tokens and their full-vocabulary log-probabilities.

    Equivalent to ``topk(log_softmax(h @ w^T), k)``: the normaliser is over the
    whole vocabulary, which the cumulative-logprob tree ordering relies on
    (reference: ``jetspec/tree/_core/topk_build.py:10-15``).
    """
    logits = F.linear(h, w).float()
    lp = torch.log_softmax(logits, dim=-1)
    vals, idx = torch.topk(lp, k, dim=-1)
    return idx, vals


# --------------------------------------------------------------------------
# mixture of experts
# --------------------------------------------------------------------------
def moe_route(router_logits: torch.Tensor, top_k: int, renorm: bool):
    """fp32 softmax over experts, top-k, optional renormalisation of the kept mass."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def moe_forward(x: torch.Tensor, gate_w: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                top_k: int, renorm: bool, router_logits: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sparse MoE block: route, run each expert's SwiGLU MLP on its tokens, combine.

    ``w_gate_up (E, 2I, H)`` and ``w_down (E, H, I)`` are the stacked expert weights
    in ``nn.Linear`` orientation.  Reference behaviour: ``jetspec/models/moe_fused.py:16-51``.
    """
    T, H = x.shape
    E = w_gate_up.shape[0]
    if router_logits is None:
        router_logits = F.linear(x, gate_w)
    wts, idx = moe_route(router_logits, top_k, renorm)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    flat_e = idx.reshape(-1)
    flat_t = torch.arange(T, device=x.device).repeat_interleave(top_k)
    flat_w = wts.reshape(-1)
    for e in range(E):
        sel = (flat_e == e).nonzero(as_tuple=True)[0]
        if sel.numel() == 0:
            continue
        tok = flat_t[sel]
        h = F.linear(x[tok], w_gate_up[e])
        h = silu_mul(h)
        y = F.linear(h, w_down[e]).float()
        out.index_add_(0, tok, y * flat_w[sel, None])
    return out.to(x.dtype)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperature: float = 0.0, generator=None) -> torch.Tensor:
    """argmax when ``temperature < 1e-5``, else a draw from ``softmax(logits / T)``.

    Reference: ``jetspec/core/sampler.py:10-17``.
    """
    if temperature < 1e-5:
        return logits.argmax(dim=-1)
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    flat = probs.reshape(-1, probs.shape[-1])
    return torch.multinomial(flat, 1, generator=generator).reshape(probs.shape[:-1])
