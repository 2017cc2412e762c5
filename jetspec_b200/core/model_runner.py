"""Single model-forward seam of the reference engine.

``ModelRunner.forward`` runs the decoder on a batch-1 token row against a
contiguous per-layer KV cache, optionally under a tree (ancestor) mask, and
returns logits plus the tapped hidden states the draft head conditions on.
Reference: ``jetspec/core/model_runner.py:90-154``.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


class DenseKVCache:
    """Contiguous ``(Hkv, capacity, D)`` K and V per layer with a shared length."""

    def __init__(self, cfg, device, dtype, capacity: int = 512):
        self.cfg, self.device, self.dtype = cfg, device, dtype
        self.length = 0
        self.capacity = 0
        self.k: list = []
        self.v: list = []
        self._grow(capacity)

    def _grow(self, cap: int) -> None:
        L, Hkv, D = self.cfg.num_hidden_layers, self.cfg.num_key_value_heads, self.cfg.head_dim
        nk = [torch.zeros(Hkv, cap, D, dtype=self.dtype, device=self.device) for _ in range(L)]
        nv = [torch.zeros(Hkv, cap, D, dtype=self.dtype, device=self.device) for _ in range(L)]
        for i in range(len(self.k)):
            nk[i][:, : self.length] = self.k[i][:, : self.length]
            nv[i][:, : self.length] = self.v[i][:, : self.length]
        self.k, self.v, self.capacity = nk, nv, cap

    def ensure(self, n: int) -> None:
        if n > self.capacity:
            self._grow(max(n, 2 * self.capacity))

    def get_seq_length(self) -> int:
        return self.length

    def crop(self, length: int) -> None:
        self.length = min(self.length, int(length))

    def select(self, past_len: int, keep_tree_indices) -> None:
        """Keep the first ``past_len`` positions, then move the tree positions
        ``past_len + keep_tree_indices[i]`` directly behind them (in that order).

        This is the physical compaction of the accepted path
        (reference: ``_select_kv_cache``, ``jetspec/core/llm.py:86-112``).
        """
        n = len(keep_tree_indices)
        if (n and n <= 64 and self.k[0].is_cuda and self.k[0].dtype == torch.bfloat16 and self.k[0].shape[-1] == 128
                and self.k[0].is_contiguous()):
            from ..ops import cuda_ext as X                   # compaction kernel (rows staged in shared memory)
            keep = torch.as_tensor(keep_tree_indices, dtype=torch.int32).to(self.device)
            for i in range(len(self.k)):
                X.kv_compact(self.k[i], self.v[i], past_len, keep)
            self.length = past_len + n
            return
        idx = torch.as_tensor(keep_tree_indices, dtype=torch.long, device=self.device) + past_len
        for i in range(len(self.k)):
            self.k[i][:, past_len:past_len + n] = self.k[i][:, idx]
            self.v[i][:, past_len:past_len + n] = self.v[i][:, idx]
        self.length = past_len + n


class ModelRunner:
    def __init__(self, model):
        self.model = model
        self.cfg = model.config

    def _kernel_attention_ok(self, ids: torch.Tensor, T: int, ancestor) -> bool:
        cfg = self.cfg
        w = self.model.lm_head.weight
        if not (ids.is_cuda and w.dtype == torch.bfloat16 and cfg.head_dim == 128):
            return False
        if cfg.sliding_window and any(t == "sliding_attention" for t in (cfg.layer_types or [])):
            return False
        return ancestor is None or T <= 256

    @staticmethod
    def _kernel_attention_args(cache, past: int, T: int, ancestor, device) -> dict:
        """The contiguous cache seen as a one-sequence paged pool: slot ``i`` is position ``i``."""
        i32 = dict(dtype=torch.int32, device=device)
        cap = cache.k[0].shape[1]
        out = {"slot_map": torch.arange(cap, **i32).view(1, cap), "seq_rows": torch.zeros(1, **i32),
               "cu_q": torch.tensor([0, T], **i32), "past": torch.tensor([past], **i32),
               "mask_bits": None, "causal": ancestor is None}
        if ancestor is not None:
            from ..tree.ancestor import pack_ancestor_bits
            out["mask_bits"] = pack_ancestor_bits(ancestor.to(device))
        return out

    def new_cache(self, capacity: int = 512) -> DenseKVCache:
        p = self.model.lm_head.weight
        return DenseKVCache(self.cfg, p.device, p.dtype, capacity)

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, past_key_values: Optional[DenseKVCache] = None,
                position_ids: Optional[torch.Tensor] = None, output_hidden_states: bool = False,
                target_layer_ids: Optional[Sequence[int]] = None, ancestor: Optional[torch.Tensor] = None,
                last_position_logits_only: bool = False, attn_kernel: bool = False):
        """Forward ``input_ids (1, T)``; new K/V are appended at ``cache.length``.

        ``ancestor (T, T) bool`` switches the new-token block from causal to tree
        masking: key ``j`` of the block is visible to query ``i`` iff
        ``ancestor[i, j]``; the cached prefix is always visible (sliding-window
        layers additionally hide keys further than the window behind the query).
        ``attn_kernel`` runs attention on the tcgen05 tree-attention kernel over the contiguous cache (the
        counterpart of the reference's dense tree-attention kernel for this path,
        ``jetspec/core/tree_attention_kernel.py:63-216``) instead of the fp32 PyTorch formula; it applies on a CUDA
        device with bf16 weights, ``head_dim`` 128, no sliding-window layers and at most 256 tree nodes, and is
        ignored otherwise.
        Returns ``(logits (1, T or 1, V), cache, target_hidden (1, T, taps*H) or None)``.
        """
        cfg = self.cfg
        ids = input_ids.reshape(-1)
        T = ids.numel()
        cache = past_key_values if past_key_values is not None else self.new_cache(max(512, 2 * T))
        past = cache.length
        cache.ensure(past + T)
        pos = (position_ids.reshape(-1) if position_ids is not None
               else torch.arange(past, past + T, device=ids.device))
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        g = Hq // Hkv
        scale = 1.0 / math.sqrt(D)
        vis = torch.ones(T, past + T, dtype=torch.bool, device=ids.device)
        vis[:, past:] = (ancestor.to(ids.device) if ancestor is not None
                         else torch.tril(torch.ones(T, T, dtype=torch.bool, device=ids.device)))
        key_pos = torch.cat((torch.arange(past, device=ids.device), pos))
        windows = {}
        use_kernel = bool(attn_kernel) and self._kernel_attention_ok(ids, T, ancestor)
        if use_kernel:
            kern = self._kernel_attention_args(cache, past, T, ancestor, ids.device)

        def attn(layer: int, q, k, v):
            cache.k[layer][:, past:past + T] = k.transpose(0, 1)
            cache.v[layer][:, past:past + T] = v.transpose(0, 1)
            if use_kernel:
                from ..ops import cuda_ext as X
                return X.paged_tree_attention(q.view(T, Hq, D).contiguous(), cache.k[layer], cache.v[layer],
                                              kern["slot_map"], kern["seq_rows"], kern["cu_q"], kern["past"],
                                              kern["mask_bits"], scale, kern["causal"], T, max_keys=past + T)
            K = cache.k[layer][:, :past + T].float()
            V = cache.v[layer][:, :past + T].float()
            qf = q.float().view(T, Hkv, g, D)
            s = torch.einsum("nhgd,hld->hgnl", qf, K) * scale
            m = vis
            if cfg.sliding_window and cfg.layer_types[layer] == "sliding_attention":
                if "w" not in windows:
                    windows["w"] = vis & ((pos[:, None] - key_pos[None, :]) < cfg.sliding_window)
                m = windows["w"]
            s = s.masked_fill(~m[None, None], float("-inf"))
            p = torch.softmax(s, -1)
            return torch.einsum("hgnl,hld->nhgd", p, V).reshape(T, Hq * D).to(q.dtype)

        taps = list(target_layer_ids) if (output_hidden_states or target_layer_ids is not None) and target_layer_ids else None
        rows = slice(T - 1, T) if last_position_logits_only else None
        logits, hidden = self.model(ids, pos, attn, tap_layers=taps, logits_rows=rows)
        cache.length = past + T
        return logits.unsqueeze(0), cache, (hidden.unsqueeze(0) if hidden is not None else None)
