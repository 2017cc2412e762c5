"""safetensors checkpoint reading and writing (sharded or single-file).

Loads straight into the parameters of an already-constructed module, one tensor
at a time, so a 16 GB checkpoint never exists twice in host memory.  A ``remap``
callable can redirect a checkpoint key to ``(parameter_name, index)`` so that
per-expert MoE tensors land inside the stacked expert parameters.

The reference loads its target through Hugging Face ``from_pretrained`` (``jetspec/models/qwen3.py:38-71``) and
fuses experts afterwards (``jetspec/models/moe_fused.py:16-116``); here the same checkpoint files are read directly
into this framework's own modules, whose parameter names are the stock ones.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Optional

import torch


def _checkpoint_files(path: str) -> list[str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(path, x) for x in files]
    single = os.path.join(path, "model.safetensors")
    if os.path.exists(single):
        return [single]
    files = sorted(x for x in os.listdir(path) if x.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files under {path}")
    return [os.path.join(path, x) for x in files]


@torch.no_grad()
def load_state_into(module: torch.nn.Module, path: str, remap: Optional[Callable] = None,
                    strict: bool = True, prefix_strip: str = "") -> None:
    from safetensors import safe_open
    params = dict(module.named_parameters())
    params.update(dict(module.named_buffers()))
    seen = set()
    seen_slices: dict = {}       # stacked parameter -> set of indices a checkpoint tensor was copied into
    for fn in _checkpoint_files(path):
        with safe_open(fn, framework="pt", device="cpu") as f:
            for key in f.keys():
                name, index = (remap(key) if remap is not None else (key, None))
                if prefix_strip and name.startswith(prefix_strip):
                    name = name[len(prefix_strip):]
                if name not in params:
                    if strict and not key.endswith("rotary_emb.inv_freq"):
                        raise KeyError(f"checkpoint key {key!r} has no parameter {name!r}")
                    continue
                dst = params[name]
                src = f.get_tensor(key)
                if index is not None:
                    dst[index].copy_(src.to(dst.dtype))
                    seen_slices.setdefault(name, set()).add(_index_key(index))
                else:
                    if tuple(dst.shape) != tuple(src.shape):
                        raise ValueError(f"{key}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
                    dst.copy_(src.to(dst.dtype))
                seen.add(name)
    if strict:
        # a stacked parameter (per-expert tensors, gate|up halves) counts as loaded only when every slice of it
        # along the leading axes the remap addresses has been written; otherwise its untouched slices would keep
        # whatever the allocator left there
        for name, got in seen_slices.items():
            want = _expected_slices(params[name], got)
            if got != want:
                lost = sorted(want - got)[:4]
                raise KeyError(f"stacked parameter {name!r} is missing {len(want - got)} of {len(want)} slices "
                               f"(first: {lost})")
        missing = [n for n, p in module.named_parameters() if n not in seen]
        # a tied lm_head is legitimately absent from the file
        missing = [n for n in missing if n != "lm_head.weight"]
        if missing:
            raise KeyError(f"parameters missing from checkpoint: {missing[:8]}{'…' if len(missing) > 8 else ''}")


def _index_key(index) -> tuple:
    """A hashable form of the index a remap returned (ints and slices along the leading axes)."""
    if not isinstance(index, tuple):
        index = (index,)
    return tuple((i.start, i.stop) if isinstance(i, slice) else int(i) for i in index)


def _expected_slices(param, got: set) -> set:
    """Every index of the form seen in ``got`` that ``param`` has: the leading integer axis runs over its
    full extent, and a sliced second axis must be covered by the same set of ranges for every leading index."""
    lead = param.shape[0]
    tails = {k[1:] for k in got}
    ranges = sorted(t[0] for t in tails if t and isinstance(t[0], tuple))
    if ranges:      # the sliced second axis must be tiled completely (gate AND up halves)
        pos = 0
        for lo, hi in ranges:
            if lo > pos:
                tails.add(((pos, lo),))
            pos = max(pos, hi)
        if pos < param.shape[1]:
            tails.add(((pos, param.shape[1]),))
    return {(e,) + t for e in range(lead) for t in tails}


def save_state(state: dict, path: str, shard_bytes: int = 4 << 30) -> None:
    """Write ``state`` as one or more safetensors shards plus the index json."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    shards, cur, cur_b = [], {}, 0
    for k, v in state.items():
        t = v.detach().to("cpu").contiguous()
        nb = t.numel() * t.element_size()
        if cur and cur_b + nb > shard_bytes:
            shards.append(cur)
            cur, cur_b = {}, 0
        cur[k] = t
        cur_b += nb
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        save_file(shards[0], os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
        return
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
        for k in sh:
            weight_map[k] = fn
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
