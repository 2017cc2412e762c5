"""safetensors checkpoint reading and writing (sharded or single-file).

Loads straight into the parameters of an already-constructed module, one tensor
at a time, so a 16 GB checkpoint never exists twice in host memory.  A ``remap``
callable can redirect a checkpoint key to ``(parameter_name, index)`` so that
per-expert MoE tensors land inside the stacked expert parameters.
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
                else:
                    if tuple(dst.shape) != tuple(src.shape):
                        raise ValueError(f"{key}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
                    dst.copy_(src.to(dst.dtype))
                seen.add(name)
    if strict:
        missing = [n for n, p in module.named_parameters() if n not in seen]
        # a tied lm_head is legitimately absent from the file
        missing = [n for n in missing if n != "lm_head.weight"]
        if missing:
            raise KeyError(f"parameters missing from checkpoint: {missing[:8]}{'…' if len(missing) > 8 else ''}")


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
