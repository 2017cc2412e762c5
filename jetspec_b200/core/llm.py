"""``LLM``: the reference decode engine (AR, chain-speculative, tree-speculative).

Contiguous KV cache, explicit masks, physical compaction of the accepted path.
Public surface follows ``jetspec/core/llm.py:115-613``: ``generate``,
``generate_chain``, ``generate_tree`` and the attributes ``model``, ``tokenizer``,
``runner``, ``device``, ``dtype``, ``eos_token_ids``.

Round invariant of the speculative loops: ``cache length == len(committed) - 1 ==
rows of target_hidden``.  The last committed token (the *anchor*) has no KV yet; it
enters the cache as node 0 of the next verify forward.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..models.qwen3 import Qwen3ForCausalLM, load_target
from ..sampling import SamplingParams, sample
from ..tree import build_ancestor_matrix, get_algorithm, gpu_tree_accept, tree_accept
from ..utils.timing import PhaseTimer
from .model_runner import ModelRunner


def resolve_eos(model, tokenizer) -> set:
    """Union of the tokenizer's and the model config's end-of-sequence ids."""
    ids = set()
    for src in (getattr(tokenizer, "eos_token_id", None), getattr(model.config, "eos_token_id", None)):
        if src is None:
            continue
        if isinstance(src, (list, tuple, set)):
            ids.update(int(x) for x in src)
        else:
            ids.add(int(src))
    return ids


def decode_text(tokenizer, ids) -> str:
    return tokenizer.decode(ids, skip_special_tokens=True) if tokenizer is not None else ""


class LLM:
    def __init__(self, model_name_or_path, device: str = "cuda", dtype: torch.dtype = torch.bfloat16,
                 attn_implementation: str = "sdpa", tokenizer=None):
        if isinstance(model_name_or_path, Qwen3ForCausalLM):
            self.model = model_name_or_path.to(device=device, dtype=dtype)
            self.tokenizer = tokenizer
        else:
            self.model, self.tokenizer = load_target(model_name_or_path, device=device, dtype=dtype)
            if tokenizer is not None:
                self.tokenizer = tokenizer
        self.device = device
        self.dtype = dtype
        self.runner = ModelRunner(self.model)
        self.eos_token_ids = resolve_eos(self.model, self.tokenizer)

    # -- helpers -------------------------------------------------------------------
    def _ids(self, prompt) -> torch.Tensor:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need a tokenizer; pass token ids (1, T) instead")
            return self.tokenizer(prompt, return_tensors="pt").input_ids.to(self.device)
        return torch.as_tensor(prompt).reshape(1, -1).to(self.device)

    def _now(self) -> float:
        if torch.device(self.device).type == "cuda":
            torch.cuda.synchronize()
        return time.perf_counter()

    @staticmethod
    def _pick(logits: torch.Tensor, temperature: float) -> int:
        row = logits.reshape(-1, logits.shape[-1])[-1]
        return int(sample(row, temperature))

    # -- autoregressive ---------------------------------------------------------
    @torch.inference_mode()
    def generate(self, prompt, sampling_params: SamplingParams = None) -> dict:
        """Plain decode.  Returns ``{"token_ids", "text", "decode_time"}``."""
        sp = sampling_params or SamplingParams()
        ids = self._ids(prompt)
        cache = self.runner.new_cache(ids.shape[1] + sp.max_new_tokens + 1)
        logits, cache, _ = self.runner.forward(ids, cache, last_position_logits_only=True)
        out = [self._pick(logits, sp.temperature)]
        t0 = self._now()
        while len(out) < sp.max_new_tokens and out[-1] not in self.eos_token_ids:
            step = torch.tensor([[out[-1]]], device=self.device)
            logits, cache, _ = self.runner.forward(step, cache, last_position_logits_only=True)
            out.append(self._pick(logits, sp.temperature))
        return {"token_ids": out, "text": decode_text(self.tokenizer, out), "decode_time": self._now() - t0}

    # -- chain speculation ---------------------------------------------------------
    @torch.inference_mode()
    def generate_chain(self, prompt, drafter, block_size: int = 4, target_layer_ids=None,
                       sampling_params: SamplingParams = None) -> dict:
        """Linear speculative decode: ``k = max(1, block_size-1)`` drafts per round, verified in one
        forward over ``[anchor | drafts]``; the longest greedy-equal prefix plus one correction is
        committed and the rejected drafts' KV cropped.  Returns ``{"token_ids","text","tpf"}``."""
        sp = sampling_params or SamplingParams()
        committed = self._ids(prompt)
        if hasattr(drafter, "reset_cache"):
            drafter.reset_cache()
        k = max(1, block_size - 1)
        taps = list(target_layer_ids) if (target_layer_ids is not None and block_size > 1) else None
        cache = self.runner.new_cache(committed.shape[1] + sp.max_new_tokens + k + 2)
        logits, cache, target_hidden = self.runner.forward(committed, cache, target_layer_ids=taps,
                                                           last_position_logits_only=True)
        first = self._pick(logits, sp.temperature)
        new_ids, rounds = [first], 0
        committed = torch.cat((committed, torch.tensor([[first]], device=self.device)), 1)
        if first in self.eos_token_ids:
            return {"token_ids": new_ids[: sp.max_new_tokens], "text": decode_text(self.tokenizer, new_ids), "tpf": 0.0}
        done = False
        while len(new_ids) < sp.max_new_tokens and not done:
            drafts = drafter.propose(committed, k, target_hidden=target_hidden).to(self.device).reshape(-1)[:k]
            step = torch.cat((committed[:, -1:], drafts.reshape(1, -1)), 1)
            past = cache.length
            logits, cache, hid = self.runner.forward(step, cache, target_layer_ids=taps)
            rounds += 1
            greedy = logits[0].argmax(-1)
            agree = (drafts == greedy[:k]).to(torch.int64)
            acc = int(torch.cumprod(agree, 0).sum())
            cache.crop(past + 1 + acc)
            if hid is not None:
                target_hidden = torch.cat((target_hidden, hid[:, : 1 + acc]), 1)
            block = torch.cat((drafts[:acc], greedy[acc].reshape(1)))
            committed = torch.cat((committed, block.reshape(1, -1)), 1)
            for t in block.tolist():
                new_ids.append(int(t))
                if int(t) in self.eos_token_ids:
                    done = True
                    break
        new_ids = new_ids[: sp.max_new_tokens]
        return {"token_ids": new_ids, "text": decode_text(self.tokenizer, new_ids),
                "tpf": (len(new_ids) / rounds if rounds else 0.0)}

    # -- tree speculation ----------------------------------------------------------
    @torch.inference_mode()
    def generate_tree(self, prompt, tree_drafter, block_size: int = 4, tree_width: int = 2, budget: int = 15,
                      algo: str = "accum_logp", algo_kwargs: Optional[dict] = None, target_layer_ids=None,
                      sampling_params: SamplingParams = None, return_stats: bool = False,
                      profile_phases: bool = False, prompt_info: Optional[dict] = None,
                      profile_table: Optional[dict] = None, tree_attn: str = "sdpa",
                      return_text: bool = True, on_round=None) -> dict:
        """Tree-speculative decode over a persistent cache.

        Per round: draft per-depth logits → build a tree of at most ``budget`` nodes →
        ONE target forward over all nodes under the ancestor mask, node ``i`` at rotary
        position ``past + depth[i]`` → accept the longest target-agreeing path plus a
        correction → compact the accepted nodes' KV behind the prefix.
        ``tree_attn``: ``"sdpa"`` (default) runs attention as the fp32 PyTorch formula, the in-repo oracle;
        ``"triton"`` / ``"kernel"`` run it on the tcgen05 tree-attention kernel when the device, dtype and geometry
        allow (see :meth:`ModelRunner.forward`), the counterpart of the reference's kernel switch for this path.
        ``on_round`` (not in the reference's signature) is called after every round with a dict of that round's
        ``committed`` ids and ``target_hidden`` as the drafter saw them, ``draft_logits``, ``tree``, the target's
        ``target_argmax`` per node, the accepted ``path``, ``accepted`` length and ``correction`` token: the hook the
        profiling collectors use instead of re-implementing the loop.
        Returns ``{"token_ids","tpf","decode_time",["text"],["accept_lengths","tree_sizes",
        "rounds",["phase_times"]]}``.
        """
        sp = sampling_params or SamplingParams()
        committed = self._ids(prompt)
        if hasattr(tree_drafter, "reset_cache"):
            tree_drafter.reset_cache()
        algo_obj = get_algorithm(algo, **(algo_kwargs or {}))
        D = block_size - 1
        taps = list(target_layer_ids) if target_layer_ids is not None else None
        timer = PhaseTimer(enabled=profile_phases)
        if tree_attn not in ("sdpa", "triton", "kernel"):
            raise ValueError(f"unknown tree_attn {tree_attn!r}; expected 'sdpa', 'triton' or 'kernel'")
        use_kernel = tree_attn != "sdpa"
        cache = self.runner.new_cache(committed.shape[1] + sp.max_new_tokens + budget + 2)
        logits, cache, target_hidden = self.runner.forward(committed, cache, target_layer_ids=taps,
                                                           last_position_logits_only=True, attn_kernel=use_kernel)
        first = self._pick(logits, sp.temperature)
        new_ids = [first]
        committed = torch.cat((committed, torch.tensor([[first]], device=self.device)), 1)
        accept_lengths, tree_sizes, rounds = [], [], 0
        done = first in self.eos_token_ids
        t0 = self._now()
        while len(new_ids) < sp.max_new_tokens and not done:
            with timer.phase("draft"):
                draft_logits = tree_drafter.propose_logits(committed, D, target_hidden=target_hidden)
            with timer.phase("tree_build"):
                tree = algo_obj.build(root_token=int(committed[0, -1]), draft_logits=draft_logits.to(self.device),
                                      block_size=block_size, tree_width=tree_width, budget=budget,
                                      device=self.device, profile_table=profile_table, prompt_info=prompt_info)
            past = cache.length
            with timer.phase("verify"):
                pos = (past + tree.depth).reshape(1, -1)
                logits, cache, hid = self.runner.forward(tree.token_ids.reshape(1, -1), cache, position_ids=pos,
                                                         target_layer_ids=taps, ancestor=build_ancestor_matrix(tree),
                                                         attn_kernel=use_kernel)
            rounds += 1
            with timer.phase("accept"):
                if sp.temperature <= 0.0:
                    path, acc, corr = gpu_tree_accept(tree.token_ids, logits[0].argmax(-1), tree.parent_indices,
                                                      tree.depth, max_depth=D)
                    path_l, corr = path.tolist(), int(corr)
                else:
                    path_l, acc, corr = tree_accept(tree, logits, sp.temperature)
            with timer.phase("kv_select"):
                cache.select(past, path_l)
            if on_round is not None:
                on_round({"committed": committed, "target_hidden": target_hidden, "draft_logits": draft_logits,
                          "tree": tree, "target_argmax": logits[0].argmax(-1), "path": list(path_l),
                          "accepted": int(acc), "correction": int(corr)})
            if hid is not None:
                target_hidden = torch.cat((target_hidden, hid[:, path_l]), 1)
            block = tree.token_ids[path_l[1:]].tolist() + [corr]
            committed = torch.cat((committed, torch.tensor([block], device=self.device)), 1)
            accept_lengths.append(acc + 1)
            tree_sizes.append(tree.num_nodes)
            for t in block:
                new_ids.append(int(t))
                if int(t) in self.eos_token_ids:
                    done = True
                    break
        new_ids = new_ids[: sp.max_new_tokens]
        out = {"token_ids": new_ids, "tpf": (len(new_ids) / rounds if rounds else 0.0),
               "decode_time": self._now() - t0}
        if return_text:
            out["text"] = decode_text(self.tokenizer, new_ids)
        if return_stats:
            out.update(accept_lengths=accept_lengths, tree_sizes=tree_sizes, rounds=rounds)
            if profile_phases:
                out["phase_times"] = timer.summary_ms_per_round(rounds)
        return out
