"""The bundled tree algorithms.

Every bundled algorithm is a *fan-out cap schedule*: it decides, per depth, how
many of the drafter's top-K candidates a node may spawn, and hands that to the
shared best-first builder.  They differ only in how the caps are chosen:

=====================  =========================================================
``accum_logp``         cap = K at every depth (the baseline)
``top2gap_fanout``     cap from the live top-1 / top-2 log-prob gap
``depth_rank_histogram`` cap from an offline per-(depth, rank) acceptance table
``task_router``        per-prompt class template (label or mean-gap fingerprint)
``reasoning_router``   chain for reasoning-like prompts, small fan-out otherwise
``class_histogram``    class template, or per-class offline histogram if given
=====================  =========================================================

Each recovers ``accum_logp`` bit-for-bit at its identity knob.  Reference counterparts:
``jetspec/tree/baselines/accum_logp.py:43-91`` (``AccumLogP``),
``jetspec/tree/tree_to_chain/fanout_cap/top2gap.py:36-114`` (``Top2GapFanout``, sigmoid cap ``:101``),
``jetspec/tree/profile_guided/depth_rank_histogram.py:39-107`` (``DepthRankHistogram``),
``jetspec/tree/semantic_aware/task_router.py:71-180`` (``PromptTaskClassifier``),
``jetspec/tree/semantic_aware/reasoning_router.py:64-185`` (``ReasoningModeDetector``),
``jetspec/tree/semantic_aware/class_histogram.py:66-224`` (``ClassifierPerClassHistogram``).
"""
from __future__ import annotations

import math
import re
from typing import Any, Optional

import torch

from .builder import build_with_per_depth_cap, topk_rows
from .registry import register_tree_algo
from .types import DraftTree, TreeAlgorithm


def _check_logits(draft_logits: torch.Tensor, block_size: int) -> int:
    D = block_size - 1
    if draft_logits.dim() != 3 or draft_logits.shape[0] != 1:
        raise ValueError(f"draft_logits must be (1, D, V); got {tuple(draft_logits.shape)}")
    if draft_logits.shape[1] != D:
        raise ValueError(f"draft_logits depth {draft_logits.shape[1]} != block_size-1 ({D})")
    return D


def _stretch(template, D: int, K: int) -> list:
    """Template → ``D`` caps; a missing tail is 1, every entry is clamped to ``[1, K]``."""
    return [max(1, min(int(template[d]) if d < len(template) else 1, K)) for d in range(D)]


def _mean_top2_gap(lps) -> Optional[float]:
    if not lps or len(lps[0]) < 2:
        return None
    return sum(r[0] - r[1] for r in lps) / len(lps)


class CapScheduleAlgorithm(TreeAlgorithm):
    """Shared ``build``: top-k extraction → ``caps_from_topk`` → best-first builder."""

    def _width(self, tree_width: int) -> int:
        return max(int(tree_width), 1)

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, **kwargs) -> list:
        raise NotImplementedError

    def device_caps_plan(self, D: int, K: int, prompt_info=None, profile_table=None) -> Optional[dict]:
        """How a round's caps follow from that round's per-depth top-k log-probs, in a form a device kernel can
        evaluate without the host (so an engine can keep drafting, tree building and verification in one graph):

        * ``{"mode": "static", "caps": [D ints]}`` - the caps do not depend on the log-probs;
        * ``{"mode": "sigmoid", "beta": b, "g_0": g}`` - ``max(1, round(K * sigmoid(-b (gap_d - g))))`` per depth;
        * ``{"mode": "gap_select", "hi": h, "lo": l, "above": [...], "below": [...], "between": [...]}`` - one of
          three cap lists by the mean top-1/top-2 gap ``g`` over the depths: ``g > hi``, ``g < lo``, otherwise.

        Everything that depends on ``prompt_info`` / ``profile_table`` is resolved here, once per request.
        :func:`eval_caps_plan` is the host evaluator (and the specification of the device kernel).  ``None`` means
        the algorithm has no such form and its caps are computed on the host every round."""
        return None

    def build(self, root_token, draft_logits, block_size, tree_width, budget, device,
              refresh_drafter_fn=None, profile_table=None, prompt_info=None, **kwargs) -> DraftTree:
        _check_logits(draft_logits, block_size)
        toks, lps = topk_rows(draft_logits, self._width(tree_width))
        caps = self.caps_from_topk(lps, tree_width, profile_table=profile_table, prompt_info=prompt_info)
        return build_with_per_depth_cap(int(root_token), toks, lps, caps, int(budget), device)


@register_tree_algo("accum_logp")
class AccumLogP(CapScheduleAlgorithm):
    """Full fan-out everywhere; expansion order by cumulative log-probability."""

    def _width(self, tree_width):
        return int(tree_width)

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, **kwargs):
        K = len(topk_logprobs_cpu[0]) if topk_logprobs_cpu else max(tree_width, 1)
        return [K] * len(topk_logprobs_cpu)

    def device_caps_plan(self, D, K, prompt_info=None, profile_table=None):
        return {"mode": "static", "caps": [int(K)] * int(D)}


def eval_caps_plan(plan: dict, topk_logprobs, K: int) -> list:
    """Evaluate a :meth:`CapScheduleAlgorithm.device_caps_plan` on one round's ``(D, K)`` log-probs (host lists).
    Equal to the algorithm's own ``caps_from_topk`` for the request the plan was made for."""
    D = len(topk_logprobs)
    if plan["mode"] == "static":
        return [int(c) for c in plan["caps"][:D]]
    if plan["mode"] == "sigmoid":
        return [sigmoid_cap(r[0] - r[1], K, plan["beta"], plan["g_0"]) for r in topk_logprobs]
    g = _mean_top2_gap(topk_logprobs)
    pick = "above" if g > plan["hi"] else "below" if g < plan["lo"] else "between"
    return [int(c) for c in plan[pick][:D]]


def _flat_lps(D: int, K: int) -> list:
    return [[0.0] * int(K) for _ in range(int(D))]


def sigmoid_cap(gap: float, K: int, beta: float, g_0: float) -> int:
    """``max(1, round(K * sigmoid(-beta * (gap - g_0))))`` with Python's round-half-even."""
    z = -beta * (gap - g_0)
    s = 1.0 / (1.0 + math.exp(-z)) if z >= 0 else math.exp(z) / (1.0 + math.exp(z))
    return max(1, int(round(K * s)))


@register_tree_algo("top2gap_fanout")
class Top2GapFanout(CapScheduleAlgorithm):
    """A decisive drafter (large top-1/top-2 gap) gets a chain, an undecided one fans out."""

    def __init__(self, beta: float = 1.0, g_0: float = 1.0):
        self.beta, self.g_0 = float(beta), float(g_0)

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, **kwargs):
        K = len(topk_logprobs_cpu[0]) if topk_logprobs_cpu else 0
        if K < 2:
            return [1] * len(topk_logprobs_cpu)
        return [sigmoid_cap(r[0] - r[1], K, self.beta, self.g_0) for r in topk_logprobs_cpu]

    def device_caps_plan(self, D, K, prompt_info=None, profile_table=None):
        if K < 2:
            return {"mode": "static", "caps": [1] * int(D)}
        return {"mode": "sigmoid", "beta": self.beta, "g_0": self.g_0}


@register_tree_algo("depth_rank_histogram")
class DepthRankHistogram(CapScheduleAlgorithm):
    """cap[d] = number of ranks whose profiled acceptance at depth ``d`` reaches ``tau``.

    ``profile_table = {"depth_rank_accept": [[…K floats…] × D], "meta": {...}}``.
    No table, or ``tau <= 0``, gives full fan-out.
    """

    def __init__(self, tau: float = 0.02):
        self.tau = float(tau)

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, profile_table=None, **kwargs):
        D = len(topk_logprobs_cpu)
        K = len(topk_logprobs_cpu[0]) if topk_logprobs_cpu else max(tree_width, 1)
        rows = profile_table.get("depth_rank_accept") if (profile_table is not None and self.tau > 0.0) else None
        if not rows:
            return [K] * D
        caps = []
        for d in range(D):
            row = rows[d] if d < len(rows) else None
            if not row:
                caps.append(K)
                continue
            keep = sum(1 for r in range(min(K, len(row))) if row[r] >= self.tau)
            caps.append(min(K, max(1, keep)))
        return caps

    def device_caps_plan(self, D, K, prompt_info=None, profile_table=None):
        return {"mode": "static", "caps": self.caps_from_topk(_flat_lps(D, K), K, profile_table=profile_table)}


CLASS_TEMPLATES = {
    "decisive_task": [1] * 15,
    "balanced_task": [3, 2] + [1] * 13,
    "uncertain_task": [7, 7] + [1] * 13,
}
TASK_ALIASES = {
    "math": "decisive_task", "code": "decisive_task", "decisive_task": "decisive_task",
    "balanced": "balanced_task", "balanced_task": "balanced_task",
    "chat": "uncertain_task", "open_ended": "uncertain_task", "uncertain_task": "uncertain_task",
}


def resolve_task_class(prompt_info: Optional[dict], lps, gap_high: float, gap_low: float) -> str:
    """Caller label if present (unknown labels → balanced), else the mean top-2 gap fingerprint."""
    if prompt_info is not None:
        label = prompt_info.get("task")
        if isinstance(label, str):
            return TASK_ALIASES.get(label, "balanced_task")
    g = _mean_top2_gap(lps)
    if g is None:
        return "balanced_task"
    if g > gap_high:
        return "decisive_task"
    if g < gap_low:
        return "uncertain_task"
    return "balanced_task"


class _RouterBase(CapScheduleAlgorithm):
    def __init__(self, gap_high: float = 2.0, gap_low: float = 1.0, templates: Optional[dict] = None,
                 force_baseline: bool = False):
        if gap_high < gap_low:
            raise ValueError(f"gap_high ({gap_high}) must be >= gap_low ({gap_low})")
        self.gap_high, self.gap_low = float(gap_high), float(gap_low)
        self.templates = {k: list(v) for k, v in (templates or CLASS_TEMPLATES).items()}
        self.force_baseline = bool(force_baseline)

    def device_caps_plan(self, D, K, prompt_info=None, profile_table=None):
        """A caller label (or the baseline switch) fixes the caps for the request; otherwise the class follows the
        mean-gap fingerprint of each round: three cap lists, one per class, made with the class as the label."""
        flat = _flat_lps(D, K)
        labelled = prompt_info is not None and isinstance(prompt_info.get("task"), str)
        if self.force_baseline or labelled or K < 2:
            return {"mode": "static", "caps": self.caps_from_topk(flat, K, prompt_info=prompt_info,
                                                                  profile_table=profile_table)}
        by = lambda cls: self.caps_from_topk(flat, K, prompt_info={"task": cls}, profile_table=profile_table)
        return {"mode": "gap_select", "hi": self.gap_high, "lo": self.gap_low, "above": by("decisive_task"),
                "below": by("uncertain_task"), "between": by("balanced_task")}


@register_tree_algo("task_router")
class TaskRouter(_RouterBase):
    """One hand-tuned fan-out template per prompt class."""

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, prompt_info=None, **kwargs):
        D, K = len(topk_logprobs_cpu), max(int(tree_width), 1)
        if self.force_baseline:
            return [K] * D
        task = resolve_task_class(prompt_info, topk_logprobs_cpu, self.gap_high, self.gap_low)
        return _stretch(self.templates.get(task) or self.templates.get("balanced_task") or [], D, K)


@register_tree_algo("class_histogram")
class ClassHistogram(_RouterBase):
    """Like ``task_router`` but prefers ``profile_table["per_class_histograms"][task]``:
    a flat list of caps, or a ``(D, K)`` acceptance matrix whose cap is the largest
    rank with positive support."""

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, prompt_info=None, profile_table=None, **kwargs):
        D, K = len(topk_logprobs_cpu), max(int(tree_width), 1)
        if self.force_baseline:
            return [K] * D
        task = resolve_task_class(prompt_info, topk_logprobs_cpu, self.gap_high, self.gap_low)
        hists = profile_table.get("per_class_histograms") if profile_table is not None else None
        entry = hists.get(task) if isinstance(hists, dict) else None
        if isinstance(entry, (list, tuple)) and entry:
            if not isinstance(entry[0], (list, tuple)):
                return _stretch([int(x) for x in entry], D, K)
            caps = []
            for d in range(D):
                row = entry[d] if d < len(entry) else []
                b = 1
                for r in range(min(len(row), K)):
                    try:
                        if float(row[r]) > 0.0:
                            b = r + 1
                    except (TypeError, ValueError):
                        break
                caps.append(max(1, min(b, K)))
            return caps
        return _stretch(self.templates.get(task) or self.templates.get("balanced_task") or [], D, K)


REASONING_MARKERS = ("<think>", "step 1", "step 1:", "let me think", "let's think", "first,", "chain of thought")
_REASONING_RE = re.compile("|".join(re.escape(m) for m in REASONING_MARKERS), re.IGNORECASE)
REASONING_LABELS = frozenset({"reasoning", "chain_of_thought", "cot", "math", "code"})


def looks_like_reasoning(prompt_info: Optional[dict], lps, gap_threshold: float) -> bool:
    """Label, then marker regex over the prompt text, then the mean-gap fingerprint."""
    if prompt_info is not None:
        mode = prompt_info.get("mode")
        if isinstance(mode, str) and mode.lower() in {"reasoning", "cot"}:
            return True
        label = prompt_info.get("task")
        if isinstance(label, str) and label.lower() in REASONING_LABELS:
            return True
        ids, tok = prompt_info.get("token_ids"), prompt_info.get("tokenizer")
        if ids is not None and tok is not None:
            try:
                text = tok.decode(list(ids))
            except Exception:
                text = None
            if text and _REASONING_RE.search(text):
                return True
        text = prompt_info.get("text")
        if isinstance(text, str) and _REASONING_RE.search(text):
            return True
    g = _mean_top2_gap(lps)
    return g is not None and g > gap_threshold


@register_tree_algo("reasoning_router")
class ReasoningRouter(CapScheduleAlgorithm):
    """Chain for step-by-step prompts, ``[2, 2, 1, …]`` otherwise."""

    def __init__(self, gap_threshold: float = 1.5, open_ended_template: Optional[list] = None,
                 force_baseline: bool = False):
        self.gap_threshold = float(gap_threshold)
        self.open_ended_template = list(open_ended_template) if open_ended_template is not None else [2, 2] + [1] * 13
        self.force_baseline = bool(force_baseline)

    def caps_from_topk(self, topk_logprobs_cpu, tree_width, prompt_info=None, **kwargs):
        D, K = len(topk_logprobs_cpu), max(int(tree_width), 1)
        if self.force_baseline:
            return [K] * D
        if looks_like_reasoning(prompt_info, topk_logprobs_cpu, self.gap_threshold):
            return [1] * D
        return _stretch(self.open_ended_template, D, K)

    def device_caps_plan(self, D, K, prompt_info=None, profile_table=None):
        D, K = int(D), max(int(K), 1)
        if self.force_baseline:
            return {"mode": "static", "caps": [K] * D}
        if looks_like_reasoning(prompt_info, [], self.gap_threshold):       # the label / the prompt text decides
            return {"mode": "static", "caps": [1] * D}
        open_caps = _stretch(self.open_ended_template, D, K)
        if K < 2:
            return {"mode": "static", "caps": open_caps}
        return {"mode": "gap_select", "hi": self.gap_threshold, "lo": float("-inf"), "above": [1] * D,
                "below": open_caps, "between": open_caps}


# --------------------------------------------------------------------------
# Planned mechanisms: documented, not registered, raise when built
# (reference: jetspec/tree/ROADMAP.md:19-29 and the three placeholder modules).
# --------------------------------------------------------------------------
class _Planned(TreeAlgorithm):
    mechanism = ""

    def build(self, *a, **k):
        raise NotImplementedError(f"{type(self).__name__} is a planned mechanism: {self.mechanism}")


class OnlineWarmup(_Planned):
    mechanism = "collect the depth-rank acceptance table online during the first requests"


class TemplateBandit(_Planned):
    mechanism = "bandit over fan-out templates rewarded by accepted length"


class PathConditionalRefresh(_Planned):
    mechanism = "re-run the drafter conditioned on the best partial path and refresh deeper logits"
