"""Sampling parameters and the token sampler."""
from __future__ import annotations

from dataclasses import dataclass

from .ops import sample  # noqa: F401  (re-export)


@dataclass
class SamplingParams:
    """``SamplingParams(temperature=0.0, max_new_tokens=256)`` — positional use is supported,
    e.g. ``SamplingParams(0.0, 64)`` (reference: ``jetspec/core/llm.py:79-82``)."""
    temperature: float = 0.0
    max_new_tokens: int = 256
