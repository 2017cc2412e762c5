"""B200-native lossless tree-speculative decoding.

Public names mirror the reference package (``jetspec/__init__.py:17-47``) and are
resolved lazily, so ``import jetspec_b200.tree`` never pulls in models or CUDA code.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "LLM": "jetspec_b200.core.llm",
    "SamplingParams": "jetspec_b200.sampling",
    "JetSpecEngine": "jetspec_b200.engine",
    "Drafter": "jetspec_b200.drafters",
    "RepeatDrafter": "jetspec_b200.drafters",
    "TargetEchoDrafter": "jetspec_b200.drafters",
    "TreeDrafter": "jetspec_b200.drafters",
    "RandomTreeDrafter": "jetspec_b200.drafters",
    "TargetEchoTreeDrafter": "jetspec_b200.drafters",
    "DraftHeadDrafter": "jetspec_b200.drafters",
    "DraftHeadTreeDrafter": "jetspec_b200.drafters",
    "OracleTreeDrafter": "jetspec_b200.drafters",
    "GraphedDraftHead": "jetspec_b200.drafters",
    "CompiledDraftHead": "jetspec_b200.drafters",
    "OracleOverrideDrafter": "jetspec_b200.drafters",
    "load_draft_head": "jetspec_b200.models",
    "load_target": "jetspec_b200.models",
}

__all__ = sorted(_LAZY)


def __getattr__(name: str):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'jetspec_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(mod), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
