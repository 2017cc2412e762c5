"""Reference engine: contiguous KV cache, explicit masks, physical KV compaction.

This is the correctness oracle for the paged engine (the role ``jetspec/core`` has
in the reference).  It shares the decoder and the tree layer with the paged
engine but none of its KV management.
"""
from .llm import LLM
from .model_runner import ModelRunner, DenseKVCache

__all__ = ["LLM", "ModelRunner", "DenseKVCache"]
