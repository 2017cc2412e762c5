"""Paged-KV decode engine."""
from ..sampling import SamplingParams
from .engine import JetSpecEngine, bucket_for_n, TREE_BUCKETS

__all__ = ["JetSpecEngine", "SamplingParams", "bucket_for_n", "TREE_BUCKETS"]
