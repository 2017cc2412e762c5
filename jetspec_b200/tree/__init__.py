"""Tree-drafting method layer: engine-agnostic, depends on torch + numpy only.

It turns per-depth draft logits into a verification tree and selects the accepted
path.  Engines import from here and nothing here imports an engine
(reference contract: ``jetspec/tree/__init__.py:10-47``).
"""
from .types import DraftTree, TreeAlgorithm
from .registry import get_algorithm, register_tree_algo, list_algorithms
from .ancestor import build_ancestor_matrix, build_packed_ancestor_matrix
from .accept import gpu_tree_accept, tree_accept
from .extend import should_extend, splice_extension
from .builder import build_from_topk, build_with_per_depth_cap
from . import algorithms  # noqa: F401  (registers the bundled algorithms)

__all__ = [
    "DraftTree", "TreeAlgorithm", "get_algorithm", "register_tree_algo", "list_algorithms",
    "build_ancestor_matrix", "build_packed_ancestor_matrix", "gpu_tree_accept", "tree_accept",
    "build_from_topk", "build_with_per_depth_cap", "should_extend", "splice_extension",
]
