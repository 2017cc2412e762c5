"""Model definitions and checkpoint loaders."""
from .config import (Qwen3Config, tiny_config, qwen3_8b_config, qwen3_30b_a3b_config, draft_head_config)
from .qwen3 import Qwen3ForCausalLM, load_target, load_tokenizer
from .draft_head import DraftHeadModel, load_draft_head, build_target_layer_ids, extract_context_feature

__all__ = [
    "Qwen3Config", "tiny_config", "qwen3_8b_config", "qwen3_30b_a3b_config", "draft_head_config",
    "Qwen3ForCausalLM", "load_target", "load_tokenizer",
    "DraftHeadModel", "load_draft_head", "build_target_layer_ids", "extract_context_feature",
]
