"""Cross-check against the reference package itself (when installed under baseline/_ref): the same
tiny fp32 checkpoint, written in the stock Hugging Face layout, must decode to the same tokens through
the reference's ``LLM`` and through this framework, for AR and for tree-speculative decoding."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "jetspec")),
                                reason="reference package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory, tiny_model):
    sys.path.insert(0, ROOT)
    from baseline.reference_arm import write_hf_config, write_tokenizer
    from jetspec_b200.models.loader import save_state
    d = str(tmp_path_factory.mktemp("tiny_ckpt"))
    write_hf_config(d, tiny_model.config, {"torch_dtype": "float32"})
    save_state(dict(tiny_model.state_dict()), d)
    write_tokenizer(d, tiny_model.config.vocab_size)
    return d


def test_reference_llm_matches_ours(checkpoint, tiny_model, tiny_prompt):
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        from jetspec import LLM as RefLLM, SamplingParams as RefSP, RandomTreeDrafter as RefRandom
    except Exception as e:  # the reference needs transformers; report rather than fail the suite
        pytest.skip(f"reference not importable here: {e}")
    from jetspec_b200 import LLM, SamplingParams, JetSpecEngine, RandomTreeDrafter
    from jetspec_b200.models import Qwen3ForCausalLM
    ref = RefLLM(checkpoint, device="cpu", dtype=torch.float32, attn_implementation="sdpa")
    ours_loaded = Qwen3ForCausalLM.from_pretrained(checkpoint, dtype=torch.float32)   # the same files load here too
    ours = LLM(ours_loaded, device="cpu", dtype=torch.float32)
    ref_ar = ref.generate(tiny_prompt, RefSP(0.0, 24))["token_ids"]
    assert ours.generate(tiny_prompt, SamplingParams(0.0, 24))["token_ids"] == ref_ar
    torch.manual_seed(0)
    ref_tree = ref.generate_tree(tiny_prompt, RefRandom(1024), block_size=5, tree_width=2, budget=8,
                                 sampling_params=RefSP(0.0, 24))["token_ids"]
    assert ref_tree == ref_ar
    eng = JetSpecEngine(ours_loaded, device="cpu", dtype=torch.float32)
    out = eng.generate_tree(tiny_prompt, RandomTreeDrafter(1024, seed=0), block_size=5, tree_width=2, budget=8,
                            sampling_params=SamplingParams(0.0, 24))["token_ids"]
    assert out == ref_ar
