"""Tier-0 gate: on a tiny fp32 Qwen3, every speculative path reproduces plain greedy decoding
token for token, for any drafter (the lossless property)."""
import pytest
import torch

from jetspec_b200 import (LLM, SamplingParams, RandomTreeDrafter, TargetEchoTreeDrafter, RepeatDrafter,
                          TargetEchoDrafter)


@pytest.fixture(scope="module")
def llm(tiny_model):
    return LLM(tiny_model, device="cpu", dtype=torch.float32)


@pytest.fixture(scope="module")
def greedy(llm, tiny_prompt):
    return llm.generate(tiny_prompt, SamplingParams(0.0, 32))["token_ids"]


def test_ar_length(greedy):
    assert len(greedy) == 32


@pytest.mark.parametrize("algo", ["accum_logp", "top2gap_fanout", "task_router", "reasoning_router",
                                  "class_histogram", "depth_rank_histogram"])
def test_tree_random_drafter_is_lossless(llm, tiny_prompt, greedy, algo):
    d = RandomTreeDrafter(1024, seed=3)
    out = llm.generate_tree(tiny_prompt, d, block_size=5, tree_width=2, budget=8, algo=algo,
                            sampling_params=SamplingParams(0.0, 32), return_stats=True)
    assert out["token_ids"] == greedy
    assert out["rounds"] == len(out["accept_lengths"]) == len(out["tree_sizes"])


def test_tree_echo_drafter_accepts_full_depth(llm, tiny_model, tiny_prompt, greedy):
    out = llm.generate_tree(tiny_prompt, TargetEchoTreeDrafter(tiny_model), block_size=5, tree_width=2, budget=8,
                            sampling_params=SamplingParams(0.0, 32), return_stats=True)
    assert out["token_ids"] == greedy
    # depth 4 / width 2 / budget 8 reaches depth 3 on the rank-1 chain: 3 accepted + 1 correction
    assert out["accept_lengths"][0] == 4
    assert out["tpf"] > 3.0


def test_chain_drafters_are_lossless(llm, tiny_model, tiny_prompt, greedy):
    sp = SamplingParams(0.0, 32)
    assert llm.generate_chain(tiny_prompt, RepeatDrafter(), block_size=4, sampling_params=sp)["token_ids"] == greedy
    r = llm.generate_chain(tiny_prompt, TargetEchoDrafter(tiny_model), block_size=4, sampling_params=sp)
    assert r["token_ids"] == greedy and r["tpf"] == pytest.approx(4.0)


def test_temperature_sampling_runs(llm, tiny_prompt):
    torch.manual_seed(0)
    out = llm.generate_tree(tiny_prompt, RandomTreeDrafter(1024, seed=1), block_size=5, tree_width=2, budget=8,
                            sampling_params=SamplingParams(0.8, 16))
    assert len(out["token_ids"]) == 16


def test_tree_attn_switch_is_validated_and_harmless_on_cpu(tiny_model, tiny_prompt):
    """``tree_attn="kernel"`` asks for the GPU attention kernel; on a CPU the request is ignored (same tokens as the
    default), and an unknown value is an error."""
    import pytest
    from jetspec_b200 import LLM, SamplingParams, RandomTreeDrafter
    llm = LLM(tiny_model, device="cpu", dtype=torch.float32)
    sp = SamplingParams(0.0, 12)
    kw = dict(block_size=5, tree_width=2, budget=8, sampling_params=sp)
    a = llm.generate_tree(tiny_prompt, RandomTreeDrafter(tiny_model.config.vocab_size, seed=1), **kw)
    b = llm.generate_tree(tiny_prompt, RandomTreeDrafter(tiny_model.config.vocab_size, seed=1), tree_attn="kernel", **kw)
    assert a["token_ids"] == b["token_ids"] == llm.generate(tiny_prompt, sp)["token_ids"]
    with pytest.raises(ValueError, match="tree_attn"):
        llm.generate_tree(tiny_prompt, RandomTreeDrafter(tiny_model.config.vocab_size, seed=1), tree_attn="flash", **kw)
