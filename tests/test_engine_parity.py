"""Engine gates on CPU fp32: paged AR == reference AR (N0), paged tree == greedy (N1),
batch == per-prompt (N2a), tree batch == per-prompt (N2b), eviction/restore keeps outputs."""
import pytest
import torch

from jetspec_b200 import (JetSpecEngine, LLM, SamplingParams, RandomTreeDrafter, TargetEchoTreeDrafter)

SP = SamplingParams(0.0, 32)


@pytest.fixture(scope="module")
def engine(tiny_model):
    return JetSpecEngine(tiny_model, device="cpu", dtype=torch.float32)


@pytest.fixture(scope="module")
def llm(tiny_model):
    return LLM(tiny_model, device="cpu", dtype=torch.float32)


@pytest.fixture(scope="module")
def prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 1024, (1, n), generator=g) for n in (5, 17, 32, 9)]


def test_n0_paged_ar_equals_reference(engine, llm, tiny_prompt):
    assert engine.generate(tiny_prompt, SP)["token_ids"] == llm.generate(tiny_prompt, SP)["token_ids"]


@pytest.mark.parametrize("drafter", ["random", "echo"])
def test_n1_paged_tree_equals_greedy(engine, llm, tiny_model, tiny_prompt, drafter):
    d = RandomTreeDrafter(1024, seed=1) if drafter == "random" else TargetEchoTreeDrafter(tiny_model)
    ref = llm.generate(tiny_prompt, SP)["token_ids"]
    out = engine.generate_tree(tiny_prompt, d, block_size=5, tree_width=2, budget=8, sampling_params=SP,
                               return_stats=True, tree_diag=True)
    assert out["token_ids"] == ref
    assert sum(out["tree_sizes"]) == sum(out["tree_nodes_per_depth"])
    hf = llm.generate_tree(tiny_prompt, d, block_size=5, tree_width=2, budget=8, sampling_params=SP, return_stats=True)
    if drafter == "echo":
        assert out["accept_lengths"] == hf["accept_lengths"]


def test_pool_holds_only_committed_plus_window(engine, tiny_prompt):
    engine.generate_tree(tiny_prompt, RandomTreeDrafter(1024, seed=1), block_size=5, tree_width=2, budget=8,
                         sampling_params=SP)
    assert engine.pool.free_page_count == engine.pool.num_pages   # everything returned


def test_tree_depth_rule(engine, tiny_prompt):
    d = RandomTreeDrafter(1024, seed=1)
    with pytest.raises(ValueError):
        engine.generate_tree(tiny_prompt, d, block_size=7, tree_depth=4, sampling_params=SamplingParams(0.0, 4))
    out = engine.generate_tree(tiny_prompt, d, tree_depth=4, tree_width=2, budget=8, sampling_params=SamplingParams(0.0, 8))
    assert len(out["token_ids"]) == 8


def test_session_mismatch_is_loud(tiny_model, tiny_prompt):
    eng = JetSpecEngine(tiny_model, device="cpu", dtype=torch.float32)
    d = RandomTreeDrafter(1024, seed=1)
    sp = SamplingParams(0.0, 8)
    eng.generate_tree(tiny_prompt, d, tree_depth=4, tree_width=2, budget=8, sampling_params=sp, session=True)
    eng.generate_tree(tiny_prompt, d, tree_depth=4, tree_width=2, budget=8, sampling_params=sp, session=True)
    with pytest.raises(ValueError, match="tree session mismatch"):
        eng.generate_tree(tiny_prompt, d, tree_depth=6, tree_width=2, budget=8, sampling_params=sp, session=True)
    long_prompt = torch.randint(0, 1024, (1, 300))
    with pytest.raises(ValueError, match="prompt_len"):
        eng.generate_tree(long_prompt, d, tree_depth=4, tree_width=2, budget=8, sampling_params=sp, session=True)


def test_n2a_batch_equals_single(engine, llm, prompts):
    singles = [llm.generate(p, SP)["token_ids"] for p in prompts]
    assert [r["token_ids"] for r in engine.generate_batch(prompts, SP)] == singles


def test_n2b_tree_batch_equals_single(engine, llm, prompts):
    singles = [llm.generate(p, SP)["token_ids"] for p in prompts]
    out = engine.generate_tree_batch(prompts, RandomTreeDrafter(1024, seed=2), block_size=5, tree_width=2, budget=8,
                                     sampling_params=SP)
    assert [r["token_ids"] for r in out] == singles
    assert all(r["tpf"] >= 1.0 for r in out)


def test_small_pool_evicts_and_restores(tiny_model, llm, prompts):
    eng = JetSpecEngine(tiny_model, device="cpu", dtype=torch.float32, num_pages=10, max_seq_len=128)
    singles = [llm.generate(p, SP)["token_ids"] for p in prompts]
    assert [r["token_ids"] for r in eng.generate_batch(prompts, SP)] == singles
    assert eng.pool.free_page_count == eng.pool.num_pages
    out = eng.generate_tree_batch(prompts, RandomTreeDrafter(1024, seed=2), block_size=5, tree_width=2, budget=8,
                                  sampling_params=SP, max_batch_size=2)
    assert [r["token_ids"] for r in out] == singles


def test_extension_is_lossless(engine, llm, tiny_model, tiny_prompt):
    class CondEcho(TargetEchoTreeDrafter):
        def propose_logits(self, context_ids, depth, target_hidden=None, **kw):
            # sharpen: a confident drafter makes the builder follow the rank-1 chain to full depth
            return 100.0 * super().propose_logits(context_ids, depth)

        def propose_logits_conditioned(self, context_ids, path_tokens, target_hidden=None, **kw):
            ctx = torch.cat((context_ids, torch.as_tensor(path_tokens).reshape(1, -1)), 1)
            return self.propose_logits(ctx, 4)
    ref = llm.generate(tiny_prompt, SP)["token_ids"]
    out = engine.generate_tree(tiny_prompt, CondEcho(tiny_model), block_size=5, tree_width=2, budget=9,
                               sampling_params=SP, return_stats=True, max_tree_depth=8,
                               extend_kwargs={"gap_threshold": -1e9, "ext_budget": 4})
    assert out["token_ids"] == ref
    assert max(out["accept_lengths"]) > 5     # accepted beyond the un-extended ceiling
