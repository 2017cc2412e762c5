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


def test_admission_does_not_evict_for_room_that_only_protected_requests_hold():
    """A waiting request whose room could only come from requests admitted in the same step must wait: the
    scheduler stops admitting instead of evicting every other running sequence and failing anyway."""
    from jetspec_b200.runtime import PagedKVPool, Scheduler, SequenceRequest
    pool = PagedKVPool(1, 1, 8, num_pages=10, page_size=4, max_seqs=8, max_seq_len=64)
    sched = Scheduler(pool, max_batch_size=8, prefill_batch_size=8)
    old = SequenceRequest(seq_id=1, input_ids=list(range(8)), max_new_tokens=4)       # 2 pages, running
    sched.admit_request(old)
    out = sched.step()
    assert [r.seq_id for r in out.admitted] == [1]
    sched.mark_decode_step(1, 5)
    # two newcomers: the first takes 6 of the 8 free pages; the second needs 5 and could only fit by also
    # taking the first newcomer's pages (protected) -- evicting sequence 1 (2 pages) would not be enough
    sched.admit_request(SequenceRequest(seq_id=2, input_ids=list(range(24)), max_new_tokens=4))
    sched.admit_request(SequenceRequest(seq_id=3, input_ids=list(range(20)), max_new_tokens=4))
    out = sched.step()
    assert [r.seq_id for r in out.admitted] == [2]
    assert out.evicted == [] and 1 in sched.running and pool.has(1)
    assert [r.seq_id for r in sched.waiting_queue] == [3]


def test_loader_rejects_a_checkpoint_that_lacks_expert_slices(tmp_path):
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config
    from jetspec_b200.models.loader import save_state
    cfg = Qwen3Config(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=16, num_experts=4, num_experts_per_tok=2,
                      moe_intermediate_size=16, norm_topk_prob=True, model_type="qwen3_moe")
    m = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.float32, device="cpu")
    m.save_pretrained(str(tmp_path / "full"))
    again = Qwen3ForCausalLM.from_pretrained(str(tmp_path / "full"), dtype=torch.float32, device="cpu")
    assert torch.equal(again.model.layers[0].mlp.w_gate_up, m.model.layers[0].mlp.w_gate_up)
    from safetensors.torch import load_file
    sd = load_file(str(tmp_path / "full" / "model.safetensors"))
    for drop in ("model.layers.0.mlp.experts.2.up_proj.weight", "model.layers.0.mlp.experts.3.down_proj.weight"):
        part = {k: v for k, v in sd.items() if k != drop}
        d = tmp_path / ("lacks_" + drop.split(".")[-2] + drop.split(".")[-3])
        cfg.save_pretrained(str(d))
        save_state(part, str(d))
        with pytest.raises(KeyError, match="missing"):
            Qwen3ForCausalLM.from_pretrained(str(d), dtype=torch.float32, device="cpu")
