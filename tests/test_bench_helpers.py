"""Unit tests of the benchmark / profiling helper functions (pure, CPU)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench"))
import profiling as P          # noqa: E402
import engine_tps as E         # noqa: E402
import reference_metrics as R  # noqa: E402


def test_summarize_tree_diag_and_report():
    m = P.summarize_tree_diag(accept_lengths=[1, 3, 3, 5], tree_nodes_per_depth=[4, 8, 8, 4, 4], output_tokens=12,
                              num_samples=2, block_size=5)
    assert m["acceptance_length"] == 3.0 and m["num_drafts"] == 4
    assert m["acceptance_length_histogram"] == [0.25, 0.0, 0.5, 0.0, 0.25]
    assert m["per_depth_acceptance_rate"] == [0.75, 0.75, 0.25, 0.25]
    assert m["avg_tree_nodes_per_depth"] == [2.0, 2.0, 1.0, 1.0]
    text = P.format_metrics_report(m, attention_backend="x", block_size=5, tree_width=2, budget=8, algo="a", drafter="d")
    assert "acceptance_length=3.000000" in text and text.endswith("\n")
    with pytest.raises(ValueError):
        P.summarize_tree_diag(accept_lengths=[9], tree_nodes_per_depth=[1], output_tokens=1, num_samples=1, block_size=5)


def test_depth_rank_profile_feeds_the_algorithm():
    seq = [0, 1, 2, 3, 4, 5, 6]
    rounds = [(2, [[2, 9], [9, 3], [8, 8]]),     # depth0 rank0 hit, depth1 rank1 hit, depth2 miss
              (5, [[7, 7], [6, 1]])]             # depth0 miss -> deeper depths not counted
    hits, trials = P.depth_rank_counts(rounds, seq, width=2, depth=3)
    assert hits == [[1, 0], [0, 1], [0, 0]] and trials == [2, 1, 1]
    prof = P.depth_rank_profile(hits, trials, {"n": 2})
    assert prof["depth_rank_accept"][0] == [0.5, 0.0]
    from jetspec_b200.tree import get_algorithm
    caps = get_algorithm("depth_rank_histogram", tau=0.4).caps_from_topk([[0, -1]] * 3, 2, profile_table=prof)
    assert caps == [1, 1, 1]


def test_conditioned_probe_verdict_and_speedup():
    v = P.conditioned_probe_verdict([10, 10, 0, 20], [0, 1, 0, 20], top=7, lift_threshold=0.15)
    assert v["verdict"] == "P3_BUILD" and v["lift"] == pytest.approx(0.5)
    assert P.conditioned_probe_verdict([0, 0], [0, 0])["verdict"] == "P3_SKIP"
    assert P.rank_of(2, torch.tensor([0.1, 0.9, 0.5])) == 1
    assert P.decode_cuda_speedup(10.0, 100, 2.0, 100) == pytest.approx(5.0)


def test_prompt_bank_sharding_and_reduction():
    bank = E.prompt_bank("gsm8k", 7, vocab=100, seed=1)
    assert len(bank) == 7 and all(96 <= p.shape[1] <= 256 for p in bank)
    parts = [E.shard(bank, r, 3) for r in range(3)]
    assert sum(len(p) for p in parts) == 7 and parts[0][1] is bank[3]
    s = E.reduce_stats(100, 2.0, 80.0, 10, world=1)
    assert s["tps"] == 50.0 and s["accept_len"] == 8.0


def test_reference_metric_rows():
    outs = [{"token_ids": [1] * 10, "accept_lengths": [1, 2, 5], "tree_sizes": [8, 8, 8], "decode_time": 0.5}]
    row = R.summarize("accum_logp", outs, [1.0], ar_tps=5.0, chain_tps=8.0)
    assert row["accept_len"] == pytest.approx(8 / 3) and row["e2e_tps"] == 10.0 and row["decode_tps"] == 20.0
    assert row["speedup_vs_ar"] == 2.0 and row["d0"] == pytest.approx(2 / 3) and row["d3"] == pytest.approx(1 / 3)


def test_all_node_rank_counts_counts_every_parent():
    all_node_rank_counts = P.all_node_rank_counts
    # depth-0 root and two depth-1 nodes are parents; the depth-2 leaf is beyond the drafted depths (D = 2)
    depths = [0, 1, 1, 2]
    topk = [[10, 11], [20, 21]]
    pick = [11, 20, 99, 5]                       # root -> rank 1; first child -> rank 0; second child -> not in top-k
    hits, totals = all_node_rank_counts(depths, pick, topk)
    assert totals == [1, 2] and hits == [[0, 1], [1, 0]]


def test_llm_round_collector_runs_on_the_reference_engine_path():
    """The LLM-path collector and the conditioned-vs-marginal probe run end to end on a tiny model."""
    import subprocess, sys, os, json
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for mode in ("llm-depth-rank", "conditioned-probe"):
        r = subprocess.run([sys.executable, os.path.join(root, "bench", "profiling.py"), mode, "--samples", "1",
                            "--max-new", "12"], capture_output=True, text=True, cwd=root)
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads(r.stdout[r.stdout.index("{"):])
        if mode == "llm-depth-rank":
            assert len(out["depth_rank_accept"]) == 4 and sum(out["meta"]["trials"]) > 0
        else:
            assert out["verdict"] in ("P3_BUILD", "P3_SKIP") and "lift" in out


def test_kernel_config_pickers_on_cpu():
    """Host-side launch policies that need no GPU: the GEMM picker's many-row rule and the attention split count."""
    from jetspec_b200.ops import cuda_ext as X
    # decode: one row tile, weight streaming -> K split over a cluster while the grid stays one wave
    assert X.pick_gemm_config(128, 4096, 4096, X.EPI_STORE)[:2] == (128, 4)
    assert X.pick_gemm_config(128, 6144, 4096, X.EPI_STORE)[:2] == (128, 2)
    # many rows: 256-column tiles; two row tiles per CTA only where that does not add a wave of (bigger) tiles
    assert X.pick_gemm_config(2048, 4096, 4096, X.EPI_STORE) == (256, 1, 3)
    assert X.pick_gemm_config(2048, 4096, 12288, X.EPI_STORE) == (256, 1, 3)
    assert X.pick_gemm_config(2048, 6144, 4096, X.EPI_STORE) == (256, 1, 1)
    assert X.pick_gemm_config(512, 4096, 4096, X.EPI_STORE) == (256, 1, 1)
    # attention: one wave of CTAs; 32 query tiles x heads leave 4 key splits, a shard with one KV head gets 16
    assert X.attn_splits_for(128, 32, 8, 2700) == 4
    assert X.attn_splits_for(128, 4, 1, 2700) == 16
    assert X.attn_splits_for(2048, 32, 8, 2700) == 1
    # in-cluster merge: up to 8 splits and only while every cluster of the launch is resident at once
    assert X.attn_merges_in_cluster(128, 32, 8, 4)
    assert not X.attn_merges_in_cluster(128, 32, 8, 16)
    assert not X.attn_merges_in_cluster(128, 32, 8, 1)
