"""Tree layer unit tests: builder vs brute force, identity-knob recovery, build_from_topk == build,
vectorised accept == host walk (duplicate siblings included), extension helpers."""
import math
import random

import pytest
import torch

from jetspec_b200.tree import (build_ancestor_matrix, build_from_topk, get_algorithm, gpu_tree_accept,
                               list_algorithms, register_tree_algo, should_extend, splice_extension, tree_accept)
from jetspec_b200.tree.algorithms import OnlineWarmup, sigmoid_cap
from jetspec_b200.tree.builder import build_with_per_depth_cap


def brute_force(root, toks, lps, caps, budget):
    """O(n^2) restatement: repeatedly expand the unexpanded node with the largest cumulative logprob."""
    D, K = len(toks), len(toks[0])
    nodes = [(root, -1, 0, 0.0)]
    pending = [(0.0, 0, 0)]
    order = 0
    while pending and len(nodes) < budget:
        best = min(pending)
        pending.remove(best)
        neg, _, i = best
        d = nodes[i][2]
        if d >= D:
            continue
        for j in range(min(caps[d], K, budget - len(nodes))):
            order += 1
            nodes.append((toks[d][j], i, d + 1, -neg + lps[d][j]))
            pending.append((-(-neg + lps[d][j]), order, len(nodes) - 1))
    return nodes


@pytest.mark.parametrize("seed", range(5))
def test_builder_matches_brute_force(seed):
    rng = random.Random(seed)
    D, K, budget = 6, 4, rng.randint(2, 40)
    toks = [[rng.randrange(1000) for _ in range(K)] for _ in range(D)]
    lps = [sorted([-rng.random() * 5 for _ in range(K)], reverse=True) for _ in range(D)]
    caps = [rng.randint(1, K) for _ in range(D)]
    t = build_with_per_depth_cap(7, toks, lps, caps, budget, "cpu")
    ref = brute_force(7, toks, lps, caps, budget)
    assert t.token_ids.tolist() == [n[0] for n in ref]
    assert t.parent_indices.tolist() == [n[1] for n in ref]
    assert t.depth.tolist() == [n[2] for n in ref]
    assert t.num_nodes <= budget
    anc = build_ancestor_matrix(t)
    for i in range(t.num_nodes):
        chain, c = set(), i
        while c >= 0:
            chain.add(c)
            c = int(t.parent_indices[c])
        assert set(torch.nonzero(anc[i]).flatten().tolist()) == chain


def test_registry_lists_the_six_algorithms():
    assert list_algorithms() == ["accum_logp", "class_histogram", "depth_rank_histogram", "reasoning_router",
                                 "task_router", "top2gap_fanout"]
    with pytest.raises(KeyError):
        get_algorithm("nope")
    with pytest.raises(ValueError):
        register_tree_algo("accum_logp")(type("X", (), {}))
    with pytest.raises(NotImplementedError):
        OnlineWarmup().build(0, None, 0, 0, 0, "cpu")


IDENTITY = [("top2gap_fanout", {"beta": 1.0, "g_0": 1e9}), ("depth_rank_histogram", {"tau": 0.0}),
            ("task_router", {"force_baseline": True}), ("reasoning_router", {"force_baseline": True}),
            ("class_histogram", {"force_baseline": True})]


@pytest.mark.parametrize("name,kw", IDENTITY)
def test_identity_knob_recovers_accum_logp(name, kw):
    torch.manual_seed(0)
    lg = torch.randn(1, 6, 300) * 3
    base = get_algorithm("accum_logp").build(3, lg, 7, 4, 30, "cpu")
    t = get_algorithm(name, **kw).build(3, lg, 7, 4, 30, "cpu")
    for f in ("token_ids", "parent_indices", "depth", "cum_logprob"):
        assert torch.equal(getattr(t, f), getattr(base, f))


@pytest.mark.parametrize("name", ["accum_logp", "top2gap_fanout", "depth_rank_histogram", "task_router"])
def test_build_from_topk_equals_build(name):
    torch.manual_seed(1)
    lg = torch.randn(1, 5, 200) * 2
    table = {"depth_rank_accept": [[0.5, 0.1, 0.01, 0.0]] * 5}
    dense = get_algorithm(name).build(9, lg, 6, 4, 20, "cpu", profile_table=table)
    lp = torch.log_softmax(lg[0], -1)
    v, i = torch.topk(lp, 4, -1)
    sparse = build_from_topk(name, 9, i, v, 20, "cpu", tree_width=4, profile_table=table)
    assert torch.equal(dense.token_ids, sparse.token_ids) and torch.equal(dense.parent_indices, sparse.parent_indices)


def test_cap_schedules():
    assert sigmoid_cap(0.0, 7, 1.0, 1.0) == max(1, round(7 / (1 + math.exp(-1))))
    assert sigmoid_cap(50.0, 7, 1.0, 1.0) == 1
    a = get_algorithm("depth_rank_histogram", tau=0.02)
    assert a.caps_from_topk([[0, -1, -2]] * 3, 3, profile_table={"depth_rank_accept": [[0.9, 0.05, 0.001], [0.9, 0.0, 0.0]]}) == [2, 1, 3]
    r = get_algorithm("task_router")
    assert r.caps_from_topk([[0, -5, -6]] * 4, 3, prompt_info={"task": "chat"}) == [3, 3, 1, 1]
    assert r.caps_from_topk([[0, -5, -6]] * 4, 3) == [1, 1, 1, 1]          # decisive by mean gap
    assert get_algorithm("reasoning_router").caps_from_topk([[0, -0.1]] * 3, 2, prompt_info={"text": "Let me think"}) == [1, 1, 1]
    assert get_algorithm("reasoning_router").caps_from_topk([[0, -0.1]] * 3, 2) == [2, 2, 1]
    ch = get_algorithm("class_histogram")
    table = {"per_class_histograms": {"decisive_task": [[0.5, 0.2, 0.0], [0.9, 0.0, 0.0]]}}
    assert ch.caps_from_topk([[0, -9, -9]] * 3, 3, prompt_info={"task": "math"}, profile_table=table) == [2, 1, 1]


@pytest.mark.parametrize("seed", range(8))
def test_vectorised_accept_equals_host_walk(seed):
    rng = random.Random(seed)
    n, V = rng.randint(2, 40), 6          # tiny vocabulary → duplicate sibling tokens happen
    parents, depths = [-1], [0]
    for i in range(1, n):
        p = rng.randrange(i)
        parents.append(p)
        depths.append(depths[p] + 1)
    tokens = [rng.randrange(V) for _ in range(n)]
    from jetspec_b200.tree import DraftTree
    tree = DraftTree(torch.tensor(tokens), torch.tensor(parents), torch.tensor(depths), n)
    logits = torch.randn(1, n, V, generator=torch.Generator().manual_seed(seed))
    path_h, acc_h, corr_h = tree_accept(tree, logits)
    path_v, acc_v, corr_v = gpu_tree_accept(tree.token_ids, logits[0].argmax(-1), tree.parent_indices, tree.depth,
                                            max_depth=max(depths))
    assert path_v.tolist() == path_h and acc_v == acc_h and int(corr_v) == corr_h


def test_extension_helpers():
    lp = torch.tensor([[-0.1, -3.0], [-0.2, -2.5]])
    assert should_extend(lp, [0, 0], gap_threshold=1.0)
    assert not should_extend(lp, [1, 0], gap_threshold=1.0)
    assert not should_extend(lp[:, :1], [0, 0], gap_threshold=0.0)
    with pytest.raises(ValueError):
        should_extend(lp, [0], gap_threshold=0.0)
    t = get_algorithm("accum_logp").build(1, torch.randn(1, 2, 50), 3, 1, 3, "cpu")
    ext = torch.randn(1, 3, 50)
    t2 = splice_extension(t, 2, ext, ext_budget=3, tree_width=2, mode="chain")
    assert t2.num_nodes == 6 and t2.parent_indices.tolist()[3:] == [2, 3, 4] and t2.depth.tolist()[3:] == [3, 4, 5]
    assert t2.token_ids.tolist()[3:] == ext[0].argmax(-1).tolist()
    t3 = splice_extension(t, 2, ext, ext_budget=3, tree_width=2, mode="subtree")
    assert t3.num_nodes == 6 and t3.parent_indices[3] == 2
    with pytest.raises(ValueError):
        splice_extension(t, 0, ext, ext_budget=1, tree_width=2)
    assert splice_extension(t, 2, ext, ext_budget=0, tree_width=2) is t


def test_host_accept_matches_vectorised_accept():
    """The list-based greedy acceptance used by the batched engine path equals the tensor version on random
    trees, including duplicate siblings (the later one wins) and ties in depth (the lower index wins)."""
    import random
    import torch
    from jetspec_b200.tree.accept import gpu_tree_accept, host_tree_accept
    rng = random.Random(0)
    for trial in range(200):
        n = rng.randint(1, 24)
        tokens, parents, depths = [rng.randint(0, 3)], [-1], [0]
        for i in range(1, n):
            p = rng.randint(0, i - 1)
            parents.append(p)
            depths.append(depths[p] + 1)
            tokens.append(rng.randint(0, 3))
        greedy = [rng.randint(0, 3) for _ in range(n)]
        path_h, acc_h, corr_h = host_tree_accept(tokens, parents, depths, greedy)
        path_g, acc_g, corr_g = gpu_tree_accept(torch.tensor(tokens), torch.tensor(greedy), torch.tensor(parents),
                                                torch.tensor(depths), max_depth=max(max(depths), 1))
        assert path_h == path_g.tolist() and acc_h == acc_g and corr_h == int(corr_g), (trial, tokens, parents, greedy)


def test_host_only_tree_carries_the_same_lists():
    """``device="host"`` builds the tree without tensors (for consumers that stage their own device buffers);
    its lists equal those of the tensor-backed tree."""
    from jetspec_b200.tree.builder import build_from_topk
    toks = [[5, 9, 2], [7, 7, 1], [3, 4, 8]]
    lps = [[-0.1, -2.5, -4.0], [-0.3, -1.5, -3.0], [-0.2, -2.0, -2.5]]
    full = build_from_topk("accum_logp", 11, toks, lps, 8, "cpu", tree_width=3)
    host = build_from_topk("accum_logp", 11, toks, lps, 8, "host", tree_width=3)
    assert host.token_ids is None and host.num_nodes == full.num_nodes
    assert host.host == full.host == (full.token_ids.tolist(), full.parent_indices.tolist(), full.depth.tolist())


def test_device_caps_plans_reproduce_every_algorithm():
    """The per-request plan a device kernel evaluates gives the algorithm's own caps for any round's log-probs,
    for every registered algorithm, with and without labels, profile tables and the baseline switch."""
    import random
    from jetspec_b200.tree import get_algorithm, list_algorithms
    from jetspec_b200.tree.algorithms import eval_caps_plan
    rng = random.Random(0)
    D, K = 6, 5
    table = {"depth_rank_accept": [[rng.random() * 0.1 for _ in range(K)] for _ in range(D)],
             "per_class_histograms": {"decisive_task": [2, 1], "uncertain_task": [[0.5, 0.2, 0.0, 0.1, 0.0]] * D}}
    cases = [("accum_logp", {}, None, None), ("top2gap_fanout", {"beta": 1.7, "g_0": 0.6}, None, None),
             ("depth_rank_histogram", {"tau": 0.03}, None, table), ("depth_rank_histogram", {}, None, None),
             ("task_router", {}, None, None), ("task_router", {}, {"task": "chat"}, None),
             ("task_router", {"force_baseline": True}, None, None),
             ("class_histogram", {}, None, table), ("class_histogram", {}, {"task": "math"}, table),
             ("reasoning_router", {}, None, None), ("reasoning_router", {}, {"text": "Let me think. 2+2"}, None),
             ("reasoning_router", {"gap_threshold": 0.4}, {"task": "poetry"}, None)]
    assert {c[0] for c in cases} == set(list_algorithms())
    for name, kw, info, prof in cases:
        algo = get_algorithm(name, **kw)
        plan = algo.device_caps_plan(D, K, prompt_info=info, profile_table=prof)
        assert plan is not None and plan["mode"] in ("static", "sigmoid", "gap_select")
        for scale in (0.05, 0.5, 1.5, 4.0):          # from near-flat to very peaked candidates
            for _ in range(20):
                lps = [sorted((-rng.random() * scale * 3 for _ in range(K)), reverse=True) for _ in range(D)]
                want = algo.caps_from_topk(lps, K, prompt_info=info, profile_table=prof)
                assert eval_caps_plan(plan, lps, K) == want, (name, kw, info)
