"""Host-side logic of the multi-GPU paths, on CPU: sharding plans (bf16 and NVFP4), routing + permutation,
and a two-process gloo run of the tensor-parallel layer plan against the single-process layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jetspec_b200.models import Qwen3ForCausalLM, tiny_config
from jetspec_b200.ops import reference as ref
from jetspec_b200.parallel.tp import shard_attention, shard_cols, shard_mlp, shard_rows, stack_rows


def test_row_and_column_shards_reassemble_the_product():
    torch.manual_seed(0)
    x, w = torch.randn(5, 64), torch.randn(48, 64)
    full = x @ w.t()
    world = 4
    cols = torch.cat([x @ shard_rows(w, r, world).t() for r in range(world)], dim=1)          # column-parallel
    assert torch.allclose(cols, full, atol=1e-5)
    rows = sum(shard_cols(x, r, world) @ shard_cols(w, r, world).t() for r in range(world))   # row-parallel
    assert torch.allclose(rows, full, atol=1e-4)


def test_nvfp4_shards_are_exact_slices():
    from jetspec_b200.models.nvfp4 import NVFP4Tensor, quantize_nvfp4
    torch.manual_seed(1)
    w = torch.randn(64, 256) * 0.05
    q = quantize_nvfp4(w, swizzle=False)
    d = q.dequantize()
    assert torch.equal(shard_rows(q, 1, 4).dequantize(), d[16:32])
    assert torch.equal(shard_cols(q, 2, 4).dequantize(), d[:, 128:192])
    assert torch.equal(stack_rows([q.rows(0, 8), q.rows(40, 48)]).dequantize(), torch.cat((d[0:8], d[40:48])))
    with pytest.raises(ValueError):
        NVFP4Tensor.cat_rows([q.rows(0, 8), quantize_nvfp4(w * 2, swizzle=False).rows(0, 8)])   # different scales
    with pytest.raises(ValueError):
        q.cols(0, 32)                                                                          # not a multiple of 64


def test_route_and_sort_groups_pairs_by_local_expert():
    from jetspec_b200.parallel.ep import route_and_sort
    torch.manual_seed(2)
    T, E, k = 37, 16, 4
    logits = torch.randn(T, E)
    first, n_local = 4, 8
    order, row_w, group_off, counts_all = route_and_sort(logits, k, True, first, n_local)
    wts, idx = ref.moe_route(logits, k, True)
    flat = idx.reshape(-1)
    assert sorted(order.tolist()) == list(range(T * k))                        # a permutation of all pairs
    assert int(counts_all.sum()) == T * k and torch.equal(counts_all, torch.bincount(flat, minlength=E))
    for e in range(n_local):
        rows = order[int(group_off[e]):int(group_off[e + 1])]
        assert bool((flat[rows] == first + e).all())
        assert rows.tolist() == sorted(rows.tolist())                          # stable: pair order kept inside a group
    tail = order[int(group_off[n_local]):]
    assert bool(((flat[tail] < first) | (flat[tail] >= first + n_local)).all())
    assert torch.allclose(row_w, wts.reshape(-1)[order])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_layer_worker(rank: int, world: int, port: int, out_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = tiny_config()
        model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.float32)          # same seed: replicas
        layer = model.model.layers[0]
        T = 6
        x = torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(3))
        pos = torch.arange(T)
        Hq, Hkv, D = cfg.num_attention_heads // world, cfg.num_key_value_heads // world, cfg.head_dim
        att = shard_attention(layer, cfg, rank, world)
        mlp = shard_mlp(layer.mlp, rank, world, lambda g, u: torch.cat((g, u), 0))
        # --- attention block with this rank's heads; the row-parallel o_proj partial is all-reduced
        h = ref.rmsnorm(x, layer.input_layernorm.weight, cfg.rms_norm_eps)
        q, k, v = ref.qkv_postprocess(ref.linear(h, att["qkv"]), att["qn"], att["kn"], pos, Hq, Hkv, D, cfg.rope_theta,
                                      cfg.rms_norm_eps)
        kk, vv = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, kk) / D ** 0.5
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shd->thd", s.softmax(-1), vv).reshape(T, Hq * D)
        part = ref.linear(o, att["o"])
        dist.all_reduce(part)
        x1 = x + part
        # --- MLP with this rank's channels
        h2 = ref.rmsnorm(x1, layer.post_attention_layernorm.weight, cfg.rms_norm_eps)
        I = mlp["gate"].shape[0]
        gu = ref.linear(h2, mlp["gu"])
        act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        part2 = ref.linear(act, mlp["down"])
        dist.all_reduce(part2)
        y = x1 + part2
        if rank == 0:
            torch.save(y, out_path)
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_layer_matches_single_process(tmp_path):
    cfg = tiny_config()
    if cfg.num_key_value_heads % 2:
        pytest.skip("tiny config cannot split its KV heads over two ranks")
    out_path = str(tmp_path / "tp.pt")
    mp.spawn(_tp_layer_worker, args=(2, _free_port(), out_path), nprocs=2, join=True)
    got = torch.load(out_path)
    # single process: the full layer through the model's own forward
    model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.float32)
    layer = model.model.layers[0]
    T, D = 6, cfg.head_dim
    x = torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(3))
    pos = torch.arange(T)
    a = layer.self_attn
    h = ref.rmsnorm(x, layer.input_layernorm.weight, cfg.rms_norm_eps)
    qkv = torch.cat((ref.linear(h, a.q_proj.weight), ref.linear(h, a.k_proj.weight), ref.linear(h, a.v_proj.weight)), -1)
    q, k, v = ref.qkv_postprocess(qkv, a.q_norm.weight, a.k_norm.weight, pos, cfg.num_attention_heads,
                                  cfg.num_key_value_heads, D, cfg.rope_theta, cfg.rms_norm_eps)
    g = cfg.num_attention_heads // cfg.num_key_value_heads
    s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(g, 1)) / D ** 0.5
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    o = torch.einsum("hts,shd->thd", s.softmax(-1), v.repeat_interleave(g, 1)).reshape(T, -1)
    x1 = x + ref.linear(o, a.o_proj.weight)
    h2 = ref.rmsnorm(x1, layer.post_attention_layernorm.weight, cfg.rms_norm_eps)
    want = x1 + ref.linear(torch.nn.functional.silu(ref.linear(h2, layer.mlp.gate_proj.weight))
                           * ref.linear(h2, layer.mlp.up_proj.weight), layer.mlp.down_proj.weight)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)


def _dp_stats_worker(rank: int, world: int, port: int, out_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench"))
        from engine_tps import reduce_stats, shard
        bank = list(range(7))
        mine = shard(bank, rank, world)
        st = reduce_stats(tokens=10 * len(mine), wall=1.0 + rank, acc_sum=3.0 * len(mine), rounds=len(mine), world=world)
        if rank == 0:
            torch.save(st, out_path)
    finally:
        dist.destroy_process_group()


def test_data_parallel_reductions_over_gloo(tmp_path):
    out_path = str(tmp_path / "dp.pt")
    mp.spawn(_dp_stats_worker, args=(2, _free_port(), out_path), nprocs=2, join=True)
    st = torch.load(out_path)
    assert st["tokens"] == 70 and st["wall_s"] == 2.0 and abs(st["tps"] - 35.0) < 1e-9 and abs(st["accept_len"] - 3.0) < 1e-9


def test_allreduce_ring_rule_holds_under_any_interleaving():
    """The receive-buffer ring of the fused all-reduce, as an executable model: for every number of collectives
    per graph replay, the cycle length the runtime picks never lets a store land on an unread cell, whatever the
    relative speed of the ranks; a ring of one buffer does, and the model says so."""
    import random
    from jetspec_b200.parallel.tp import AllReduceRingModel, ring_mod_for
    rng = random.Random(0)
    for world in (2, 4, 8):
        for calls in list(range(2, 14)) + [36, 60, 62, 72, 73, 74, 96]:
            mod = ring_mod_for(calls)
            assert calls % mod != 1
            bufs = [c % mod for c in range(calls)] * 4          # four replays of the same graph, back to back
            for trial in range(6):
                m = AllReduceRingModel(world, bufs, two_shot=trial % 2 == 0)
                if trial == 0:
                    m.run(lambda ready: ready[0])                # rank 0 always first
                elif trial == 1:
                    m.run(lambda ready: ready[-1])               # the last rank always first
                else:
                    m.run(lambda ready: rng.choice(ready))
    assert ring_mod_for(1) == 4 and ring_mod_for(61) == 4      # no cycle length helps: covered by the round's barrier
    # eager calls take buffers by call count modulo the same cycle: any cycle of two or more is safe ...
    for two_shot in (True, False):
        AllReduceRingModel(4, [c % 2 for c in range(9)], two_shot).run(lambda ready: rng.choice(ready))
    # ... the two-shot form would even survive a single buffer (nobody can start the next collective before every
    # rank has consumed its first-phase cells), the one-shot form does not: a fast rank's next push meets cells
    # its slow peer has not consumed
    AllReduceRingModel(4, [0] * 6).run(lambda ready: rng.choice(ready))
    import pytest
    with pytest.raises(AssertionError, match="overwrote"):
        for _ in range(50):
            AllReduceRingModel(4, [0] * 6, two_shot=False).run(lambda ready: rng.choice(ready))


def test_ep_slab_layout_is_a_partition():
    """The placement rule of the expert-parallel dispatch: for any count matrix the row ranges that the sources
    write on an owner are disjoint, each expert's rows are contiguous (all sources, in rank order), and together
    they cover exactly the rows the owner's grouped GEMMs run over."""
    import random
    from jetspec_b200.parallel.ep import slab_layout
    rng = random.Random(3)
    for world, n_local in ((2, 4), (4, 2), (8, 16)):
        E = world * n_local
        for _ in range(10):
            counts = [[rng.choice([0, 0, 1, 3, 17, 64]) for _ in range(E)] for _ in range(world)]
            base, group_off = slab_layout(counts, n_local)
            for owner in range(world):
                covered = []
                for le in range(n_local):
                    e = owner * n_local + le
                    lo = group_off[owner][le]
                    for src in range(world):
                        assert base[src][e] == lo                      # sources follow each other inside the expert
                        covered.append((lo, lo + counts[src][e]))
                        lo += counts[src][e]
                    assert lo == group_off[owner][le + 1]
                covered = [c for c in covered if c[1] > c[0]]
                assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))      # no gap, no overlap
                total = sum(counts[s][owner * n_local + le] for s in range(world) for le in range(n_local))
                assert group_off[owner][n_local] == total
