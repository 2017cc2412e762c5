"""Worker for the multi-GPU tests (launched by torch.distributed.run, one rank per GPU).

Checks the fused row-parallel GEMM + all-reduce and the vocabulary-parallel argmax against their
unfused NCCL twins, then (optionally) a tensor-parallel tree decode against the single-GPU engine.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def disagg_main(rank):
    """Target on rank 0, draft head on rank 1: the remote head must reproduce the local head's rounds."""
    from jetspec_b200 import JetSpecEngine, SamplingParams, DraftHeadTreeDrafter
    from jetspec_b200.engine.disagg import DraftWorker, RemoteDraftHead
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config, DraftHeadModel, draft_head_config
    from jetspec_b200.parallel.handoff import HandoffChannel
    cfg = Qwen3Config(vocab_size=8192, hidden_size=1024, intermediate_size=2048, num_hidden_layers=4,
                      num_attention_heads=8, num_key_value_heads=8, head_dim=128)
    model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.bfloat16, device="cuda", init="stable")
    taps, D, K, budget = [0, 1, 3], 8, 4, 32
    hcfg = draft_head_config(cfg, num_layers=1, block_size=D + 1, target_layer_ids=taps)
    head = DraftHeadModel.random_init(hcfg, seed=5, dtype=torch.bfloat16, device="cuda")
    chan = HandoffChannel(None, nodes=32, tap_width=len(taps) * cfg.hidden_size, depth=D, width=K)
    ok = True
    if rank == 0:
        prompt = torch.randint(0, cfg.vocab_size, (1, 40), generator=torch.Generator().manual_seed(0))
        sp = SamplingParams(0.0, 40)
        eng = JetSpecEngine(model, device="cuda:0", dtype=torch.bfloat16, max_seq_len=512)
        local = eng.generate_tree(prompt, DraftHeadTreeDrafter(head, model, block_size=D + 1), tree_depth=D, tree_width=K,
                                  budget=budget, sampling_params=sp, return_stats=True)
        remote = eng.generate_tree(prompt, RemoteDraftHead(chan, taps, D + 1), tree_depth=D, tree_width=K,
                                   budget=budget, sampling_params=sp, return_stats=True)
        ok = (remote["token_ids"] == local["token_ids"] and remote["accept_lengths"] == local["accept_lengths"]
              and remote["tree_sizes"] == local["tree_sizes"])
        print(f"disaggregated drafting: tokens equal {remote['token_ids'] == local['token_ids']}, "
              f"rounds {remote['rounds']} vs {local['rounds']}, same trees {remote['tree_sizes'] == local['tree_sizes']}", flush=True)
    else:
        worker = DraftWorker(head, model.model.embed_tokens.weight, model.lm_head.weight, chan, width=K,
                             vocab_size=cfg.vocab_size, max_ctx=512)
        steps = worker.serve()
        print(f"draft worker served {steps} steps", flush=True)
    from jetspec_b200.ops import cuda_ext as X
    X.check_status("cuda")
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_WORKER_OK" if int(flag) == 1 else "TP_WORKER_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


def ep_engine_main(rank, world):
    """Expert-parallel engine: every rank decodes its OWN request (different prompt, different drafter, hence a
    different number of rounds) while the experts are sharded; each rank's tokens must equal what a one-GPU
    engine produces for that request."""
    from jetspec_b200 import JetSpecEngine, SamplingParams, RandomTreeDrafter, OracleTreeDrafter
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config
    from jetspec_b200.parallel import TokenShardedEP
    from jetspec_b200.ops import cuda_ext as X
    cfg = Qwen3Config(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=3,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128, num_experts=8,
                      num_experts_per_tok=2, moe_intermediate_size=256, norm_topk_prob=True, model_type="qwen3_moe")
    model = Qwen3ForCausalLM.random_init(cfg, seed=2, dtype=torch.bfloat16, device="cuda", init="stable")
    dev = f"cuda:{torch.cuda.current_device()}"
    prompt = torch.randint(0, cfg.vocab_size, (1, 20 + 9 * rank), generator=torch.Generator().manual_seed(rank))
    sp = SamplingParams(0.0, 24 + 4 * rank)                    # ranks finish at different times
    solo = JetSpecEngine(model, device=dev, dtype=torch.bfloat16, max_seq_len=512)
    want = solo.generate(prompt, sp)["token_ids"]
    ep = TokenShardedEP(None, cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, max_tokens=128)
    eng = JetSpecEngine(model, device=dev, dtype=torch.bfloat16, max_seq_len=512, expert_parallel=ep)
    ar = eng.generate(prompt, sp)["token_ids"]
    rnd = eng.generate_tree(prompt, RandomTreeDrafter(cfg.vocab_size, seed=3 + rank), tree_depth=4, tree_width=2,
                            budget=8, sampling_params=sp, return_stats=True)
    oracle = OracleTreeDrafter(prompt[0].tolist() + want, cfg.vocab_size, tree_width=3, mean_accept=2.0 + rank,
                               max_accept=5, seed=rank)
    orc = eng.generate_tree(prompt, oracle, tree_depth=6, tree_width=3, budget=16, sampling_params=sp, return_stats=True)
    X.check_status("cuda")
    ok = ar == want and rnd["token_ids"] == want and orc["token_ids"] == want
    print(f"[rank {rank}] ep engine: AR ok {ar == want}, random-tree ok {rnd['token_ids'] == want} "
          f"({rnd['rounds']} rounds), oracle-tree ok {orc['token_ids'] == want} ({orc['rounds']} rounds, "
          f"{orc['tpf']:.2f} tokens/round)", flush=True)
    ep.close()
    del eng, solo, model
    torch.cuda.empty_cache()
    ok &= ep_engine_a3b_geometry(rank, world, dev)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_WORKER_OK" if int(flag) == 1 else "TP_WORKER_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


def ep_engine_a3b_geometry(rank, world, dev) -> bool:
    """The same check at the layer geometry of Qwen3-30B-A3B (128 experts, top-8, hidden 2048, expert width 768,
    32 query / 4 KV heads), four layers deep: 128-node trees, a real draft head inside the round graph, an oracle
    script with a different acceptance profile (hence a different number of rounds) on every rank."""
    from jetspec_b200 import JetSpecEngine, SamplingParams, OracleTreeDrafter, OracleOverrideDrafter, DraftHeadTreeDrafter
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config, DraftHeadModel, draft_head_config
    from jetspec_b200.parallel import TokenShardedEP
    from jetspec_b200.ops import cuda_ext as X
    cfg = Qwen3Config(vocab_size=8192, hidden_size=2048, intermediate_size=6144, num_hidden_layers=4,
                      num_attention_heads=32, num_key_value_heads=4, head_dim=128, num_experts=128,
                      num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True, model_type="qwen3_moe")
    model = Qwen3ForCausalLM.random_init(cfg, seed=4, dtype=torch.bfloat16, device="cuda", init="stable")
    head = DraftHeadModel.random_init(draft_head_config(cfg, num_layers=1, block_size=21, num_taps=3), seed=5,
                                      dtype=torch.bfloat16, device="cuda")
    # prompt lengths that need a different number of 128-token prefill chunks on every rank (2 on rank 0, 3 on rank 1,
    # ... 6 on rank 7): the ranks with shorter prompts sit the others' extra chunks out and keep serving their rows
    prompt = torch.randint(0, cfg.vocab_size, (1, 200 + 70 * rank), generator=torch.Generator().manual_seed(10 + rank))
    sp = SamplingParams(0.0, 96)
    want = [(int(prompt[0, -1]) + 1 + i) % cfg.vocab_size for i in range(96)]
    ep = TokenShardedEP(None, cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, max_tokens=128)
    eng = JetSpecEngine(model, device=dev, dtype=torch.bfloat16, max_seq_len=2048, expert_parallel=ep)
    ar = eng.generate(prompt, sp)["token_ids"]
    oracle = OracleTreeDrafter(prompt[0].tolist() + want, cfg.vocab_size, tree_width=7, mean_accept=3.0 + 2 * rank,
                               max_accept=19, seed=rank)
    drafter = OracleOverrideDrafter(DraftHeadTreeDrafter(head, model, block_size=21), oracle)
    out = eng.generate_tree(prompt, drafter, tree_depth=20, tree_width=7, budget=128, sampling_params=sp,
                            return_stats=True, session=True)
    X.check_status("cuda")
    good = ar == want and out["token_ids"] == want
    print(f"[rank {rank}] ep engine, A3B layer geometry: AR ok {ar == want}, tree ok {out['token_ids'] == want} "
          f"({out['rounds']} rounds, {out['tpf']:.2f} tokens/round)", flush=True)
    ep.close()
    return good


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    if len(sys.argv) > 1 and sys.argv[1] == "disagg":
        return disagg_main(rank)
    if len(sys.argv) > 1 and sys.argv[1] == "ep_engine":
        return ep_engine_main(rank, world)
    from jetspec_b200.ops import cuda_ext as X
    from jetspec_b200.parallel import TensorParallel, shard_cols, shard_rows
    X.load()
    tp = TensorParallel(None, m_cap=512, n_max=4096)
    g = torch.Generator(device="cuda").manual_seed(0)       # same seed: every rank builds the full tensors
    ok = True
    for (M, N, K) in [(128, 4096, 4096), (21, 1024, 2048), (300, 512, 1024), (1, 4096, 12288)]:
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
        res = torch.randn(M, N, generator=g, device="cuda").to(torch.bfloat16)
        xl, wl = shard_cols(x, rank, world), shard_cols(w, rank, world)
        for rep in range(6):                                 # several turns of the buffer ring
            out = res.clone()
            tp.gemm_allreduce(xl, wl, out, residual=out)
            torch.cuda.synchronize()
        ref = x.float() @ w.float().t() + res.float()
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        # the same all-reduce with the FOLLOWING RMSNorm computed by its finishing kernel
        nw = (1.0 + 0.1 * torch.randn(N, generator=g, device="cuda")).to(torch.bfloat16)
        out2, h2 = res.clone(), torch.empty_like(res)
        for rep in range(3):
            out2.copy_(res)
            tp.gemm_allreduce(xl, wl, out2, residual=out2, norm_w=nw, norm_out=h2, eps=1e-6)
            torch.cuda.synchronize()
        o32 = out2.float()
        h_ref = o32 * torch.rsqrt(o32.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        err_n = float((h2.float() - h_ref).abs().max() / h_ref.abs().max())
        same_x = torch.equal(out2, out)
        base = torch.empty_like(res)
        tp.gemm_allreduce_nccl(xl, wl, base, residual=res)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], t) for t in gathered)      # replicas must be bit-identical
        dist.all_gather(gathered, h2)
        same &= all(torch.equal(gathered[0], t) for t in gathered)
        if rank == 0:
            print(f"gemm_allreduce[{tp.mode}] M={M} N={N} K={K}: rel err {err:.2e}, fused norm err {err_n:.2e}, "
                  f"same residual {same_x}, replicas identical {same}", flush=True)
        ok &= err < 1.5e-2 and err_n < 1.5e-2 and same and same_x
    # vocabulary-parallel argmax
    M, V, H = 128, 8192, 512
    h = torch.randn(M, H, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(V, H, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    wl = shard_rows(w, rank, world)
    nt = X.n_tiles(wl.shape[0])
    ws = {"val": torch.empty(M, nt, dtype=torch.float32, device="cuda"), "idx": torch.empty(M, nt, dtype=torch.int32, device="cuda")}
    out_idx = torch.empty(M, dtype=torch.int32, device="cuda")
    for _ in range(3):
        tp.lm_head_argmax(h, wl, rank * (V // world), ws, out_idx)
        torch.cuda.synchronize()
    logits = h.float() @ w.float().t()
    chosen = logits.gather(1, out_idx.long()[:, None]).squeeze(1)
    gap = float((logits.max(-1).values - chosen).max())
    if rank == 0:
        print(f"tp argmax: worst shortfall {gap:.3e}", flush=True)
    ok &= gap < 0.05
    # vocabulary-parallel top-k with full-vocabulary log-probabilities (the draft head's logits)
    Mt, Kt = 20, 7
    ht = h[:Mt].contiguous()
    tk_ws = {"val": torch.empty(Mt, nt, 8, dtype=torch.float32, device="cuda"),
             "idx": torch.empty(Mt, nt, 8, dtype=torch.int32, device="cuda"),
             "lse": torch.empty(Mt, nt, 2, dtype=torch.float32, device="cuda")}
    o_tok = torch.empty(Mt, Kt, dtype=torch.int32, device="cuda")
    o_lp = torch.empty(Mt, Kt, dtype=torch.float32, device="cuda")
    for _ in range(3):
        tp.lm_head_topk_logprobs(ht, wl, rank * (V // world), Kt, tk_ws, o_tok, o_lp)
        torch.cuda.synchronize()
    lsm = torch.log_softmax(logits[:Mt], -1)
    ref_lp, ref_tok = lsm.topk(Kt, -1)
    lp_err = float((o_lp - lsm.gather(1, o_tok.long())).abs().max())          # the reported log-prob is the token's own
    short = float((ref_lp - o_lp).abs().max())                                 # and the k-th best is as good as the true one
    gathered = [torch.empty_like(o_tok) for _ in range(world)]
    dist.all_gather(gathered, o_tok)
    same_t = all(torch.equal(gathered[0], t) for t in gathered)
    if rank == 0:
        print(f"tp top-k: log-prob err {lp_err:.3e}, shortfall vs exact top-k {short:.3e}, replicas identical {same_t}",
              flush=True)
    ok &= lp_err < 2e-2 and short < 2e-2 and same_t
    ok &= ep_check(rank, world)
    ok &= ep_dispatch_check(rank, world)
    ok &= nvfp4_check(tp, rank, world)
    X.check_status("cuda")
    if len(sys.argv) > 1 and sys.argv[1] == "engine":
        ok &= engine_check(tp, rank, world)
        if (1024 // world) % 256 == 0:          # the 4-bit GEMM wants K-slices that are multiples of 256
            ok &= engine_check(tp, rank, world, nvfp4=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_WORKER_OK" if int(flag) == 1 else "TP_WORKER_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


def ep_check(rank, world) -> bool:
    """Fused expert-parallel MoE layer against its NCCL twin and the single-device reference."""
    from jetspec_b200.parallel.ep import ExpertParallel
    from jetspec_b200.ops import reference as ref
    E, H, I, k, T = 16, 512, 128, 4, 96
    g = torch.Generator(device="cuda").manual_seed(7)
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).to(torch.bfloat16)
    x, gate = bf(T, H), bf(E, H, sc=0.5)
    wgu, wd = bf(E, 2 * I, H, sc=0.06), bf(E, H, I, sc=0.06)
    logits = x.float() @ gate.float().t()
    ep = ExpertParallel(None, E, k, H, max_tokens=128)
    gu_l, dn_l = ep.shard(wgu, wd)
    good = True
    for _ in range(4):                                   # several turns of the buffer ring
        out = ep.moe_layer(x, gate, gu_l, dn_l, True, router_logits=logits)
        torch.cuda.synchronize()
    exp = x.float() + ref.moe_forward(x.float(), gate.float(), wgu.float(), wd.float(), k, True, router_logits=logits)
    base = ep.moe_layer_nccl(x, gate, wgu, wd, True, router_logits=logits)
    err = float((out.float() - exp).abs().max() / exp.abs().max())
    err_b = float((base.float() - exp).abs().max() / exp.abs().max())
    twin = ep.moe_layer_grouped_nccl(x, gate, gu_l, dn_l, True, router_logits=logits)
    err_b = max(err_b, float((twin.float() - exp).abs().max() / exp.abs().max()))
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    same = all(torch.equal(gathered[0], t) for t in gathered)
    if rank == 0:
        print(f"ep moe layer: rel err {err:.2e} (nccl twin {err_b:.2e}), replicas identical {same}", flush=True)
    return err < 2e-2 and err_b < 2e-2 and same


def ep_dispatch_check(rank, world) -> bool:
    """Token-sharded expert parallelism: every rank brings its OWN tokens (different counts per rank, one rank
    idle in one of the rounds); results against the single-device reference on those tokens."""
    from jetspec_b200.parallel.ep import TokenShardedEP
    from jetspec_b200.ops import reference as ref
    E, H, I, k = 16, 512, 128, 4
    g = torch.Generator(device="cuda").manual_seed(21)            # same seed: every rank builds the full weights
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).to(torch.bfloat16)
    gate, wgu, wd = bf(E, H, sc=0.5), bf(E, 2 * I, H, sc=0.06), bf(E, H, I, sc=0.06)
    nw = (1.0 + 0.1 * torch.randn(H, generator=g, device="cuda")).to(torch.bfloat16)
    ep = TokenShardedEP(None, E, k, H, max_tokens=128)
    gu_l, dn_l = ep.shard(wgu, wd)
    good = True
    worst = 0.0
    for rnd in range(5):                                          # several turns of the buffer rings
        T = [96, 37, 128, 1, 64, 80, 5, 100][(rank + rnd) % 8]
        idle = rnd == 2 and rank == world - 1                     # one rank sits a round out
        gl = torch.Generator(device="cuda").manual_seed(100 * rnd + rank)
        x = torch.randn(T, H, generator=gl, device="cuda").to(torch.bfloat16)
        hn = torch.randn(T, H, generator=gl, device="cuda").to(torch.bfloat16)
        if idle:
            ep.idle_layer(gate, gu_l, dn_l, True)
            torch.cuda.synchronize()
            continue
        out, h2 = torch.empty_like(x), torch.empty_like(x)
        ep.moe_layer(x, hn, gate, gu_l, dn_l, True, out=out, norm_w=nw, norm_out=h2, eps=1e-6)
        torch.cuda.synchronize()
        logits = hn.float() @ gate.float().t()
        exp = x.float() + ref.moe_forward(hn.float(), gate.float(), wgu.float(), wd.float(), k, True, router_logits=logits)
        err = float((out.float() - exp).abs().max() / exp.abs().max())
        o32 = out.float()
        h_ref = o32 * torch.rsqrt(o32.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        err_n = float((h2.float() - h_ref).abs().max() / h_ref.abs().max())
        worst = max(worst, err, err_n)
        good &= err < 2e-2 and err_n < 2e-2
    from jetspec_b200.ops import cuda_ext as X
    X.check_status("cuda")
    flag = torch.tensor([worst], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"ep token-sharded dispatch: worst rel err over ranks and rounds {float(flag):.2e}", flush=True)
    ep.close()
    return good


def nvfp4_check(tp, rank, world) -> bool:
    """Row-parallel NVFP4 GEMM fused with the all-reduce against the dequantised per-rank products."""
    from jetspec_b200.ops import cuda_ext as X
    from jetspec_b200.models.nvfp4 import quantize_nvfp4, nvfp4_linear_reference
    from jetspec_b200.parallel import shard_cols
    g = torch.Generator(device="cuda").manual_seed(11)
    good = True
    for (M, N, K) in [(128, 4096, 4096), (21, 1024, 2048), (1, 4096, 12288 // 2 * 2)]:
        if (K // world) % 256:
            continue
        x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
        res = torch.randn(M, N, generator=g, device="cuda").to(torch.bfloat16)
        qw = quantize_nvfp4(w.float(), swizzle=False)
        ql = shard_cols(qw, rank, world)
        xl = shard_cols(x, rank, world)
        for rep_ in range(5):
            out = res.clone()
            tp.gemm_allreduce_nvfp4(X.quant_nvfp4(xl), ql, out, residual=out)
            torch.cuda.synchronize()
        part = nvfp4_linear_reference(xl, ql)
        dist.all_reduce(part)
        ref = part + res.float()
        err = float((out.float() - ref).abs().max() / ref.abs().max())
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        if rank == 0:
            print(f"nvfp4 gemm_allreduce M={M} N={N} K={K}: rel err {err:.2e}, replicas identical {same}", flush=True)
        good &= err < 1.5e-2 and same
    return good


def engine_check(tp, rank, world, nvfp4: bool = False) -> bool:
    from jetspec_b200 import JetSpecEngine, SamplingParams, OracleTreeDrafter
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config
    cfg = Qwen3Config(vocab_size=8192, hidden_size=1024, intermediate_size=2048, num_hidden_layers=4,
                      num_attention_heads=8, num_key_value_heads=8, head_dim=128)
    model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.bfloat16, device="cuda", init="stable")
    if nvfp4:
        from jetspec_b200.models.nvfp4 import quantize_model_nvfp4
        quantize_model_nvfp4(model)
    prompt = torch.randint(0, cfg.vocab_size, (1, 40), generator=torch.Generator().manual_seed(0))
    sp = SamplingParams(0.0, 48)
    eng = JetSpecEngine(model, device=f"cuda:{torch.cuda.current_device()}", dtype=torch.bfloat16, max_seq_len=512,
                        tensor_parallel=tp)
    ar = eng.generate(prompt, sp)["token_ids"]
    expect = [(int(prompt[0, -1]) + 1 + i) % cfg.vocab_size for i in range(48)]   # the stable init counts upwards
    oracle = OracleTreeDrafter(prompt[0].tolist() + ar, cfg.vocab_size, tree_width=4, mean_accept=3.0, max_accept=7, seed=1)
    out = eng.generate_tree(prompt, oracle, tree_depth=8, tree_width=4, budget=32, sampling_params=sp, return_stats=True)
    good = ar == expect and out["token_ids"] == expect and out["tpf"] > 2.0
    if rank == 0:
        print(f"tp engine{' (nvfp4)' if nvfp4 else ''}: AR ok {ar == expect}, tree ok {out['token_ids'] == expect}, tokens/round {out['tpf']:.2f}", flush=True)
    if not nvfp4:
        # a real draft head inside the round graph (vocabulary-parallel top-k) and continuous batching through the
        # sharded stack: every request must reproduce the counting sequence
        from jetspec_b200 import DraftHeadTreeDrafter, RandomTreeDrafter
        from jetspec_b200.models import DraftHeadModel, draft_head_config
        hcfg = draft_head_config(cfg, num_layers=1, block_size=9, num_taps=3)
        head = DraftHeadModel.random_init(hcfg, seed=5, dtype=torch.bfloat16, device="cuda")
        hout = eng.generate_tree(prompt, DraftHeadTreeDrafter(head, model, block_size=9), tree_depth=8, tree_width=4,
                                 budget=32, sampling_params=sp, return_stats=True)
        good &= hout["token_ids"] == expect
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, cfg.vocab_size, (1, n), generator=g) for n in (17, 40, 9)]
        sp2 = SamplingParams(0.0, 20)
        want = [[(int(p[0, -1]) + 1 + i) % cfg.vocab_size for i in range(20)] for p in prompts]
        bouts = eng.generate_tree_batch(prompts, RandomTreeDrafter(cfg.vocab_size, seed=7), block_size=5, tree_width=3,
                                        budget=16, sampling_params=sp2)
        b_ok = [o["token_ids"] for o in bouts] == want
        a_ok = [o["token_ids"] for o in eng.generate_batch(prompts, sp2)] == want
        if rank == 0:
            print(f"tp engine: in-graph head ok {hout['token_ids'] == expect}, tree batch ok {b_ok}, AR batch ok {a_ok}",
                  flush=True)
        good &= b_ok and a_ok
    return good


if __name__ == "__main__":
    main()
