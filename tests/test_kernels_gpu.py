"""Numerics of every sm_100a kernel against the plain PyTorch fp32 reference of the same op."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_TOL = 8e-3   # the tolerance the reference engine uses for its bf16 kernel gate


@pytest.fixture(scope="module")
def ext():
    from jetspec_b200.ops import cuda_ext
    cuda_ext.load()
    yield cuda_ext
    cuda_ext.check_status("cuda")


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-6))


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 512, 1024), (21, 384, 512), (300, 256, 2048), (1, 1024, 4096)])
@pytest.mark.parametrize("split", [1, 2, 3, 4])
@pytest.mark.parametrize("deep", [False, True])
def test_gemm_store(ext, M, N, K, split, deep):
    x, w = rnd(M, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    ref = x.float() @ w.float().t()
    out = ext.gemm(x, w, split=split, deep=deep)
    torch.cuda.synchronize()
    assert rel_err(out, ref) < BF16_TOL
    ext.check_status("cuda")


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths_and_residual(ext, bn):
    x, w, r = rnd(100, 768, seed=3), rnd(1024, 768, scale=0.05, seed=4), rnd(100, 1024, seed=5)
    ref = x.float() @ w.float().t() + r.float()
    out = r.clone()
    ext.gemm(x, w, out=out, residual=out, bn=bn, split=2)   # in place on the residual stream
    torch.cuda.synchronize()
    assert rel_err(out, ref) < BF16_TOL


def test_gemm_many_row_tiles_picks_wide_tiles(ext):
    """Many row tiles (prefill, batched verify): the picker switches to 128x256 tiles with the deep pipeline
    as long as that still leaves at least 64 CTAs."""
    M, N, K = 2000, 1024, 512
    assert ext.pick_gemm_config(M, N, K, ext.EPI_STORE) == (256, 1, 1)
    assert ext.pick_gemm_config(512, 1024, K, ext.EPI_STORE)[0] == 128
    x, w, r = rnd(M, K, seed=3), rnd(N, K, scale=0.05, seed=4), rnd(M, N, seed=5)
    out = ext.gemm(x, w, residual=r)
    torch.cuda.synchronize()
    assert rel_err(out, x.float() @ w.float().t() + r.float()) < BF16_TOL
    ext.check_status("cuda")


@pytest.mark.parametrize("M", [2048, 1000, 257, 129, 128])
def test_gemm_two_row_tiles_per_cta(ext, M):
    """deep = 3: one CTA computes two 128-row tiles (two accumulators) from every weight stage; row counts that leave
    the second tile partly or wholly empty, store (+ residual) and SwiGLU epilogues."""
    N, K = 1024, 768
    x, w, r = rnd(M, K, seed=3), rnd(N, K, scale=0.05, seed=4), rnd(M, N, seed=5)
    out = ext.gemm(x, w, residual=r, bn=256, split=1, deep=3)
    torch.cuda.synchronize()
    assert rel_err(out, x.float() @ w.float().t() + r.float()) < BF16_TOL
    g, u = w[: N // 2], w[N // 2:]
    act = ext.gemm(x, ext.interleave_gate_up(g, u, 256), epi=ext.EPI_SWIGLU, bn=256, split=1, deep=3)
    torch.cuda.synchronize()
    ref = torch.nn.functional.silu(x.float() @ g.float().t()) * (x.float() @ u.float().t())
    assert rel_err(act, ref) < BF16_TOL
    ext.check_status("cuda")
    assert ext.pick_gemm_config(2048, 4096, 4096, ext.EPI_STORE) == (256, 1, 3)     # 128 CTAs, one wave
    assert ext.pick_gemm_config(2048, 6144, 4096, ext.EPI_STORE) == (256, 1, 1)     # would be two waves of big tiles


def test_gemm_fp32_out(ext):
    x, w = rnd(64, 512, seed=6), rnd(128, 512, scale=0.05, seed=7)
    out = ext.gemm(x, w, epi=ext.EPI_STORE_F32, split=2)
    assert rel_err(out, x.float() @ w.float().t()) < 1e-4


@pytest.mark.parametrize("split", [1, 2, 4])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_swiglu(ext, split, bn):
    M, H, I = 77, 512, 1024
    x, g, u = rnd(M, H, seed=8), rnd(I, H, scale=0.05, seed=9), rnd(I, H, scale=0.05, seed=10)
    w = ext.interleave_gate_up(g, u, bn)
    ref = torch.nn.functional.silu(x.float() @ g.float().t()) * (x.float() @ u.float().t())
    out = ext.gemm(x, w, epi=ext.EPI_SWIGLU, bn=bn, split=split)
    torch.cuda.synchronize()
    assert rel_err(out, ref) < BF16_TOL


@pytest.mark.parametrize("split", [1, 2])
def test_gemm_swiglu_192_column_tiles(ext, split):
    """The 192-column tile (96 gate + 96 up columns): one even wave for a 24576-wide gate/up (opt-in, measured slower)."""
    M, H, I = 128, 512, 1152
    x, g, u = rnd(M, H, seed=8), rnd(I, H, scale=0.05, seed=9), rnd(I, H, scale=0.05, seed=10)
    w = ext.interleave_gate_up(g, u, 192)
    ref = torch.nn.functional.silu(x.float() @ g.float().t()) * (x.float() @ u.float().t())
    for deep in (0, 1):
        out = ext.gemm(x, w, epi=ext.EPI_SWIGLU, bn=192, split=split, deep=deep)
        torch.cuda.synchronize()
        assert rel_err(out, ref) < BF16_TOL


def test_lm_head_argmax(ext):
    M, V, H = 128, 5000, 512       # V not a multiple of the tile width
    h, w = rnd(M, H, seed=11), rnd(V, H, scale=0.05, seed=12)
    idx, val = ext.lm_head_argmax(h, w)
    logits = (h.float() @ w.float().t())
    ref_val, ref_idx = logits.max(-1)
    torch.cuda.synchronize()
    # bf16 rounding of the logits can reorder near-ties: require the chosen logit to be within tolerance of the max
    chosen = logits.gather(1, idx.long()[:, None]).squeeze(1)
    assert float((ref_val - chosen).max()) < BF16_TOL * float(ref_val.abs().max())
    assert float((idx.long() == ref_idx).float().mean()) > 0.95


@pytest.mark.parametrize("M", [20, 32, 100])      # <= 32 rows: the shared-memory epilogue; more: one thread per row
def test_lm_head_topk_logprobs(ext, M):
    V, H, K = 5000, 512, 7
    h, w = rnd(M, H, seed=13), rnd(V, H, scale=0.08, seed=14)
    tok, lp = ext.lm_head_topk_logprobs(h, w, K)
    ref_lp_all = torch.log_softmax(h.float() @ w.float().t(), -1)
    ref_lp, ref_tok = torch.topk(ref_lp_all, K, -1)
    torch.cuda.synchronize()
    assert torch.allclose(lp, ref_lp, atol=2e-3, rtol=0)
    assert float((tok.long() == ref_tok).float().mean()) > 0.97
    # every returned log-prob is the true log-prob of the returned token
    assert torch.allclose(lp, ref_lp_all.gather(1, tok.long()), atol=2e-3, rtol=0)


@pytest.mark.parametrize("M", [1, 21, 32])
def test_lm_head_topk_two_pass_matches_epilogue(ext, M, monkeypatch):
    """Few rows over a vocabulary of many tiles: logits stored by the fp32 epilogue + slice pass + merge against the
    in-epilogue top-k and against the fp32 reference (a vocabulary that is not a multiple of the slice width)."""
    V, H, K = 20004, 512, 8
    h, w = rnd(M, H, seed=13), rnd(V, H, scale=0.08, seed=14)
    assert ext.TOPK_TWO_PASS and M <= ext.TOPK_TWO_PASS_ROWS and ext.n_tiles(V) >= ext.TOPK_SLICES
    tok2, lp2 = ext.lm_head_topk_logprobs(h, w, K)
    monkeypatch.setattr(ext, "TOPK_TWO_PASS", False)
    tok1, lp1 = ext.lm_head_topk_logprobs(h, w, K)
    torch.cuda.synchronize()
    assert torch.equal(tok1, tok2)                       # same fp32 accumulators, same order and tie-break
    assert torch.allclose(lp1, lp2, atol=1e-5, rtol=0)
    ref_lp_all = torch.log_softmax(h.float() @ w.float().t(), -1)
    assert torch.allclose(lp2, ref_lp_all.gather(1, tok2.long()), atol=2e-3, rtol=0)
    assert torch.allclose(lp2, torch.topk(ref_lp_all, K, -1).values, atol=2e-3, rtol=0)
    ext.check_status("cuda")


def test_elementwise(ext):
    from jetspec_b200.ops import reference as ref
    x, w = rnd(37, 4096, seed=15), rnd(4096, seed=16)
    assert rel_err(ext.rmsnorm(x, w, 1e-6), ref.rmsnorm(x.float(), w.float(), 1e-6)) < BF16_TOL
    gu = rnd(19, 2048, seed=17)
    assert rel_err(ext.silu_mul(gu), ref.silu_mul(gu.float())) < BF16_TOL
    table = rnd(1000, 256, seed=18)
    ids = torch.randint(0, 1000, (33,), device="cuda", dtype=torch.int32)
    assert torch.equal(ext.embed(ids, table), table[ids.long()])
    dst = torch.zeros(8, 512, dtype=torch.bfloat16, device="cuda")
    idx = torch.tensor([5, 1, 1, 30, 2, 0, 0, 0], dtype=torch.int32, device="cuda")
    nv = torch.tensor([5], dtype=torch.int32, device="cuda")
    ext.gather_rows(table, idx, dst, dst_col0=256, n_valid=nv)
    assert torch.equal(dst[:5, 256:], table[idx[:5].long()]) and float(dst[5:].abs().sum()) == 0 and float(dst[:, :256].abs().sum()) == 0


def test_qkv_post(ext):
    from jetspec_b200.ops import reference as ref
    T, Hq, Hkv, D, S = 23, 8, 2, 128, 64
    qkv = rnd(T, (Hq + 2 * Hkv) * D, seed=19)
    qw, kw = rnd(D, seed=20).abs() + 0.5, rnd(D, seed=21).abs() + 0.5
    pos = torch.randint(0, 30000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(S, device="cuda")[:T].to(torch.int32)
    kp = torch.zeros(Hkv, S, D, dtype=torch.bfloat16, device="cuda")
    vp = torch.zeros_like(kp)
    q = torch.empty(T, Hq, D, dtype=torch.bfloat16, device="cuda")
    ext.qkv_post(qkv, qw, kw, pos, slots, ext.inv_freq(D, 1e6, "cuda"), q, kp, vp, Hq, Hkv, 1e-6)
    rq, rk, rv = ref.qkv_postprocess(qkv.float(), qw.float(), kw.float(), pos.long(), Hq, Hkv, D, 1e6, 1e-6)
    torch.cuda.synchronize()
    assert rel_err(q, rq) < 2 * BF16_TOL
    assert rel_err(kp[:, slots.long()].transpose(0, 1), rk) < 2 * BF16_TOL
    assert torch.equal(vp[:, slots.long()].transpose(0, 1), qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D))


def _random_tree_bits(n, words, rng):
    from jetspec_b200.tree.ancestor import ancestor_bits_np
    import numpy as np
    parents = [-1] + [rng.randrange(i) for i in range(1, n)]
    return torch.from_numpy(ancestor_bits_np(parents, n, words).view(np.int32))


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (8, 1), (4, 4)])
# the tcgen05 kernel merges 2..8 key splits inside a cluster (with 8, some splits of the short sequences own no key
# tile at all); 12 takes the separate merge launch
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 6, 8, 12])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("impl", ["mma", "tc"])
def test_paged_tree_attention(ext, Hq, Hkv, splits, causal, impl):
    from jetspec_b200.ops import reference as ref
    rng = random.Random(7)
    D, S, max_len = 128, 4096, 1024
    pasts, ns = [300, 0, 77], [40, 9, 130]
    B, T = len(ns), sum(ns)
    kp, vp = rnd(Hkv, S, D, seed=22), rnd(Hkv, S, D, seed=23)
    q = rnd(T, Hq, D, seed=24)
    slot_map = torch.zeros(4, max_len, dtype=torch.int32, device="cuda")
    perm = torch.randperm(S, device="cuda").to(torch.int32)
    off = 0
    rows = [2, 0, 3]
    for b in range(B):
        L = pasts[b] + ns[b]
        slot_map[rows[b], :L] = perm[off:off + L]
        off += L
    cu = torch.tensor([0] + list(torch.tensor(ns).cumsum(0)), dtype=torch.int32, device="cuda")
    W = 5
    bits = None
    if not causal:
        bits = torch.zeros(T, W, dtype=torch.int32)
        s = 0
        for n in ns:
            bits[s:s + n] = _random_tree_bits(n, W, rng)
            s += n
        bits = bits.cuda()
    seq_rows = torch.tensor(rows, dtype=torch.int32, device="cuda")
    past = torch.tensor(pasts, dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    out = ext.paged_tree_attention(q, kp, vp, slot_map, seq_rows, cu, past, bits, scale, causal, max(ns), splits=splits,
                                   impl=impl)
    exp = ref.paged_tree_attention(q.float(), kp.float(), vp.float(), slot_map, seq_rows, cu, past, bits, scale, causal)
    torch.cuda.synchronize()
    assert rel_err(out, exp) < BF16_TOL
    ext.check_status("cuda")


@pytest.mark.parametrize("seed", range(4))
def test_device_tree_build_and_accept_match_host(ext, seed):
    import ctypes
    from jetspec_b200.tree.builder import build_with_per_depth_cap
    from jetspec_b200.tree import gpu_tree_accept
    from jetspec_b200.tree.ancestor import ancestor_bits_np
    rng = random.Random(seed)
    D, K, budget, NB, W = 20, 7, rng.choice([128, 100, 37]), 128, 4
    toks = [[rng.randrange(50) for _ in range(K)] for _ in range(D)]      # small vocabulary: duplicates happen
    lps = [sorted([-rng.random() * 4 for _ in range(K)], reverse=True) for _ in range(D)]
    lps = torch.tensor(lps, dtype=torch.float32).tolist()                 # fp32-representable, as the device sees them
    caps = [rng.randint(1, K) for _ in range(D)]
    past, max_len = 50, 512
    host = build_with_per_depth_cap(11, toks, lps, caps, budget, "cpu")
    dev = "cuda"
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    committed = torch.zeros(max_len, dtype=torch.int32, device=dev)
    committed[past] = 11
    state = i32([past, 0, 0, 0, 0, 0, 0, 0])
    slot_row = torch.randperm(max_len, device=dev).to(torch.int32)
    slot_before = slot_row.clone()
    o = {k: torch.zeros(NB, dtype=torch.int32, device=dev) for k in ("tok", "par", "dep", "pos", "slot")}
    bits = torch.zeros(NB, W, dtype=torch.int32, device=dev)
    lib = ext.load()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ext.status_word(dev)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tk, lp, cp = i32(toks), torch.tensor(lps, dtype=torch.float32, device=dev), i32(caps)
    zero = i32([0])
    assert lib.js_tree_build(p(tk), p(lp), p(cp), D, K, budget, NB, W, p(committed), p(state), p(slot_row), p(zero), max_len,
                             p(o["tok"]), p(o["par"]), p(o["dep"]), p(o["pos"]), p(o["slot"]), p(bits), p(st), 0, s) == 0
    torch.cuda.synchronize()
    n = host.num_nodes
    assert int(state[5]) == n
    assert o["tok"][:n].tolist() == host.token_ids.tolist()
    assert o["par"][:n].tolist() == host.parent_indices.tolist()
    assert o["dep"][:n].tolist() == host.depth.tolist()
    assert o["pos"][:n].tolist() == (past + host.depth).tolist()
    assert torch.equal(o["slot"], slot_row[past:past + NB])
    import numpy as np
    exp_bits = torch.from_numpy(ancestor_bits_np(host.parent_indices.tolist(), n, W).view(np.int32))
    assert torch.equal(bits[:n].cpu(), exp_bits)
    # accept + commit against the host implementation
    greedy = torch.tensor([rng.randrange(50) for _ in range(NB)], dtype=torch.int32, device=dev)
    path_h, acc_h, corr_h = gpu_tree_accept(host.token_ids, greedy[:n].cpu().long(), host.parent_indices, host.depth,
                                            max_depth=D)
    path_idx = torch.zeros(64, dtype=torch.int32, device=dev)
    result = torch.zeros(64, dtype=torch.int32, device=dev)
    eos = i32([49])
    assert lib.js_tree_accept_commit(p(o["tok"]), p(o["par"]), p(o["dep"]), p(greedy), NB, p(state), p(slot_row),
                                     p(zero), max_len, p(committed), max_len, p(eos), 1, 1000, p(path_idx), p(result),
                                     p(st), 0, s) == 0
    torch.cuda.synchronize()
    assert int(result[0]) == acc_h and int(result[1]) == int(corr_h)
    assert path_idx[:acc_h + 1].tolist() == path_h.tolist()
    new_tokens = host.token_ids[path_h[1:]].tolist() + [int(corr_h)]
    assert committed[past + 1:past + 2 + acc_h].tolist() == new_tokens
    assert int(state[0]) == past + acc_h + 1
    # the window is a permutation with the accepted nodes' slots first
    win_before, win_after = slot_before[past:past + NB], slot_row[past:past + NB]
    assert sorted(win_before.tolist()) == sorted(win_after.tolist())
    assert win_after[:acc_h + 1].tolist() == win_before[path_h].tolist()
    assert torch.equal(slot_row[:past], slot_before[:past]) and torch.equal(slot_row[past + NB:], slot_before[past + NB:])
    ext.check_status(dev)


@pytest.mark.parametrize("T", [5, 200])
def test_grouped_moe_matches_reference(ext, T):
    from jetspec_b200.ops import reference as ref
    E, H, I, k = 16, 256, 128, 4
    x = rnd(T, H, seed=30)
    gate = rnd(E, H, scale=0.5, seed=31)
    wgu, wd = rnd(E, 2 * I, H, scale=0.06, seed=32), rnd(E, H, I, scale=0.06, seed=33)
    logits = (x.float() @ gate.float().t())            # same routing for both sides
    out = ext.moe_forward(x, gate, wgu, wd, k, True, router_logits=logits)
    exp = ref.moe_forward(x.float(), gate.float(), wgu.float(), wd.float(), k, True, router_logits=logits)
    torch.cuda.synchronize()
    assert rel_err(out, exp) < 2 * BF16_TOL
    # residual fused into the combine kernel: exactly the rounding of a separate bf16 add
    res = rnd(T, H, seed=34)
    want = res + out
    got = ext.moe_forward(x, gate, wgu, wd, k, True, router_logits=logits, residual=res)
    torch.cuda.synchronize()
    assert got.data_ptr() == res.data_ptr() and torch.equal(got, want)
    ext.check_status("cuda")


@pytest.mark.parametrize("epi", ["store", "swiglu"])
def test_grouped_gemm_finishes_groups_larger_than_the_launch_covers(ext, epi):
    """The grouped GEMM is launched for ``max_rows_per_group`` rows per group; a group with more rows is still
    computed completely (its CTAs walk on through its remaining row tiles), empty groups cost nothing."""
    import ctypes
    lib = ext.load()
    H, N = 256, 256
    counts = [300, 5, 0, 700, 128, 1]                       # rows per group; the launch covers 128
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    total, G = off[-1], len(counts)
    x = rnd(total, H, seed=40)
    w = rnd(G, N, H, scale=0.05, seed=41)
    group_off = torch.tensor(off, dtype=torch.int32, device="cuda")
    out_cols = N // 2 if epi == "swiglu" else N
    out = torch.full((total, out_cols), float("nan"), dtype=torch.bfloat16, device="cuda")
    if epi == "swiglu":
        from jetspec_b200.parallel.ep import interleave_experts
        wk = interleave_experts(w)                          # (G*N, H): per tile N/2... gate rows then up rows
    else:
        wk = w.reshape(G * N, H).contiguous()
    rc = lib.js_gemm_bf16_grouped(ext._p(x), ext._p(wk), ext._p(out), total, N, H, x.stride(0), wk.stride(0),
                                  out.stride(0), ext.EPI_SWIGLU if epi == "swiglu" else ext.EPI_STORE, G,
                                  ext._p(group_off), 128, None, None, None, None, 1,
                                  ext._p(ext.status_word("cuda")), 0, ext._stream())
    torch.cuda.synchronize()
    assert rc == 0
    ext.check_status("cuda")
    for g in range(G):
        rows = slice(off[g], off[g + 1])
        y = x[rows].float() @ w[g].float().t()
        if epi == "swiglu":
            y = torch.nn.functional.silu(y[:, :N // 2]) * y[:, N // 2:]
        if counts[g]:
            assert rel_err(out[rows], y) < BF16_TOL, f"group {g}"


@pytest.mark.parametrize("T,E,k,renorm", [(96, 128, 8, True), (5, 16, 4, False), (1024, 128, 8, True)])
def test_moe_route_and_sort_kernels(ext, T, E, k, renorm):
    from jetspec_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(T + E)
    logits = torch.randn(T, E, generator=g, device="cuda") * 2
    w_ref, i_ref = ref.moe_route(logits, k, renorm)
    w, i = ext.moe_route(logits, k, renorm)
    assert torch.equal(i.long(), i_ref)
    assert float((w - w_ref).abs().max()) < 1e-6
    first, n_local = E // 4, E // 2                       # this "rank" owns the middle half of the experts
    order, row_w, group_off, counts_all = ext.moe_route_sort(logits, k, renorm, first, n_local)
    flat = i_ref.reshape(-1)
    local = flat - first
    key = torch.where((local >= 0) & (local < n_local), local, torch.full_like(local, n_local))
    exp_order = torch.argsort(key, stable=True)
    assert torch.equal(order.long(), exp_order)
    assert float((row_w - w_ref.reshape(-1)[exp_order]).abs().max()) < 1e-6
    assert torch.equal(group_off[1:].long(), torch.bincount(key, minlength=n_local + 1)[:n_local].cumsum(0))
    assert int(group_off[0]) == 0
    assert torch.equal(counts_all.long(), torch.bincount(flat, minlength=E))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sample_temperature_kernel(ext, dtype):
    N, V, T = 64, 151936, 0.7
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = (torch.randn(N, V, generator=g, device="cuda") * 3).to(dtype)
    gs = torch.Generator(device="cuda").manual_seed(11)
    out = ext.sample_temperature(logits, T, gs)
    u = torch.rand(N, dtype=torch.float32, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11))
    cdf = torch.softmax(logits.double() / T, -1).cumsum(-1)
    hi = cdf.gather(1, out[:, None]).squeeze(1)
    lo = torch.where(out > 0, cdf.gather(1, (out - 1).clamp_min(0)[:, None]).squeeze(1), torch.zeros_like(hi))
    assert bool(((u.double() >= lo - 1e-5) & (u.double() <= hi + 1e-5)).all())       # inverse CDF of the same uniforms
    cold = ext.sample_temperature(logits, 1e-3, gs)                                    # T -> 0: the arg max
    top = logits.float().max(-1).values                                                # (bf16 logits have tied maxima)
    assert torch.equal(logits.float().gather(1, cold[:, None]).squeeze(1), top)


def test_kv_compact_kernel(ext):
    Hkv, cap, D, past = 4, 300, 128, 37
    k, v = rnd(Hkv, cap, D, seed=31), rnd(Hkv, cap, D, seed=32)
    keep = torch.tensor([0, 2, 3, 9, 10, 40], dtype=torch.int32)     # overlapping source and destination ranges
    k0, v0 = k.clone(), v.clone()
    ext.kv_compact(k, v, past, keep)
    torch.cuda.synchronize()
    idx = keep.long().cuda() + past
    assert torch.equal(k[:, past:past + 6], k0[:, idx]) and torch.equal(v[:, past:past + 6], v0[:, idx])
    assert torch.equal(k[:, :past], k0[:, :past]) and torch.equal(k[:, past + 6:], k0[:, past + 6:])


@pytest.mark.parametrize("impl", ["mma", "tc"])
def test_corrupt_slot_map_is_reported_not_followed(ext, impl):
    """A slot index outside the pool must never be dereferenced: the kernel substitutes slot 0, records a status
    code the host reads after the step, and the context stays usable."""
    Hq, Hkv, D, S, n, past = 8, 2, 128, 256, 16, 40
    kp, vp, q = rnd(Hkv, S, D, seed=41), rnd(Hkv, S, D, seed=42), rnd(n, Hq, D, seed=43)
    slot_map = torch.arange(S, dtype=torch.int32, device="cuda").view(1, S).clone()
    slot_map[0, 7] = 10 ** 6                       # corrupted metadata
    slot_map[0, 9] = -3
    cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    rows = torch.zeros(1, dtype=torch.int32, device="cuda")
    pl = torch.tensor([past], dtype=torch.int32, device="cuda")
    out = ext.paged_tree_attention(q, kp, vp, slot_map, rows, cu, pl, None, 1 / math.sqrt(D), True, n, splits=1, impl=impl)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    with pytest.raises(RuntimeError, match="KV slot out of range"):
        ext.check_status("cuda")
    ext.check_status("cuda")                        # the word is cleared by the read; later kernels run normally
    x, w = rnd(8, 256, seed=44), rnd(128, 256, seed=45)
    assert rel_err(ext.gemm(x, w), x.float() @ w.float().t()) < BF16_TOL
