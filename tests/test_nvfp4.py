"""NVFP4: quantiser properties on CPU, kernels against the PyTorch oracle on the GPU."""
import pytest
import torch

from jetspec_b200.models.nvfp4 import (NVFP4Linear, dequantize_nvfp4, nvfp4_linear_reference, quantize_model_nvfp4,
                                       quantize_nvfp4, swizzle_scales, unswizzle_scales)


def test_codes_and_scales_round_trip():
    torch.manual_seed(0)
    w = torch.randn(192, 256) * 0.02
    q = quantize_nvfp4(w)
    assert q.packed.shape == (192, 128) and q.scales.shape == (192, 16) and q.outer.dim() == 0
    d = q.dequantize()
    # 4-bit values with a scale per 16: ~10 % error on gaussian data, never worse than half a step of the block
    assert float((d - w).norm() / w.norm()) < 0.12
    # every dequantised value is representable: quantising again changes nothing
    assert torch.equal(quantize_nvfp4(d).dequantize(), d)
    # the largest magnitude of the tensor survives within one e2m1 step
    assert abs(float(d.abs().max()) - float(w.abs().max())) <= float(w.abs().max()) / 6


def test_e2m1_grid_and_ties():
    # exact grid points (scaled so that the block scale is 1.0 after e4m3 rounding) are reproduced
    grid = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 0.0])
    x = grid.repeat(4).view(1, 64)
    q = quantize_nvfp4(x, per_row=True)
    assert torch.allclose(q.dequantize(), x, rtol=0, atol=1e-6)
    # midpoints round to the code with an even mantissa: 2.5 -> 2, 3.5 -> 4, 5 -> 4, 0.25 -> 0, 0.75 -> 1
    mid = torch.tensor([2.5, 3.5, 5.0, 0.25, 0.75, 1.25, 1.75, 6.0] + [0.0] * 8).repeat(4).view(1, 64)
    want = torch.tensor([2.0, 4.0, 4.0, 0.0, 1.0, 1.0, 2.0, 6.0] + [0.0] * 8).repeat(4).view(1, 64)
    assert torch.allclose(quantize_nvfp4(mid, per_row=True).dequantize(), want, rtol=0, atol=1e-6)


def test_scale_tile_order():
    torch.manual_seed(1)
    q = quantize_nvfp4(torch.randn(300, 512))
    sw = q.scales_swizzled
    assert sw.numel() == 3 * (512 // 64) * 512                      # rows padded to 384
    raw = q.scales.view(torch.uint8)
    for r, b in [(0, 0), (77, 9), (131, 31), (299, 17)]:
        off = ((r // 128) * (512 // 64) + b // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + b % 4
        assert int(sw[off]) == int(raw[r, b])
    assert torch.equal(unswizzle_scales(sw, 300, 512).view(torch.uint8), raw)
    assert torch.equal(swizzle_scales(q.scales), sw)


def test_per_row_mode_and_linear_oracle():
    torch.manual_seed(2)
    x = torch.randn(7, 256) * torch.logspace(-2, 2, 7).view(7, 1)     # rows of very different magnitude
    qa = quantize_nvfp4(x, per_row=True)
    assert qa.outer.shape == (7,)
    err = (qa.dequantize() - x).norm(dim=1) / x.norm(dim=1)
    assert float(err.max()) < 0.13                                     # each row keeps its own dynamic range
    w = torch.randn(64, 256) * 0.05
    qw = quantize_nvfp4(w)
    y = nvfp4_linear_reference(x, qw)
    ref = x @ w.t()
    assert float((y - ref).norm() / ref.norm()) < 0.2
    lin = NVFP4Linear(w)
    assert torch.allclose(lin(x), y, rtol=1e-5, atol=1e-5)


def test_quantize_model_replaces_linears():
    from jetspec_b200.models import Qwen3ForCausalLM, tiny_config
    cfg = tiny_config()
    m = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.float32)
    n = quantize_model_nvfp4(m)
    assert n == 7 * cfg.num_hidden_layers
    assert isinstance(m.model.layers[0].self_attn.q_proj, NVFP4Linear)
    assert isinstance(m.lm_head, torch.nn.Linear)
    # q/k/v share one outer scale, so the fused matrix the kernels use is an exact row stack of them
    a = m.model.layers[0].self_attn
    assert float(a.q_proj.outer) == float(a.k_proj.outer) == float(a.v_proj.outer)
    # greedy decoding through the public API runs on the quantised weights
    from jetspec_b200 import LLM, SamplingParams
    out = LLM(m, device="cpu", dtype=torch.float32).generate(torch.arange(6).view(1, -1), SamplingParams(0.0, 4))
    assert len(out["token_ids"]) == 4


# ----------------------------------------------------------------------------- GPU
@pytest.fixture(scope="module")
def ext():
    from jetspec_b200.ops import cuda_ext
    cuda_ext.load()
    yield cuda_ext
    cuda_ext.check_status("cuda")


def _rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K", [(1, 256), (21, 1024), (128, 4096), (200, 12288)])
def test_quant_kernel_matches_quantiser_bytes(ext, M, K):
    x = _rnd(M, K, seed=M + K) * torch.logspace(-1, 1, M, device="cuda").view(M, 1).to(torch.bfloat16)
    buf = ext.quant_nvfp4(x)
    torch.cuda.synchronize()
    q = quantize_nvfp4(x.float(), per_row=True)
    assert torch.equal(buf["outer"], q.outer)
    assert torch.equal(buf["sf"], q.scales_swizzled)
    assert torch.equal(buf["packed"], q.packed)


@pytest.mark.gpu
def test_quant_kernel_fused_rmsnorm(ext):
    from jetspec_b200.ops import reference as ref
    from jetspec_b200.models.nvfp4 import NVFP4Tensor
    M, K = 40, 2048
    x, w = _rnd(M, K, seed=3), (_rnd(K, seed=4) * 0.1 + 1).to(torch.bfloat16)
    normed = torch.empty_like(x)
    buf = ext.quant_nvfp4(x, norm_w=w, eps=1e-6, norm_out=normed)
    torch.cuda.synchronize()
    want = ref.rmsnorm(x, w, 1e-6)
    assert float((normed.float() - want.float()).abs().max()) <= 2 * float(want.float().abs().max()) * 2 ** -8
    # the codes are the quantisation of exactly the bf16 norm the kernel wrote
    q = quantize_nvfp4(normed.float(), per_row=True)
    assert torch.equal(buf["packed"], q.packed) and torch.equal(buf["sf"], q.scales_swizzled)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(128, 512, 1024), (21, 384, 512), (300, 256, 2048), (1, 1024, 4096)])
@pytest.mark.parametrize("split", [1, 2, 4])
def test_gemm_nvfp4_matches_dequantised_product(ext, M, N, K, split):
    x, w = _rnd(M, K, seed=1), _rnd(N, K, scale=0.05, seed=2)
    qw = quantize_nvfp4(w.float())
    out = ext.gemm_nvfp4(x, qw, split=min(split, K // 256))
    torch.cuda.synchronize()
    ext.check_status("cuda")
    ref = nvfp4_linear_reference(x, qw)              # same codes and scales, fp32 products and sums
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < 8e-3
    # and the 4-bit result stays near the bf16 product (quantisation noise only)
    full = x.float() @ w.float().t()
    assert float((out.float() - full).norm() / full.norm()) < 0.2


@pytest.mark.gpu
def test_gemm_nvfp4_epilogues(ext):
    M, H, I = 100, 1024, 1536
    x, res = _rnd(M, H, seed=5), _rnd(M, H, seed=6)
    wo = quantize_nvfp4(_rnd(H, H, scale=0.05, seed=7).float())
    out = ext.gemm_nvfp4(x, wo, residual=res)
    ref = nvfp4_linear_reference(x, wo) + res.float()
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < 8e-3
    f32 = ext.gemm_nvfp4(x, wo, epi=ext.EPI_STORE_F32)
    assert float((f32 - nvfp4_linear_reference(x, wo)).abs().max()) < 1e-3 * float(ref.abs().max())
    g, u = _rnd(I, H, scale=0.05, seed=8), _rnd(I, H, scale=0.05, seed=9)
    qgu = quantize_nvfp4(ext.interleave_gate_up(g, u).float())
    act = ext.gemm_nvfp4(x, qgu, epi=ext.EPI_SWIGLU)
    y = nvfp4_linear_reference(x, qgu).view(M, I // 64, 2, 64)
    want = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, I)
    assert float((act.float() - want).abs().max() / want.abs().max()) < 8e-3
    torch.cuda.synchronize()
    ext.check_status("cuda")


@pytest.mark.gpu
def test_nvfp4_linear_module_on_gpu(ext):
    w = _rnd(512, 1024, scale=0.05, seed=11)
    lin = NVFP4Linear(w.float()).cuda()
    x = _rnd(3, 9, 1024, seed=12)
    y = lin(x)
    ref = nvfp4_linear_reference(x.view(-1, 1024), lin.qweight).view(3, 9, 512)
    assert y.shape == (3, 9, 512) and float((y.float() - ref).abs().max() / ref.abs().max()) < 8e-3


@pytest.mark.gpu
def test_engine_on_nvfp4_weights_is_lossless_and_tracks_the_oracle(ext):
    """Graph-captured AR and tree rounds on 4-bit weights: the tree path reproduces the AR tokens, and both follow
    the fp32 oracle that multiplies the same codes and scales with plain PyTorch."""
    import copy
    from jetspec_b200 import JetSpecEngine, LLM, SamplingParams, RandomTreeDrafter
    from jetspec_b200.models import Qwen3ForCausalLM, Qwen3Config
    cfg = Qwen3Config(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128)
    model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.bfloat16, device="cuda", init="stable")
    assert quantize_model_nvfp4(model) == 7 * cfg.num_hidden_layers
    prompt = torch.randint(0, 4096, (1, 48), generator=torch.Generator().manual_seed(0))
    sp = SamplingParams(0.0, 40)
    eng = JetSpecEngine(model, device="cuda", dtype=torch.bfloat16, max_seq_len=1024)
    ar = eng.generate(prompt, sp)["token_ids"]
    tree = eng.generate_tree(prompt, RandomTreeDrafter(4096, seed=1), tree_depth=8, tree_width=4, budget=60,
                             sampling_params=sp, return_stats=True)
    assert tree["token_ids"] == ar
    oracle = LLM(copy.deepcopy(model).float(), device="cuda", dtype=torch.float32).generate(prompt, sp)["token_ids"]
    agree = sum(a == b for a, b in zip(ar, oracle)) / len(ar)
    assert agree > 0.9
    ext.check_status("cuda")
