"""The torch.library op boundary and the Hugging Face attention backend (CPU: oracle implementations)."""
import math

import pytest
import torch

from jetspec_b200.ops import reference as ref


def _case():
    torch.manual_seed(0)
    Hq, Hkv, D, S, n, past = 4, 2, 16, 64, 5, 7
    kp, vp, q = torch.randn(Hkv, S, D), torch.randn(Hkv, S, D), torch.randn(n, Hq, D)
    slot_map = torch.randperm(S).to(torch.int32).view(1, S)
    rows, cu = torch.zeros(1, dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32)
    pl = torch.tensor([past], dtype=torch.int32)
    return q, kp, vp, slot_map, rows, cu, pl, 1 / math.sqrt(D)


def test_custom_ops_match_the_oracle_and_trace_as_single_nodes():
    import jetspec_b200.ops.library  # noqa: F401  (registers torch.ops.jetspec_b200.*)
    q, kp, vp, slot_map, rows, cu, pl, scale = _case()
    out = torch.ops.jetspec_b200.paged_tree_attn(q, kp, vp, slot_map, rows, cu, pl, None, scale, True)
    assert torch.allclose(out, ref.paged_tree_attention(q, kp, vp, slot_map, rows, cu, pl, None, scale, True))
    x, w = torch.randn(3, 8), torch.randn(6, 8)
    assert torch.allclose(torch.ops.jetspec_b200.linear_bf16(x, w), x @ w.t())
    assert torch.equal(torch.ops.jetspec_b200.lm_head_argmax(x, w), (x @ w.t()).argmax(-1))
    # shape propagation without running the kernels (what torch.compile / export rely on)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode() as mode:
        fq, fk, fv = (mode.from_tensor(t) for t in (q, kp, vp))
        fo = torch.ops.jetspec_b200.paged_tree_attn(fq, fk, fv, mode.from_tensor(slot_map), mode.from_tensor(rows),
                                                    mode.from_tensor(cu), mode.from_tensor(pl), None, scale, True)
        assert tuple(fo.shape) == (q.shape[0], q.shape[1] * q.shape[2])
    torch.library.opcheck(torch.ops.jetspec_b200.linear_bf16, (x, w), test_utils=("test_schema", "test_faketensor"))


def test_hf_backend_dense_fallback_and_paged_path():
    from jetspec_b200.ops.hf_backend import BACKEND_NAME, PagedHandle, paged_tree_attention_forward, register_hf_backend
    assert register_hf_backend() == BACKEND_NAME
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    assert BACKEND_NAME in ALL_ATTENTION_FUNCTIONS
    q, kp, vp, slot_map, rows, cu, pl, scale = _case()
    n, Hq, D = q.shape
    Hkv, past = kp.shape[0], int(pl[0])
    # dense fallback == causal SDPA
    qq, kk, vv = q.transpose(0, 1)[None], torch.randn(1, Hkv, n, D), torch.randn(1, Hkv, n, D)
    out, _ = paged_tree_attention_forward(None, qq, kk, vv, None, scaling=scale)
    g = Hq // Hkv
    want = torch.nn.functional.scaled_dot_product_attention(qq, kk.repeat_interleave(g, 1), vv.repeat_interleave(g, 1),
                                                            is_causal=True, scale=scale)
    assert torch.allclose(out, want.transpose(1, 2), atol=1e-6)
    # paged path: new rows are scattered to their slots, then attended together with the prefix
    class Layer:                                   # the attribute transformers sets on attention modules
        layer_idx = 0
    pools_k, pools_v = kp[None].clone(), vp[None].clone()
    new_slots = slot_map[0, past:past + n].clone()
    handle = PagedHandle(pools_k, pools_v, slot_map, rows, cu, pl, new_slots, None, True)
    out2, _ = paged_tree_attention_forward(Layer(), qq, kk, vv, None, scaling=scale, paged_handle=handle)
    kp2, vp2 = kp.clone(), vp.clone()
    kp2[:, new_slots.long()] = kk[0]
    vp2[:, new_slots.long()] = vv[0]
    want2 = ref.paged_tree_attention(q, kp2, vp2, slot_map, rows, cu, pl, None, scale, True)
    assert torch.allclose(out2.reshape(n, Hq * D), want2, atol=1e-6)
