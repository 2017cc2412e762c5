"""The allocation-free LM-head argmax entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory on the decode path (a graph is
being captured elsewhere in the process, the memory budget is frozen, or the caller is a foreign
runtime that owns all buffers).  For them ``js_lm_head_argmax_static`` keeps its scratch in a
fixed ``__device__`` array.  It must give exactly what the allocating path gives, call after call
(the scratch keeps the previous call's contents, so the second call checks that nothing stale
leaks through)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_argmax_matches_allocating_path_twice():
    from jetspec_b200.ops import cuda_ext as X
    lib = X.load()
    fn = lib.js_lm_head_argmax_static
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(123)
    for call, (M, V, H) in enumerate([(128, 20000, 512), (37, 9000, 1024)]):   # second call: smaller, other shape
        h = torch.randn(M, H, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(V, H, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        ref_idx, ref_val = X.lm_head_argmax(h, w)
        out_idx = torch.full((M,), -7, dtype=torch.int32, device="cuda")
        out_val = torch.zeros(M, dtype=torch.float32, device="cuda")
        rc = fn(p(h), p(w), M, V, H, h.stride(0), w.stride(0), p(out_idx), p(out_val), stream)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call}: rc {rc}"
        assert torch.equal(out_idx, ref_idx), f"call {call}: tokens differ"
        assert torch.allclose(out_val, ref_val, rtol=0, atol=8e-3 * float(ref_val.abs().max()))
        word = ctypes.c_int(-1)                      # the status word of the static path is readable and clean
        lib.js_lm_head_argmax_static_status.restype = ctypes.c_int
        assert lib.js_lm_head_argmax_static_status(ctypes.byref(word), stream) == 0 and word.value == 0
    # sizes beyond the built-in scratch are refused, not truncated
    assert fn(p(h), p(w), 129, V, H, h.stride(0), w.stride(0), p(out_idx), p(out_val), stream) == -30
    assert fn(p(h), p(w), 1, 200000, H, h.stride(0), w.stride(0), p(out_idx), p(out_val), stream) == -30
