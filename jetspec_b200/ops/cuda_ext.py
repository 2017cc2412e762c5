"""Loader and thin tensor-level wrappers for the sm_100a kernel library.

The kernels live in ``csrc/*.cu`` and are compiled by ``nvcc`` for
``compute_100a/sm_100a`` into one shared library inside the package
(``jetspec_b200/_C/libjetspec_sm100.so``).  They export plain C entry points that
take raw device pointers and a stream, so there is no framework ABI to match and
the library builds in seconds; this module binds them with ``ctypes`` and passes
``tensor.data_ptr()`` and the current CUDA stream (launches are therefore
graph-capturable).

On a machine with a GPU a missing or unloadable library is an error, never a
silent fallback.

What these kernels stand in for in the reference: the fused verify stack's cuBLAS GEMMs and ATen glue
(``jetspec/inference_engine/compiled_verify_stack.py:170-272``), the Triton paged tree-attention kernel
(``jetspec/inference_engine/paged_tree_attn.py:55-367``, op wrapper ``paged_tree_attn_op.py:29-79``), the dense
tree-attention kernel of the HF path (``jetspec/core/tree_attention_kernel.py:63-216``), the graphed accept
(``jetspec/inference_engine/graph_capture.py:240-323``) and the grouped-GEMM MoE (``jetspec/models/moe_fused.py:16-116``).
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
import sys
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ROOT = os.path.dirname(_PKG)
# kernel sources: inside the installed package (wheel), else beside it (source checkout)
_CSRC = os.path.join(_PKG, "csrc") if os.path.isdir(os.path.join(_PKG, "csrc")) else os.path.join(_ROOT, "csrc")
_OUT_DIR = os.path.join(_PKG, "_C")
LIB_PATH = os.path.join(_OUT_DIR, "libjetspec_sm100.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]

_lib = None


def sources() -> list:
    return sorted(glob.glob(os.path.join(_CSRC, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(_CSRC, "*.cuh")) + glob.glob(os.path.join(_CSRC, "*.h"))
    return any(os.path.getmtime(f) > t for f in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a into the in-tree shared library."""
    if not force and not _stale():
        return LIB_PATH
    if not os.path.isdir(_CSRC):
        raise RuntimeError(f"kernel sources not found at {_CSRC}")
    os.makedirs(_OUT_DIR, exist_ok=True)
    # Several ranks may find the library stale at the same moment: one builds under a file lock, into a
    # temporary name that replaces the library atomically; the others wait and then find it fresh.
    import fcntl
    with open(os.path.join(_OUT_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale():
                return LIB_PATH
            nvcc = os.environ.get("NVCC", "nvcc")
            tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
            # one object per source, compiled concurrently and kept beside the library, so a change to one
            # kernel file recompiles that file only; headers invalidate everything
            obj_dir = os.path.join(_OUT_DIR, "obj")
            os.makedirs(obj_dir, exist_ok=True)
            hdr_time = max([os.path.getmtime(f) for f in glob.glob(os.path.join(_CSRC, "*.cuh")) +
                            glob.glob(os.path.join(_CSRC, "*.h"))] or [0.0])
            compile_flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas=-v"] if verbose else [])
            jobs = []
            for src in sources():
                obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
                fresh = (not force and os.path.exists(obj)
                         and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time))
                jobs.append((src, obj, fresh))
            procs = [(src, subprocess.Popen([nvcc] + compile_flags + ["-I", _CSRC, "-c", src, "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
                     for src, obj, fresh in jobs if not fresh]
            log = []
            for src, pr in procs:
                out, err = pr.communicate()
                log.append(err)
                if pr.returncode != 0:
                    for _, other in procs:
                        if other.poll() is None:
                            other.kill()
                    raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{out}\n{err}")
            r = subprocess.run([nvcc] + NVCC_FLAGS + [obj for _, obj, _ in jobs] + ["-o", tmp],
                               capture_output=True, text=True)
            if r.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError(f"nvcc link failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, LIB_PATH)
            if verbose:
                print("".join(log), file=sys.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load():
    """``ctypes`` handle of the kernel library (built on first use when a compiler is present)."""
    global _lib
    if _lib is not None:
        return _lib
    if _stale():
        try:
            build()
        except Exception as e:  # no compiler on this machine: use an existing library if there is one
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(f"sm_100a kernel library is missing and could not be built: {e}") from e
    lib = ctypes.CDLL(LIB_PATH)
    for name in ("js_gemm_bf16", "js_paged_tree_attention", "js_embed", "js_rmsnorm", "js_qkv_post", "js_silu_mul",
                 "js_gather_rows", "js_argmax_merge", "js_topk_merge", "js_tree_build", "js_tree_accept_commit",
                 "js_draft_prep"):
        getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


# ------------------------------------------------------------------ helpers
_vp = ctypes.c_void_p


def _p(t: Optional[torch.Tensor]):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_cur_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream of the current device as a raw handle.  ``torch.cuda.current_stream()`` builds a Python
    ``Stream`` object and resolves the device index on every call (~10 us, paid per kernel launch on the eager
    path); the raw accessor is a plain C call."""
    if _raw_stream is not None and _cur_device is not None:
        return _vp(_raw_stream(_cur_device()))
    return _vp(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels write an error code to (0 = ok)."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else (torch.cuda.current_device() if dev.type == "cuda" else -1)
    if key not in _status:
        with torch.inference_mode(False):       # a normal tensor: it is cleared in place from any calling context
            _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


STATUS_NAMES = {0: "ok", 1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free stage",
                3: "timeout waiting for the accumulator", 4: "timeout waiting for a peer flag",
                5: "KV slot out of range", 6: "tree node index out of range",
                7: "expert-parallel dispatch: a rank's expert counts never arrived",
                8: "expert-parallel dispatch: a source rank's rows never arrived",
                9: "all-reduce tail / expert combine: partial cells never arrived",
                10: "all-reduce tail: a slice owner's result cells never arrived",
                11: "vocabulary-parallel top-k: a rank's record never arrived",
                12: "expert-parallel dispatch: more rows for one expert than the grouped launch covers"}


def check_status(device) -> None:
    """Raise if any kernel recorded an error since the last check (one host sync)."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"kernel status {code}: {STATUS_NAMES.get(code, 'unknown')}")


_inv_freq: dict = {}


def inv_freq(head_dim: int, theta: float, device) -> torch.Tensor:
    key = (head_dim, float(theta), str(device))
    if key not in _inv_freq:
        from .reference import rope_inv_freq
        _inv_freq[key] = rope_inv_freq(head_dim, theta, device).contiguous()
    return _inv_freq[key]


# ------------------------------------------------------------------ GEMM
EPI_STORE, EPI_SWIGLU, EPI_ARGMAX, EPI_TOPK, EPI_STORE_F32 = 0, 1, 2, 3, 4
SM_COUNT = 148
_DEEP = os.environ.get("JETSPEC_GEMM_DEEP", "0") == "1"
_SPLIT_DEEP = os.environ.get("JETSPEC_SPLIT_DEEP")      # force the split-K pipeline: 1 = 192 KB, 2 = 128 KB, 0 = 96 KB
_SPLIT_DEEP = int(_SPLIT_DEEP) if _SPLIT_DEEP is not None else None


# measured best (bn, split, deep) per (M, N, K, epilogue); filled from the tuning sweep
GEMM_TUNING: dict = {}


def gemm_supported(M: int, N: int, K: int) -> bool:
    return K % 8 == 0 and N % 8 == 0 and K >= 64


def gu_tile(intermediate: int) -> int:
    """Tile width of the fused gate/up GEMM (the weight is interleaved at this granularity): 128, or the value of
    ``JETSPEC_GU_TILE`` (128, 192 or 256).  192 columns turn Qwen3-8B's 192 tiles of 128 columns (two CTAs on 44 of
    the 148 SMs) into one even wave of 128 CTAs, but measured slower in the decode round (5.77 against 5.61 ms):
    with one CTA per SM nothing streams while a tile's SwiGLU epilogue runs, whereas two shallow CTAs per SM
    overlap one's epilogue with the other's loads."""
    env = os.environ.get("JETSPEC_GU_TILE")
    return int(env) if env else 128


def pick_gemm_config(M: int, N: int, K: int, epi: int, bn: Optional[int] = None):
    """``(bn, split, deep)``: tile width, K-split cluster size, pipeline variant.

    Decode shapes are weight-streaming bound, so the goal is enough CTAs to cover the
    SMs (two CTAs fit per SM with the shallow pipeline) without re-reading the
    activations more than necessary.
    """
    key = (M, N, K, epi)
    if key in GEMM_TUNING:
        return GEMM_TUNING[key]
    m_tiles = (M + 127) // 128
    if bn is None and epi == EPI_STORE and m_tiles >= 4 and N % 256 == 0 and m_tiles * (N // 256) >= 64:
        # prefill / batched verify (>= 512 rows): compute bound, and a 128x128 tile asks more of the L2-to-SM path
        # than it gives; 128x256 tiles with the deep pipeline measured 5-12 % faster at 2048 rows
        # (qkv 97 -> 91 us, o 62 -> 56, down 182 -> 165) and equal or better at 512.  From 1024 rows on, two row tiles
        # per CTA (deep = 3: 256 x 256 outputs per CTA, every weight stage feeds two accumulators) when that does not
        # cost a wave: at 2048 rows o 53.9 -> 48.7 us, down 155.4 -> 146.3 (128 CTAs, one wave), but qkv
        # 88.1 -> 96.2 (192 CTAs: two waves of big tiles against three of small ones), gate/up equal.
        if m_tiles >= 8:
            t1, t2 = m_tiles * (N // 256), ((m_tiles + 1) // 2) * (N // 256)
            if 2 * ((t2 + SM_COUNT - 1) // SM_COUNT) <= (t1 + SM_COUNT - 1) // SM_COUNT:
                return 256, 1, 3
        return 256, 1, 1
    bn = bn or 128
    tiles = m_tiles * ((N + bn - 1) // bn)
    kb = (K + 63) // 64
    split = 1
    if epi in (EPI_STORE, EPI_STORE_F32, EPI_SWIGLU):
        # SwiGLU tiles hold two (gate, up) chunk pairs, so a split of 4 leaves two CTAs of each cluster without
        # output columns; it still pays when the projection is narrow (tensor-parallel shards: 24 tiles -> 96 CTAs)
        max_split = 4
        # Measured on chains of L2-cold GEMMs (M = 128): a K split helps while the whole grid is one
        # wave of one CTA per SM AND the clusters can be placed (a cluster lives inside one GPC, so only
        # ~32 clusters of 4, ~40 of 3 or ~72 of 2 fit at once; 48 clusters of 3 ran as two waves).
        room = {2: 72, 3: 40, 4: 32}
        for c in (4, 3, 2):
            if c <= max_split and tiles <= room[c] and tiles * c <= SM_COUNT and kb // c >= 4:
                split = c
                break
    if split > 1:
        # deep pipeline (192 KB, one CTA per SM; the receive area aliases the stages), except for the narrow shards of
        # a tensor-parallel rank (at most 96 CTAs with at most 16 k-blocks each): 128 KB serves those as well and
        # leaves room for the next kernel's CTA and its first weight stages on the same SM (compute-only round of a
        # 1/8 shard: 2.96 -> 2.92 ms).  The full-size o_proj (128 CTAs) measured slower that way inside the round
        # (5.45 -> 5.50 ms) although faster in a chain of its own.  JETSPEC_SPLIT_DEEP forces 1 (192 KB), 2 (128 KB)
        # or 0 (96 KB) for every split launch.
        if _SPLIT_DEEP is not None:
            return bn, split, _SPLIT_DEEP
        return bn, split, (2 if (kb + split - 1) // split <= 16 and tiles * split <= 96 else 1)
    # no split: a deep pipeline when the tiles fit one CTA per SM, else two shallow CTAs per SM
    return bn, 1, (1 if tiles <= SM_COUNT or _DEEP else 0)


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, epi: int = EPI_STORE, bn: Optional[int] = None,
         split: Optional[int] = None, deep: Optional[bool] = None, pdl: bool = False,
         part_val=None, part_idx=None, part_lse=None, trace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out = x @ w.T`` (+ ``residual``) on the tcgen05 kernel.  ``x (M, K)``, ``w (N, K)`` bf16."""
    lib = load()
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1
    cb, cs, cd = pick_gemm_config(M, N, K, epi, bn)
    bn = bn or cb
    split = split or cs
    deep = cd if deep is None else deep
    if out is None:
        if epi == EPI_SWIGLU:
            out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=x.device)
        elif epi == EPI_STORE_F32:
            out = torch.empty(M, N, dtype=torch.float32, device=x.device)
        elif epi in (EPI_STORE,):
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    ldc = out.stride(0) if out is not None else 0
    rc = lib.js_gemm_bf16(_p(x), _p(w), _p(out), _p(residual), M, N, K, x.stride(0), w.stride(0), ldc, epi, bn,
                          split, int(deep), _p(part_val), _p(part_idx), _p(part_lse),
                          _p(status_word(x.device)), _p(trace), int(pdl), _stream())
    _check(rc, f"js_gemm_bf16(M={M},N={N},K={K},epi={epi},bn={bn},split={split})")
    return out


def interleave_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor, bn: int = 128) -> torch.Tensor:
    """Weight layout for the SwiGLU epilogue: every ``bn``-row tile holds ``bn/2`` gate rows
    followed by the ``bn/2`` up rows of the same outputs."""
    I, H = gate_w.shape
    h = bn // 2
    assert I % h == 0
    if not isinstance(gate_w, torch.Tensor):      # NVFP4: stack, then permute rows (exact: rows are independent)
        t = torch.arange(I, device=gate_w.packed.device).view(I // h, h)
        order = torch.cat((t, t + I), dim=1).reshape(-1)
        return type(gate_w).cat_rows([gate_w, up_w]).index_rows(order)
    g = gate_w.view(I // h, h, H)
    u = up_w.view(I // h, h, H)
    return torch.cat((g, u), dim=1).reshape(2 * I, H).contiguous()


def n_tiles(N: int, bn: int = 128) -> int:
    return (N + bn - 1) // bn


# ------------------------------------------------------------------ NVFP4
def nvfp4_act_buffers(M: int, K: int, device) -> dict:
    """Device buffers one quantised activation matrix needs (allocate once, reuse across graph replays)."""
    tiles = (M + 127) // 128
    return {"packed": torch.zeros(M, K // 2, dtype=torch.uint8, device=device),
            "sf": torch.zeros(tiles * (K // 64) * 512, dtype=torch.uint8, device=device),
            "outer": torch.zeros(M, dtype=torch.float32, device=device), "M": M, "K": K}


def quant_nvfp4(x: torch.Tensor, buf: Optional[dict] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6,
                norm_out: Optional[torch.Tensor] = None, pdl: bool = False) -> dict:
    """Quantise ``x (M, K)`` bf16 to NVFP4 with one outer scale per row; with ``norm_w`` the RMSNorm of ``x`` is
    quantised instead (and also written to ``norm_out`` as bf16 when given)."""
    lib = load()
    M, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    if buf is None:
        buf = nvfp4_act_buffers(M, K, x.device)
    assert buf["K"] == K and buf["M"] >= M
    lib.js_quant_nvfp4.restype = ctypes.c_int
    rc = lib.js_quant_nvfp4(_p(x), x.stride(0), _p(norm_w), ctypes.c_float(eps), M, K, _p(buf["packed"]), _p(buf["sf"]),
                            _p(buf["outer"]), _p(norm_out), norm_out.stride(0) if norm_out is not None else 0,
                            int(pdl), _stream())
    _check(rc, f"js_quant_nvfp4(M={M},K={K})")
    return buf


def pick_nvfp4_split(M: int, N: int, K: int, epi: int) -> int:
    """K split for the NVFP4 GEMM: same placement rule as the bf16 kernel (clusters of 4 / 2 that fit one wave)."""
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    kb = K // 256
    max_split = 2 if epi == EPI_SWIGLU else 4
    room = {2: 72, 4: 32}
    for c in (4, 2):
        if c <= max_split and tiles <= room[c] and tiles * c <= SM_COUNT and kb // c >= 2:
            return c
    return 1


def gemm_nvfp4(x, qw, out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
               epi: int = EPI_STORE, split: Optional[int] = None, pdl: bool = False, act_buf: Optional[dict] = None):
    """``out = q(x) @ dequant(qw).T`` on the block-scaled tcgen05 kernel.

    ``x`` is either a bf16 ``(M, K)`` matrix (quantised here, per row) or the dict ``quant_nvfp4`` returned;
    ``qw`` is an ``NVFP4Tensor`` with per-tensor outer scale and swizzled block scales.
    """
    lib = load()
    act = x if isinstance(x, dict) else quant_nvfp4(x, act_buf, pdl=pdl)
    M = x.shape[0] if not isinstance(x, dict) else act.get("rows", act["M"])
    N, K = qw.shape
    assert act["K"] == K
    qw.swizzled()
    split = split or pick_nvfp4_split(M, N, K, epi)
    dev = qw.packed.device
    if out is None:
        out = torch.empty(M, N // 2 if epi == EPI_SWIGLU else N,
                          dtype=torch.float32 if epi == EPI_STORE_F32 else torch.bfloat16, device=dev)
    if not hasattr(qw, "_w_scale"):
        qw._w_scale = float(qw.outer)           # one host read per weight, outside any graph capture
    lib.js_gemm_nvfp4.restype = ctypes.c_int
    rc = lib.js_gemm_nvfp4(_p(act["packed"]), _p(act["sf"]), _p(act["outer"]), _p(qw.packed), _p(qw.scales_swizzled),
                           ctypes.c_float(qw._w_scale), _p(out), _p(residual), M, N, K, act["packed"].stride(0),
                           qw.packed.stride(0), out.stride(0), epi, split, _p(status_word(dev)), int(pdl), _stream())
    _check(rc, f"js_gemm_nvfp4(M={M},N={N},K={K},epi={epi},split={split})")
    return out


def lm_head_argmax(h: torch.Tensor, w: torch.Tensor, ws: Optional[dict] = None, pdl: bool = False,
                   out_idx: Optional[torch.Tensor] = None, out_val: Optional[torch.Tensor] = None):
    """Greedy token per row: vocabulary GEMM with a per-tile argmax epilogue, then a merge.
    The ``(M, V)`` logits are never written."""
    lib = load()
    M, N = h.shape[0], w.shape[0]
    nt = n_tiles(N)
    if ws is None:
        ws = {"val": torch.empty(M, nt, dtype=torch.float32, device=h.device),
              "idx": torch.empty(M, nt, dtype=torch.int32, device=h.device)}
    gemm(h, w, out=None, epi=EPI_ARGMAX, bn=128, split=1, pdl=pdl, part_val=ws["val"], part_idx=ws["idx"])
    if out_idx is None:
        out_idx = torch.empty(M, dtype=torch.int32, device=h.device)
    if out_val is None:
        out_val = torch.empty(M, dtype=torch.float32, device=h.device)
    _check(lib.js_argmax_merge(_p(ws["val"]), _p(ws["idx"]), nt, M, _p(out_idx), _p(out_val), int(pdl), _stream()),
           "js_argmax_merge")
    return out_idx, out_val


# Few-row top-k over the vocabulary in two passes over materialised logits (JETSPEC_TOPK_TWO_PASS=0: inside the GEMM
# epilogue, as for many rows).  The partial lists reuse the epilogue's workspace: (rows, slices, 8) fits (rows, tiles, 8).
TOPK_TWO_PASS = os.environ.get("JETSPEC_TOPK_TWO_PASS", "1") != "0"
TOPK_TWO_PASS_ROWS = 32
TOPK_SLICES = 64


def lm_head_topk_logprobs(h: torch.Tensor, w: torch.Tensor, k: int, ws: Optional[dict] = None, pdl: bool = False,
                          out_tok: Optional[torch.Tensor] = None, out_lp: Optional[torch.Tensor] = None):
    """Per-row top-``k`` tokens with full-vocabulary log-probabilities, without materialising logits."""
    lib = load()
    assert 1 <= k <= 8
    M, N = h.shape[0], w.shape[0]
    nt = n_tiles(N)
    if ws is None:
        ws = {"val": torch.empty(M, nt, 8, dtype=torch.float32, device=h.device),
              "idx": torch.empty(M, nt, 8, dtype=torch.int32, device=h.device),
              "lse": torch.empty(M, nt, 2, dtype=torch.float32, device=h.device)}
    if out_tok is None:
        out_tok = torch.empty(M, k, dtype=torch.int32, device=h.device)
    if out_lp is None:
        out_lp = torch.empty(M, k, dtype=torch.float32, device=h.device)
    if TOPK_TWO_PASS and M <= TOPK_TWO_PASS_ROWS and N % 4 == 0 and nt >= TOPK_SLICES:
        # A draft block has a few rows, so one warp per CTA would carry the in-epilogue sorted insertion and the
        # weight stream stalls behind it.  Store the (few) logits with the plain fp32 epilogue instead, which streams
        # at the argmax epilogue's rate, and take the top-k from them in two small passes (they stay in L2).
        if "logits" not in ws or ws["logits"].shape[0] < M or ws["logits"].shape[1] != N:
            ws["logits"] = torch.empty(max(M, TOPK_TWO_PASS_ROWS), N, dtype=torch.float32, device=h.device)
        logits = ws["logits"][:M]
        gemm(h, w, out=logits, epi=EPI_STORE_F32, bn=128, split=1, pdl=pdl)
        lib.js_logits_topk_slices.restype = ctypes.c_int
        _check(lib.js_logits_topk_slices(_p(logits), ctypes.c_longlong(logits.stride(0)), M, N, TOPK_SLICES,
                                         _p(ws["val"]), _p(ws["idx"]), _p(ws["lse"]), int(pdl), _stream()),
               "js_logits_topk_slices")
        _check(lib.js_topk_merge(_p(ws["val"]), _p(ws["idx"]), _p(ws["lse"]), TOPK_SLICES, M, k, _p(out_tok),
                                 _p(out_lp), int(pdl), _stream()), "js_topk_merge")
        return out_tok, out_lp
    gemm(h, w, out=None, epi=EPI_TOPK, bn=128, split=1, pdl=pdl, part_val=ws["val"], part_idx=ws["idx"],
         part_lse=ws["lse"])
    _check(lib.js_topk_merge(_p(ws["val"]), _p(ws["idx"]), _p(ws["lse"]), nt, M, k, _p(out_tok), _p(out_lp),
                             int(pdl), _stream()), "js_topk_merge")
    return out_tok, out_lp


# ------------------------------------------------------------------ elementwise
def embed(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, pdl: bool = False):
    lib = load()
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _check(lib.js_embed(_p(ids), _p(table), _p(out), T, H, V, int(pdl), _stream()), "js_embed")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None, pdl: bool = False):
    lib = load()
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    o2 = out.reshape(-1, shp[-1])
    _check(lib.js_rmsnorm(_p(x2), _p(w), _p(o2), x2.shape[0], shp[-1], x2.stride(0), o2.stride(0),
                          ctypes.c_float(eps), int(pdl), _stream()), "js_rmsnorm")
    return out.reshape(shp)


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, pdl: bool = False):
    lib = load()
    T, I2 = gate_up.shape
    gate_up = gate_up.contiguous()
    if out is None:
        out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib.js_silu_mul(_p(gate_up), _p(out), T, I2 // 2, int(pdl), _stream()), "js_silu_mul")
    return out


def qkv_post(qkv: torch.Tensor, q_norm_w, k_norm_w, positions: torch.Tensor, slots: torch.Tensor,
             freq: torch.Tensor, q_out: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: torch.Tensor,
             Hq: int, Hkv: int, eps: float, n_valid: Optional[torch.Tensor] = None, pdl: bool = False):
    """Per-head RMSNorm + RoPE on the fused QKV rows; q → ``q_out``, k/v → pools at ``slots``."""
    lib = load()
    T = qkv.shape[0]
    S = k_pool.shape[1]
    _check(lib.js_qkv_post(_p(qkv), qkv.stride(0), _p(q_norm_w), _p(k_norm_w), _p(positions), _p(slots), _p(freq),
                           _p(q_out), _p(k_pool), _p(v_pool), T, Hq, Hkv, S, ctypes.c_float(eps), _p(n_valid),
                           _p(status_word(qkv.device)), int(pdl), _stream()), "js_qkv_post")
    return q_out


def gather_rows(src: torch.Tensor, idx: Optional[torch.Tensor], dst: torch.Tensor, dst_col0: int = 0,
                n_valid: Optional[torch.Tensor] = None, rows: Optional[int] = None, pdl: bool = False):
    lib = load()
    rows = rows if rows is not None else (idx.numel() if idx is not None else src.shape[0])
    H = src.shape[1]
    _check(lib.js_gather_rows(_p(src), src.stride(0), _p(idx), _p(n_valid), _p(dst), dst.stride(0), dst_col0, rows, H,
                              src.shape[0], int(pdl), _stream()), "js_gather_rows")
    return dst


# ------------------------------------------------------------------ attention
def attn_splits(q_tiles: int, Hkv: int, max_keys: int) -> int:
    # the launcher adds one q tile per sequence for raggedness; keep the whole grid in ONE wave
    # (two CTAs fit per SM) and give every split at least a couple of key tiles
    ctas = max(1, (q_tiles + 1) * Hkv)
    want = max(1, (2 * SM_COUNT) // ctas)
    return max(1, min(want, (max_keys + 127) // 128, 16))


ATTN_CLUSTER_SPLITS = 8       # key splits the tcgen05 kernel merges inside one cluster (kMaxClusterSplits)
ATTN_IMPL = os.environ.get("JETSPEC_ATTN", "tc")     # "tc": tcgen05 kernel where it applies; "mma": mma.sync kernel


def attn_impl(Hq: int, Hkv: int, W: int = 0) -> str:
    G = Hq // Hkv
    return "tc" if ATTN_IMPL == "tc" and 128 % G == 0 and W <= 8 else "mma"


_ATTN_ROOM: dict = {}


def _attn_cluster_room(G: int, splits: int) -> int:
    """Clusters of ``splits`` CTAs of the tcgen05 attention kernel the current device holds at once."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    key = (dev, G, splits)
    if key not in _ATTN_ROOM:
        n = 0
        if dev >= 0:
            lib = load()
            lib.js_attn_tc_max_active_clusters.restype = ctypes.c_int
            n = int(lib.js_attn_tc_max_active_clusters(int(G), int(splits)))
        if n <= 0:       # no device / no answer: what was measured on a 148-SM part, else a conservative guess
            n = {2: 72, 3: 40, 4: 32}.get(splits, SM_COUNT // (splits + 2))
        _ATTN_ROOM[key] = n
    return _ATTN_ROOM[key]


def attn_merges_in_cluster(T: int, Hq: int, Hkv: int, splits: int) -> bool:
    """Whether the tcgen05 kernel merges ``splits`` key splits itself (they form one cluster and exchange partial
    outputs through distributed shared memory): up to ATTN_CLUSTER_SPLITS, and only while all clusters of the
    launch are resident at once (a cluster lives inside one GPC: 148 SMs hold 33 clusters of 4 but only 15 of 8)."""
    G = Hq // Hkv
    if attn_impl(Hq, Hkv) != "tc" or not 2 <= splits <= ATTN_CLUSTER_SPLITS:
        return False
    npt = 128 // G
    return ((T + npt - 1) // npt) * Hkv <= _attn_cluster_room(G, splits)


def attn_splits_for(T: int, Hq: int, Hkv: int, max_keys: int) -> int:
    """Key splits for ``T`` query tokens: fill the SMs with ONE wave of CTAs, a couple of key tiles per split."""
    G = Hq // Hkv
    if attn_impl(Hq, Hkv) == "tc":                      # 128 rows per CTA, one CTA per SM
        # one wave of CTAs, a couple of key tiles per split.  Measured on the decode round (prefix ~2.5 k keys): more,
        # shorter splits win even when they need the separate merge launch (TP=2: 9 splits + merge 4.60 ms per round,
        # 6 splits merged inside a cluster 4.71 ms), because the kernel's time is the chain of key tiles of one CTA.
        npt = 128 // G
        ctas = max(1, ((T + npt - 1) // npt) * Hkv)
        return max(1, min(SM_COUNT // ctas, (max_keys + 127) // 128, 16))
    npt = max(1, 64 // G)
    return attn_splits((T + npt - 1) // npt, Hkv, max_keys)


def paged_tree_attention(q, k_pool, v_pool, slot_map, seq_rows, cu_q, past_lens, mask_bits, scale: float,
                         causal: bool, max_q: int, out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
                         ws: Optional[dict] = None, max_keys: Optional[int] = None, pdl: bool = False,
                         impl: Optional[str] = None):
    """Ragged paged attention with tree (packed-bit) or causal masking.  See
    :func:`jetspec_b200.ops.reference.paged_tree_attention` for the contract."""
    lib = load()
    T, Hq, D = q.shape
    assert D == 128
    Hkv, S = k_pool.shape[0], k_pool.shape[1]
    B = seq_rows.numel()
    G = Hq // Hkv
    if out is None:
        out = torch.empty(T, Hq * D, dtype=q.dtype, device=q.device)
    if splits is None:
        mk = max_keys if max_keys is not None else slot_map.shape[1]
        splits = attn_splits_for(T, Hq, Hkv, mk)
    ws_o = ws_ml = None
    if splits > 1:
        if ws is None:
            ws = {"o": torch.empty(splits, T, Hq, D, dtype=torch.float32, device=q.device),
                  "ml": torch.empty(splits, T, Hq, 2, dtype=torch.float32, device=q.device)}
        ws_o, ws_ml = ws["o"], ws["ml"]
    W = mask_bits.shape[1] if mask_bits is not None else 0
    impl = impl or attn_impl(Hq, Hkv, W)
    fn = lib.js_paged_tree_attention_tc if impl == "tc" else lib.js_paged_tree_attention
    fn.restype = ctypes.c_int
    _check(fn(_p(q), _p(k_pool), _p(v_pool), _p(slot_map), _p(seq_rows), _p(cu_q),
              _p(past_lens), _p(mask_bits), _p(out), _p(ws_o), _p(ws_ml),
              _p(status_word(q.device)), B, T, Hq, Hkv, S, slot_map.shape[1], W,
              int(bool(causal)), int(splits), ctypes.c_float(scale), int(pdl), _stream()),
           f"js_paged_tree_attention[{impl}]")
    return out


def l2_prefetch(t: torch.Tensor, max_bytes: Optional[int] = None, ctas: int = 8) -> None:
    """Ask the memory system to pull the first ``max_bytes`` of ``t`` into L2 (launch on the CURRENT stream;
    the kernel only issues ``cp.async.bulk.prefetch.L2`` requests and exits)."""
    lib = load()
    n = t.numel() * t.element_size()
    if max_bytes is not None:
        n = min(n, int(max_bytes))
    lib.js_l2_prefetch.restype = ctypes.c_int
    _check(lib.js_l2_prefetch(_p(t), ctypes.c_size_t(n), int(ctas), _stream()), "js_l2_prefetch")


# ------------------------------------------------------------------ routing, sampling, compaction
def moe_route(router_logits: torch.Tensor, top_k: int, renorm: bool, pdl: bool = False):
    """``(weights (T, k) fp32, experts (T, k) int32)``: softmax over the experts, top-k, optional renormalisation."""
    lib = load()
    lg = router_logits.float().contiguous()
    T, E = lg.shape
    wts = torch.empty(T, top_k, dtype=torch.float32, device=lg.device)
    idx = torch.empty(T, top_k, dtype=torch.int32, device=lg.device)
    lib.js_moe_route.restype = ctypes.c_int
    _check(lib.js_moe_route(_p(lg), T, E, top_k, int(bool(renorm)), _p(wts), _p(idx), int(pdl), _stream()), "js_moe_route")
    return wts, idx


def moe_route_sort(router_logits: torch.Tensor, top_k: int, renorm: bool, first_expert: int, n_local: int,
                   pdl: bool = False, with_tokens: bool = False):
    """Routing plus the stable permutation of the (token, choice) pairs by local expert, all on the device.
    Returns ``(order int32 (T*k), row_weight fp32 (T*k), group_off int32 (n_local+1), counts_all int32 (E))``."""
    lib = load()
    wts, idx = moe_route(router_logits, top_k, renorm, pdl)
    T, E = router_logits.shape
    P = T * top_k
    dev = wts.device
    order = torch.empty(P, dtype=torch.int32, device=dev)
    row_w = torch.empty(P, dtype=torch.float32, device=dev)
    group_off = torch.empty(n_local + 1, dtype=torch.int32, device=dev)
    counts_all = torch.empty(E, dtype=torch.int32, device=dev)
    tok = torch.empty(P, dtype=torch.int32, device=dev) if with_tokens else None
    lib.js_moe_sort.restype = ctypes.c_int
    _check(lib.js_moe_sort(_p(idx), _p(wts), P, E, int(first_expert), int(n_local), _p(order), _p(row_w), _p(group_off),
                           _p(counts_all), int(top_k), _p(tok), int(pdl), _stream()), "js_moe_sort")
    if with_tokens:
        return order, row_w, group_off, counts_all, tok
    return order, row_w, group_off, counts_all


def sample_temperature(logits: torch.Tensor, temperature: float, generator=None) -> torch.Tensor:
    """Draw one token per row from ``softmax(logits / temperature)`` (inverse CDF with one uniform per row)."""
    lib = load()
    shp = logits.shape[:-1]
    flat = logits.reshape(-1, logits.shape[-1])
    if flat.dtype not in (torch.float32, torch.bfloat16):
        flat = flat.float()
    flat = flat.contiguous()
    N, V = flat.shape
    u = torch.rand(N, dtype=torch.float32, device=flat.device, generator=generator)
    out = torch.empty(N, dtype=torch.int64, device=flat.device)
    lib.js_sample_temperature.restype = ctypes.c_int
    _check(lib.js_sample_temperature(_p(flat), int(flat.dtype == torch.bfloat16), N, V, flat.stride(0),
                                     ctypes.c_float(temperature), _p(u), _p(out), _stream()), "js_sample_temperature")
    return out.view(shp)


def kv_compact(k: torch.Tensor, v: torch.Tensor, past_len: int, keep: torch.Tensor) -> None:
    """In place: positions ``past_len + i`` of ``k, v (Hkv, capacity, 128)`` take the rows ``past_len + keep[i]``."""
    lib = load()
    assert k.dtype == torch.bfloat16 and k.shape[-1] == 128 and k.is_contiguous() and v.is_contiguous()
    keep = keep.to(device=k.device, dtype=torch.int32).contiguous()
    lib.js_kv_compact.restype = ctypes.c_int
    _check(lib.js_kv_compact(_p(k), _p(v), k.shape[0], k.shape[1], int(past_len), _p(keep), keep.numel(), _stream()),
           "js_kv_compact")


# ------------------------------------------------------------------ MoE (grouped through the dense GEMM)
_moe_cache: dict = {}


def moe_forward(x, gate_w, w_gate_up, w_down, top_k: int, renorm: bool, router_logits=None, residual=None):
    """Sparse MoE on one GPU: route, sort the (token, choice) pairs by expert, run all experts'
    SwiGLU MLPs with two grouped tcgen05 GEMMs (one launch each), combine with the routing weights.
    With ``residual`` (T, H) the combine kernel adds the layer output onto it in place and returns it."""
    from . import reference as ref
    from ..parallel.ep import interleave_experts, route_and_sort
    lib = load()
    T, H = x.shape
    E, I2, _ = w_gate_up.shape
    I = I2 // 2
    if I % 64 or H % 128:
        y = ref.moe_forward(x, gate_w, w_gate_up, w_down, top_k, renorm, router_logits)
        return y if residual is None else residual.add_(y)
    key = (w_gate_up.data_ptr(), w_down.data_ptr())
    if key not in _moe_cache:
        _moe_cache[key] = (interleave_experts(w_gate_up), w_down.reshape(E * H, I).contiguous())
    gu, dn = _moe_cache[key]
    if router_logits is None:
        router_logits = gemm(x, gate_w, epi=EPI_STORE_F32) if gemm_supported(T, E, H) else torch.nn.functional.linear(x, gate_w)
    on_device = E <= 256 and T * top_k <= 16384
    if on_device:    # router + permutation kernels: int32 order, no host synchronisation, static shapes
        order, row_w, group_off, _, tok = moe_route_sort(router_logits.float(), top_k, renorm, 0, E, with_tokens=True)
    else:
        order, row_w, group_off, _ = route_and_sort(router_logits, top_k, renorm, 0, E)
        tok = torch.div(order, top_k, rounding_mode="floor")
    if on_device and x.dtype == torch.bfloat16 and x.stride(1) == 1:
        xs = torch.empty(T * top_k, H, dtype=x.dtype, device=x.device)
        gather_rows(x, tok, xs)                   # expert-sorted copy of the token rows
    else:
        xs = x.index_select(0, tok)
    h = torch.empty(T * top_k, I, dtype=x.dtype, device=x.device)
    ys = torch.empty(T * top_k, H, dtype=x.dtype, device=x.device)
    st = _p(status_word(x.device))
    # launch for a few times the balanced rows per expert (an expert can hold at most T rows); hotter experts are
    # finished by their CTAs walking on through the remaining row tiles, empty tiles are never launched in bulk
    cover = min(T, ((4 * T * top_k // E + 128 + 127) // 128) * 128)
    _check(lib.js_gemm_bf16_grouped(_p(xs), _p(gu), _p(h), T * top_k, 2 * I, H, xs.stride(0), gu.stride(0), h.stride(0),
                                    EPI_SWIGLU, E, _p(group_off), cover, None, None, None, None, 1, st, 0, _stream()),
           "grouped gate/up")
    _check(lib.js_gemm_bf16_grouped(_p(h), _p(dn), _p(ys), T * top_k, H, I, h.stride(0), dn.stride(0), ys.stride(0),
                                    EPI_STORE, E, _p(group_off), cover, None, None, None, None, 1, st, 0, _stream()),
           "grouped down")
    if on_device and x.dtype == torch.bfloat16:
        # weighted sum of each token's expert outputs in choice order (fixed order, no atomics)
        fused = residual is not None and residual.dtype == x.dtype and residual.stride(1) == 1
        out = residual if fused else torch.empty(T, H, dtype=x.dtype, device=x.device)
        inv = torch.empty(T * top_k, dtype=torch.int32, device=x.device)
        lib.js_moe_combine.restype = ctypes.c_int
        _check(lib.js_moe_combine(_p(ys), ys.stride(0), _p(order), _p(row_w), T, top_k, H, _p(inv),
                                  _p(residual) if fused else None, _p(out), out.stride(0), 0, _stream()),
               "js_moe_combine")
        return out if fused or residual is None else residual.add_(out)
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    out.index_add_(0, tok.long(), ys.float() * row_w[:, None])
    out = out.to(x.dtype)
    return out if residual is None else residual.add_(out)
