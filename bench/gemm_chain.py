"""Per-shape GEMM time inside a CUDA-graph chain over rotating weight copies (L2-cold), ours against cuBLAS.

Every shape is launched back to back on ``R`` different weight matrices (more than twice the L2 in total), the whole
chain is one CUDA graph, and the figure printed is graph time / launches: this is how the GEMMs run inside a decode
round (cold weights, no host gaps), unlike a single launch between two events.

    python bench/gemm_chain.py                 # the four decoder shapes of Qwen3-8B at 128 rows, all configurations
    M=21 ONLY=qkv,down python bench/gemm_chain.py
    SHARDS=4 python bench/gemm_chain.py        # the same layer as one rank of a tensor-parallel job of 4 sees it
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from jetspec_b200.ops import cuda_ext as X  # noqa: E402

SHAPES = [("qkv", 6144, 4096, 0), ("o", 4096, 4096, 0), ("gu", 24576, 4096, 1), ("down", 4096, 12288, 0)]
HBM_GBS = 6548.0          # measured copy bandwidth of this pool's B200s


def chain_time(launch, n_copies: int, reps: int = 3) -> float:
    """Microseconds per launch of ``launch(i)`` run over ``n_copies`` operands twice inside one graph."""
    for i in range(n_copies):
        launch(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(2):
            for i in range(n_copies):
                launch(i)
    ts = []
    for _ in range(reps + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return min(ts[1:]) * 1e3 / (2 * n_copies)


def main():
    X.load()
    M = int(os.environ.get("M", 128))
    only = os.environ.get("ONLY")
    shards = int(os.environ.get("SHARDS", 1))       # column-parallel qkv / gate-up, row-parallel o / down
    shapes = [(n, N // shards if n in ("qkv", "gu") else N, K if n in ("qkv", "gu") else K // shards, e)
              for n, N, K, e in SHAPES]
    for name, N, K, epi in shapes:
        if only and name not in only.split(","):
            continue
        size = N * K * 2
        R = int(os.environ.get("COPIES", 0)) or max(4, (400 << 20) // size + 1)     # COPIES=1: weights stay in L2
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(R)]
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N // (2 if epi == 1 else 1), device="cuda", dtype=torch.bfloat16)
        full = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        res = {"cublas": round(chain_time(lambda i: torch.matmul(x, ws[i].t(), out=full), R), 1),
               "picked": round(chain_time(lambda i: X.gemm(x, ws[i], out=out, epi=epi, pdl=True), R), 1)}
        for deep in ((0, 2, 1) if not os.environ.get("PICKED_ONLY") else ()):
            for bn in (128, 256):
                for split in (1, 2, 3, 4, 6, 8):
                    for pdl in ((0, 1) if bn == 128 else (1,)):
                        try:
                            t = chain_time(lambda i: X.gemm(x, ws[i], out=out, epi=epi, bn=bn, split=split, deep=deep,
                                                            pdl=bool(pdl)), R)
                        except Exception:
                            continue
                        res[f"bn{bn}_budget{deep}_split{split}_pdl{pdl}"] = round(t, 1)
        if M >= 512 and not os.environ.get("PICKED_ONLY"):      # two row tiles per CTA (256 x 256 per CTA)
            try:
                res["bn256_two_row_tiles_pdl1"] = round(chain_time(
                    lambda i: X.gemm(x, ws[i], out=out, epi=epi, bn=256, split=1, deep=3, pdl=True), R), 1)
            except Exception:
                pass
        X.check_status("cuda")
        print(json.dumps({"shape": name, "M": M, "N": N, "K": K, "ideal_us_at_measured_copy_bw": round(size / HBM_GBS / 1e3, 1),
                          "picked_config": X.pick_gemm_config(M, N, K, epi), "us": res}), flush=True)
        del ws
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
