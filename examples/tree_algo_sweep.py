"""Sweep tree algorithms x budgets and report tokens per verify forward and the exact-prefix length
against plain greedy decoding (bf16 may flip a near-tie after many exact tokens; fp32 is exact).

Environment: JETSPEC_SWEEP_BUDGETS="8,16,32", JETSPEC_SWEEP_WIDTH=4, JETSPEC_SWEEP_MAXNEW=48.
Reference counterpart: ``examples/tree/jetspec_tree_algo_sweep.py:55-120`` (exact-prefix report ``:69-74``)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout

from jetspec_b200 import JetSpecEngine, SamplingParams, TargetEchoTreeDrafter  # noqa: E402
from jetspec_b200.models import Qwen3ForCausalLM, tiny_config  # noqa: E402
from jetspec_b200.tree import list_algorithms  # noqa: E402
from jetspec_b200.utils import env_int, env_str  # noqa: E402

if __name__ == "__main__":
    budgets = [int(b) for b in env_str("JETSPEC_SWEEP_BUDGETS", "8,16,32").split(",")]
    width, max_new = env_int("JETSPEC_SWEEP_WIDTH", 4), env_int("JETSPEC_SWEEP_MAXNEW", 48)
    model = Qwen3ForCausalLM.random_init(tiny_config(), seed=0)
    eng = JetSpecEngine(model, device="cpu", dtype=torch.float32)
    prompt = torch.randint(0, 1024, (1, 24), generator=torch.Generator().manual_seed(0))
    sp = SamplingParams(0.0, max_new)
    greedy = eng.generate(prompt, sp)["token_ids"]
    drafter = TargetEchoTreeDrafter(model)
    print(f"{'algorithm':24s} {'budget':>6s} {'tok/fwd':>8s} {'exact prefix':>12s}")
    for algo in list_algorithms():
        for b in budgets:
            out = eng.generate_tree(prompt, drafter, block_size=7, tree_width=width, budget=b, algo=algo, sampling_params=sp)
            exact = next((i for i, (x, y) in enumerate(zip(out["token_ids"], greedy)) if x != y), len(greedy))
            print(f"{algo:24s} {b:6d} {out['tpf']:8.2f} {exact:12d}")
