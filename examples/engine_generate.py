"""Paged engine: AR vs batched decode, checking that a batch reproduces per-prompt outputs.

    python examples/engine_generate.py [/path/to/model]

Reference counterpart: ``examples/engine/jetspec_engine_generate.py:19-64``."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout

from jetspec_b200 import JetSpecEngine, SamplingParams  # noqa: E402
from jetspec_b200.models import Qwen3ForCausalLM, tiny_config  # noqa: E402

if __name__ == "__main__":
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    model = sys.argv[1] if len(sys.argv) > 1 else Qwen3ForCausalLM.random_init(tiny_config(), seed=0, dtype=dt)
    eng = JetSpecEngine(model, device=dev, dtype=dt, block_size=16)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.cfg.vocab_size, (1, n), generator=g) for n in (7, 19, 12)]
    sp = SamplingParams(0.0, 24)
    singles = [eng.generate(p, sp)["token_ids"] for p in prompts]
    batch = [r["token_ids"] for r in eng.generate_batch(prompts, sp)]
    print("batch == single:", [a == b for a, b in zip(batch, singles)], eng.last_stats)
