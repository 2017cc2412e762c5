"""Plain autoregressive generation with the reference engine (`LLM`).

    python examples/simple_generate.py /path/to/Qwen3-8B "The capital of France is"

Without arguments a tiny random-init model is used so the script runs anywhere (CPU included).
Reference counterpart: ``examples/basic/simple_generate.py:10-21``."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout

from jetspec_b200 import LLM, SamplingParams  # noqa: E402
from jetspec_b200.models import Qwen3ForCausalLM, tiny_config  # noqa: E402

if __name__ == "__main__":
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    if len(sys.argv) > 1:
        llm = LLM(sys.argv[1], device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
        prompt = sys.argv[2] if len(sys.argv) > 2 else "Hello"
    else:
        llm = LLM(Qwen3ForCausalLM.random_init(tiny_config(), seed=0), device="cpu", dtype=torch.float32)
        prompt = torch.randint(0, 1024, (1, 16))
    out = llm.generate(prompt, SamplingParams(temperature=0.0, max_new_tokens=32))
    print(out["text"] or out["token_ids"])
