"""Quantise a target's linears to NVFP4 and decode with the tree engine.

    python examples/nvfp4_generate.py [MODEL_DIR]

Without a model directory a small random-init Qwen3 stands in (GPU: block-scaled tcgen05 GEMMs; CPU: the oracle).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from jetspec_b200 import JetSpecEngine, RandomTreeDrafter, SamplingParams  # noqa: E402
from jetspec_b200.models import Qwen3Config, Qwen3ForCausalLM  # noqa: E402
from jetspec_b200.models.nvfp4 import quantize_model_nvfp4  # noqa: E402


def main():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    if len(sys.argv) > 1:
        model = Qwen3ForCausalLM.from_pretrained(sys.argv[1], dtype=dt).to(dev)
    else:
        cfg = Qwen3Config(vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=128)
        model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=dt, device=dev, init="stable")
    n = quantize_model_nvfp4(model)
    print(f"{n} linear layers now hold e2m1 codes + e4m3 block scales")
    eng = JetSpecEngine(model, device=dev, dtype=dt, max_seq_len=512)
    prompt = torch.randint(0, model.config.vocab_size, (1, 32), generator=torch.Generator().manual_seed(0))
    sp = SamplingParams(0.0, 32)
    ar = eng.generate(prompt, sp)["token_ids"]
    out = eng.generate_tree(prompt, RandomTreeDrafter(model.config.vocab_size, seed=1), tree_depth=4, tree_width=2,
                            budget=8, sampling_params=sp, return_stats=True)
    print("greedy :", ar[:16])
    print("tree   :", out["token_ids"][:16], f"({out['rounds']} rounds, lossless: {out['token_ids'] == ar})")


if __name__ == "__main__":
    main()
