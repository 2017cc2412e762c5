"""Tree-speculative decoding with a draft head (README quick-start of the reference, same call).

    python examples/tree_generate.py /path/to/Qwen3-8B /path/to/draft-head "prompt"

Without arguments: tiny random target + random head on CPU (lossless, low acceptance).
Reference counterpart: ``examples/tree/jetspec_tree_generate.py:25-51``."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout

from jetspec_b200 import JetSpecEngine, SamplingParams, DraftHeadTreeDrafter, load_draft_head  # noqa: E402
from jetspec_b200.models import Qwen3ForCausalLM, DraftHeadModel, draft_head_config, tiny_config  # noqa: E402

if __name__ == "__main__":
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = torch.bfloat16 if dev == "cuda" else torch.float32
    if len(sys.argv) > 2:
        eng = JetSpecEngine(sys.argv[1], device=dev, dtype=dt, block_size=16)
        head = load_draft_head(sys.argv[2], device=dev, dtype=dt)
        prompt = sys.argv[3] if len(sys.argv) > 3 else "Explain speculative decoding in one paragraph."
        depth, width, budget = 20, 7, 128
    else:
        cfg = tiny_config()
        eng = JetSpecEngine(Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=dt), device=dev, dtype=dt)
        head = DraftHeadModel.random_init(draft_head_config(cfg, 1, 5, target_layer_ids=[0, 1]), seed=1, dtype=dt, device=dev)
        prompt = torch.randint(0, cfg.vocab_size, (1, 16))
        depth, width, budget = 4, 2, 8
    drafter = DraftHeadTreeDrafter(head, eng.model, block_size=depth + 1, target_layer_ids=head.target_layer_ids)
    out = eng.generate_tree(prompt, drafter, tree_depth=depth, tree_width=width, budget=budget,
                            target_layer_ids=head.target_layer_ids, sampling_params=SamplingParams(0.0, 64),
                            return_stats=True)
    print(out["text"] or out["token_ids"])
    print(f"tokens/round {out['tpf']:.2f} over {out['rounds']} rounds")
