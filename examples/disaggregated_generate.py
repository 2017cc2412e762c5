"""Target on GPU 0, draft head on GPU 1 (two processes, NVLink peer memory between them).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/disaggregated_generate.py

Rank 0 owns the target and drives `generate_tree` with a `RemoteDraftHead`; rank 1 serves draft steps with a
`DraftWorker`.  Tapped hidden rows, the accepted path and the drafted top-k cross GPUs inside the CUDA graphs.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from jetspec_b200 import JetSpecEngine, SamplingParams  # noqa: E402
from jetspec_b200.engine.disagg import DraftWorker, RemoteDraftHead  # noqa: E402
from jetspec_b200.models import DraftHeadModel, Qwen3Config, Qwen3ForCausalLM, draft_head_config  # noqa: E402
from jetspec_b200.parallel.handoff import HandoffChannel  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank = dist.get_rank()
    cfg = Qwen3Config(vocab_size=8192, hidden_size=1024, intermediate_size=2048, num_hidden_layers=4,
                      num_attention_heads=8, num_key_value_heads=8, head_dim=128)
    model = Qwen3ForCausalLM.random_init(cfg, seed=0, dtype=torch.bfloat16, device="cuda", init="stable")
    taps, D, K, budget = [0, 1, 3], 8, 4, 32
    head = DraftHeadModel.random_init(draft_head_config(cfg, 1, D + 1, target_layer_ids=taps), seed=5,
                                      dtype=torch.bfloat16, device="cuda")
    chan = HandoffChannel(None, nodes=32, tap_width=len(taps) * cfg.hidden_size, depth=D, width=K)
    if rank == 0:
        eng = JetSpecEngine(model, device=f"cuda:{local}", dtype=torch.bfloat16, max_seq_len=512)
        prompt = torch.randint(0, cfg.vocab_size, (1, 40), generator=torch.Generator().manual_seed(0))
        out = eng.generate_tree(prompt, RemoteDraftHead(chan, taps, D + 1), tree_depth=D, tree_width=K, budget=budget,
                                sampling_params=SamplingParams(0.0, 48), return_stats=True)
        print(f"{len(out['token_ids'])} tokens in {out['rounds']} rounds: {out['token_ids'][:12]} ...")
    else:
        steps = DraftWorker(head, model.model.embed_tokens.weight, model.lm_head.weight, chan, width=K,
                            vocab_size=cfg.vocab_size, max_ctx=512).serve()
        print(f"draft worker served {steps} steps")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
