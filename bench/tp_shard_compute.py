"""Compute-only twin of a tensor-parallel decode round: ONE GPU runs the per-rank work of a TP=N job without any
communication, i.e. the headline benchmark on a model whose heads, MLP width and vocabulary slice are 1/N of
Qwen3-8B's (the draft head keeps its full-size layer, as it does under real TP).  The difference between this
round time and the measured TP=N round time is what the collectives and rank skew cost.

    python bench/tp_shard_compute.py --shards 4 --steps 3 --warmup 3

All other flags are those of ``bench.py``.  The JSON line is ``bench.py``'s own; read ``config.ms_per_round``
(``value`` and ``vs_baseline`` describe a model that is not the benchmark's and mean nothing here).
"""
from __future__ import annotations

import copy
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import bench
    import jetspec_b200.models as models
    from jetspec_b200.models import Qwen3Config
    argv = sys.argv[1:]
    shards = 4
    if "--shards" in argv:
        i = argv.index("--shards")
        shards = int(argv[i + 1])
        del argv[i:i + 2]
    full = bench.model_config("qwen3-8b")
    if full.num_attention_heads % shards or full.intermediate_size % shards or full.vocab_size % shards:
        raise SystemExit(f"--shards {shards} does not divide the model")

    def shard_config(_name):
        return Qwen3Config(vocab_size=full.vocab_size // shards, hidden_size=full.hidden_size,
                           intermediate_size=full.intermediate_size // shards,
                           num_hidden_layers=full.num_hidden_layers,
                           num_attention_heads=full.num_attention_heads // shards,
                           num_key_value_heads=max(1, full.num_key_value_heads // shards), head_dim=full.head_dim)

    real_head_config = models.draft_head_config

    def head_config(target, **kw):          # the head's own layer is replicated under TP: keep it full-size
        t = copy.copy(full)
        t.vocab_size = target.vocab_size
        return real_head_config(t, **kw)

    bench.model_config = shard_config
    models.draft_head_config = head_config
    print(f"[tp_shard_compute] one rank's share of TP={shards}, no collectives", file=sys.stderr)
    sys.argv = [os.path.join(ROOT, "bench.py")] + argv
    bench.main()


if __name__ == "__main__":
    main()
