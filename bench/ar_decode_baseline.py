"""Raw autoregressive decode baseline: prefill, then one-token steps, decode-only timing.

The denominator of every "speedup over autoregressive decoding" figure, measured on its own (counterpart of the
reference's ``bench/reference/hf_fa2_decode_baseline.py:52-199``, which times a stock Hugging Face model with
FlashAttention-2).  Three arms on the same prompt, each reporting prefill time, decode time and decode tokens/s:

* ``engine``: this framework's paged engine; on a GPU every step is one CUDA-graph replay of the kernel path
  (``JetSpecEngine.generate``), timed on the device around the steps only;
* ``llm``: the reference-style engine (``LLM.generate``: contiguous cache, module forward per step);
* ``hf`` (``--hf DIR``): a stock ``transformers`` model loaded from a checkpoint directory, plain
  ``model(...)`` steps with its own KV cache, when ``transformers`` can load the directory.

    python bench/ar_decode_baseline.py --model qwen3-8b --prompt-len 512 --new 256
    python bench/ar_decode_baseline.py --model small --new 32            # runs on CPU too
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def time_engine(eng, prompt, new: int) -> dict:
    """Prefill and decode timed separately: a 1-token request isolates the prefill, the rest is decode."""
    from jetspec_b200 import SamplingParams
    eng.generate(prompt, SamplingParams(0.0, 4))                    # warm-up: pool, module load, graph capture
    _sync()
    t0 = time.perf_counter()
    eng.generate(prompt, SamplingParams(0.0, 1))
    _sync()
    prefill = time.perf_counter() - t0
    t0 = time.perf_counter()
    out = eng.generate(prompt, SamplingParams(0.0, new))
    _sync()
    total = time.perf_counter() - t0
    n = len(out["token_ids"])
    decode = max(total - prefill, 1e-9)
    return {"output_tokens": n, "prefill_time": prefill, "decode_time": decode,
            "decode_tokens_per_s": (n - 1) / decode if n > 1 else 0.0, "e2e_tokens_per_s": n / total}


def time_llm(llm, prompt, new: int) -> dict:
    from jetspec_b200 import SamplingParams
    llm.generate(prompt, SamplingParams(0.0, 2))
    _sync()
    t0 = time.perf_counter()
    llm.generate(prompt, SamplingParams(0.0, 1))
    _sync()
    prefill = time.perf_counter() - t0
    t0 = time.perf_counter()
    out = llm.generate(prompt, SamplingParams(0.0, new))
    _sync()
    total = time.perf_counter() - t0
    n = len(out["token_ids"])
    decode = max(total - prefill, 1e-9)
    return {"output_tokens": n, "prefill_time": prefill, "decode_time": decode,
            "decode_tokens_per_s": (n - 1) / decode if n > 1 else 0.0, "e2e_tokens_per_s": n / total}


@torch.inference_mode()
def time_hf(path: str, prompt, new: int, device: str, dtype) -> dict:
    from transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(path, dtype=dtype).to(device).eval()
    ids = prompt.to(device)
    _sync()
    t0 = time.perf_counter()
    out = model(input_ids=ids, use_cache=True, logits_to_keep=1)
    _sync()
    prefill = time.perf_counter() - t0
    cache, tok = out.past_key_values, out.logits[:, -1].argmax(-1, keepdim=True)
    n = 1
    t0 = time.perf_counter()
    for _ in range(new - 1):
        out = model(input_ids=tok, past_key_values=cache, use_cache=True, logits_to_keep=1)
        cache, tok = out.past_key_values, out.logits[:, -1].argmax(-1, keepdim=True)
        n += 1
    _sync()
    decode = max(time.perf_counter() - t0, 1e-9)
    return {"output_tokens": n, "prefill_time": prefill, "decode_time": decode,
            "decode_tokens_per_s": (n - 1) / decode if n > 1 else 0.0, "e2e_tokens_per_s": n / (prefill + decode)}


def main():
    from bench import model_config
    from jetspec_b200 import JetSpecEngine, LLM
    from jetspec_b200.models import Qwen3ForCausalLM
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b", choices=["qwen3-8b", "qwen3-30b-a3b", "small"])
    ap.add_argument("--checkpoint", default=None, help="a checkpoint directory instead of random-init weights")
    ap.add_argument("--hf", default=None, help="also time a stock transformers model loaded from this directory")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--arms", default="engine,llm")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev, dt = ("cuda", torch.bfloat16) if cuda else ("cpu", torch.float32)
    cfg = model_config(args.model)
    model = (Qwen3ForCausalLM.from_pretrained(args.checkpoint, dtype=dt, device=dev) if args.checkpoint
             else Qwen3ForCausalLM.random_init(cfg, seed=args.seed, dtype=dt, device=dev, init="stable"))
    prompt = torch.randint(0, model.config.vocab_size, (1, args.prompt_len),
                           generator=torch.Generator().manual_seed(args.seed))
    res = {"bench": "autoregressive decode baseline", "model": args.checkpoint or args.model,
           "prompt_len": args.prompt_len, "new_tokens": args.new, "dtype": str(dt).split(".")[-1]}
    arms = [a.strip() for a in args.arms.split(",") if a.strip()]
    if "engine" in arms:
        eng = JetSpecEngine(model, device=dev, dtype=dt, max_seq_len=args.prompt_len + args.new + 64)
        res["engine"] = time_engine(eng, prompt, args.new)
    if "llm" in arms:
        res["llm"] = time_llm(LLM(model, device=dev, dtype=dt), prompt, args.new)
    if args.hf:
        try:
            res["hf"] = time_hf(args.hf, prompt, args.new, dev, dt)
        except Exception as e:  # noqa: BLE001 - a checkpoint transformers cannot load is reported, not fatal
            res["hf"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
