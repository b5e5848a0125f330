#!/usr/bin/env python
"""Walk through the inference modes of the recurrent-depth model (script form of the reference's
examples/inference_demo.ipynb): plain generation at a chosen depth, KV-cache sharing between recurrence steps and what it
does to cache memory, continuous compute (latent reuse), adaptive per-token depth, and the FLOP count per token.

Runs on CPU with a tiny random model by default; pass a local HF folder and a tokenizer folder for a real model.

    python examples/inference_demo.py
    python examples/inference_demo.py --model /path/to/hf_folder --tokenizer /path/to/tokenizer --device cuda
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from recurrent_pretraining_b200.models.hf import RavenForCausalLM  # noqa: E402
from recurrent_pretraining_b200.models.hf_config import RavenConfig  # noqa: E402
from recurrent_pretraining_b200.models.kv_cache import RecurrentKVCache  # noqa: E402


def tiny_model():
    torch.manual_seed(0)
    cfg = RavenConfig(n_embd=128, n_heads=4, n_layers=8, block_size=256, vocab_size=512, intermediate_size=256,
                      n_layers_in_recurrent_block=4, n_layers_in_prelude=2, n_layers_in_coda=2, mean_recurrence=8)
    return RavenForCausalLM(cfg).eval()


def section(title):
    print(f"\n=== {title} " + "=" * max(0, 70 - len(title)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--prompt", default="The capital of Westphalia is")
    ap.add_argument("--max_new_tokens", type=int, default=12)
    a = ap.parse_args(argv)
    if a.model:
        model = RavenForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16 if a.device != "cpu" else None)
        model = model.to(a.device).eval()
    else:
        model = tiny_model().to(a.device)
    if a.tokenizer:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(a.tokenizer)
        ids = torch.tensor([tok.encode(a.prompt)], device=a.device)
        show = lambda t: tok.decode(t)  # noqa: E731
    else:
        ids = torch.tensor([[b % model.config.vocab_size for b in a.prompt.encode()]], device=a.device)
        show = lambda t: " ".join(str(int(x)) for x in t)  # noqa: E731
    r = model.config.mean_recurrence

    section("1. generation at different recurrence depths")
    for steps in sorted({max(1, r // 4), r, 2 * r}):
        t0 = time.time()
        out = model.generate(ids, max_new_tokens=a.max_new_tokens, num_steps=steps, init_scale=0.0)
        print(f"num_steps={steps:3d}  {time.time() - t0:5.2f}s  ->  {show(out[0, ids.shape[1]:])}")

    section("2. KV-cache sharing across recurrence steps")
    for strategy in ("full", "latest-m4", f"latest-m4-compress-s{model.config.n_layers_in_recurrent_block}",
                     "latest-m4-compress-s16"):
        cache = RecurrentKVCache(lookup_strategy=strategy, core_layers=model.config.n_layers_in_recurrent_block,
                                 prelude_layers=model.config.n_layers_in_prelude)
        out = model.generate(ids, max_new_tokens=a.max_new_tokens, num_steps=r, init_scale=0.0,
                             cache_lookup_strategy=strategy, past_key_values=cache, return_dict_in_generate=True)
        kv = out["past_key_values"]
        print(f"{strategy:28s} cache {kv.get_memory_usage():8.3f} MiB  ->  {show(out['sequences'][0, ids.shape[1]:])}")

    section("3. continuous compute: start each token from the previous token's latent")
    out = model.generate(ids, max_new_tokens=a.max_new_tokens, num_steps=max(1, r // 4), continuous_compute=True)
    print(f"num_steps={max(1, r // 4)} with latent reuse  ->  {show(out[0, ids.shape[1]:])}")

    section("4. adaptive depth per token (exit when successive predictions agree)")
    for crit, thr in (("kl", 5e-4), ("entropy-diff", 1e-3), ("latent-diff", 0.03), ("argmax-stability", 5)):
        out = model.generate(ids, max_new_tokens=a.max_new_tokens, num_steps=2 * r, criterion=crit, exit_threshold=thr,
                             return_dict_in_generate=True)
        steps = [int(s[0]) if isinstance(s, (list, tuple)) else int(s) for s in out["scores"].get("compute_steps", [])]
        mean = sum(steps) / max(len(steps), 1)
        print(f"{crit:18s} mean steps {mean:5.1f} of {2 * r}  per token {steps}")

    section("5. FLOPs per generated token")
    c = model.config
    E, I, V = c.n_embd, c.intermediate_size, c.vocab_size
    per_block = 2 * (3 * E * E + E * E + 3 * E * I)
    fixed = (c.n_layers_in_prelude + c.n_layers_in_coda) * per_block + 2 * E * V
    for steps in (r // 2, r, 2 * r):
        total = fixed + steps * (c.n_layers_in_recurrent_block * per_block + 2 * 2 * E * E)
        print(f"num_steps={steps:3d}: {total / 1e9:8.3f} GFLOP per token (weights only, attention over the cache not counted)")


if __name__ == "__main__":
    main()
