"""Decode throughput of raven-3.5B on one GPU (one replica): prompt 512 uniform-random tokens, 256 generated tokens,
greedy, r = 32 with the per-recurrence-step KV cache; optional KL exit (5e-4, max r 64) with latent reuse.

``python -m recurrent_pretraining_b200.utils.decode_bench [--batches 1,8,32,64] [--new 256] [--prompt 512] [--kl]
[--eager] [--reference]``.  Device-timed with CUDA events around the generation loop (prefill excluded and reported
separately); weights are random-init.  ``--eager`` times this repository's HF-style token loop, ``--reference`` the
unmodified reference HF model in a hand-written cached loop (its ``generate`` no longer runs under transformers 5).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def build_model(name):
    from ..config import ModelConfig
    from ..models.hf import RavenForCausalLM
    from ..models.hf_config import RavenConfig

    cfg = ModelConfig.from_name(name)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = RavenForCausalLM(RavenConfig.from_model_config(cfg))
    return model.to(torch.bfloat16).eval()


def time_region(fn):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="nebel-raven-3.5b")
    ap.add_argument("--batches", default="1,8,32,64")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--kl", action="store_true")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--reference", action="store_true")
    ap.add_argument("--cache", default="full")
    ap.add_argument("--profile", action="store_true", help="print per-kernel time shares of a few decode tokens")
    args = ap.parse_args()
    from ..engine.decode import DecodeEngine

    model = build_model(args.model)
    V = model.config.padded_vocab_size
    for B in [int(b) for b in args.batches.split(",")]:
        ids = torch.randint(0, V - 100, (B, args.prompt), device="cuda")
        rec = {"model": args.model, "batch": B, "prompt": args.prompt, "new_tokens": args.new, "r": args.steps,
               "cache": args.cache}
        max_steps = 64 if args.kl else args.steps
        eng = DecodeEngine(model, B, args.prompt + args.new + 1, num_steps=args.steps, cache_lookup_strategy=args.cache,
                           max_steps=max_steps)
        rec["kv_cache_GiB"] = round(eng.cache.get_memory_usage() / 1024, 2)
        kw = dict(criterion="kl", exit_threshold=5e-4, max_steps=64, continuous_compute=True) if args.kl else {}
        eng.generate(ids, 4, **kw)  # warm-up: graph capture
        t_pre, _ = time_region(lambda: eng.prefill(ids, args.steps))
        t_all, (toks, stats) = time_region(lambda: eng.generate(ids, args.new, **kw))
        t_dec = t_all - t_pre
        mean_r = sum(sum(s) for s in stats["steps"]) / max(1, B * len(stats["steps"]))
        rec.update({"engine_prefill_ms": round(t_pre, 1), "engine_decode_tok_s": round(B * (args.new - 1) / (t_dec / 1e3), 1),
                    "engine_ms_per_token": round(t_dec / (args.new - 1), 2), "mean_recurrence": round(mean_r, 2),
                    "weight_stream_GBps": round(eng.weight_bytes_per_recurrence * mean_r / (t_dec / (args.new - 1)) / 1e6, 0),
                    "device_status": stats["device_status"]})
        if args.profile:
            from torch.profiler import ProfilerActivity, profile

            eng.prefill(ids, args.steps)
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                eng.generate(ids, 4, **kw)
                torch.cuda.synchronize()
            rows = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
            total = sum(e.device_time_total for e in rows)
            print(f"profile batch {B}: total kernel time {total / 1e3:.1f} ms (prefill + 3 tokens)")
            for e in rows[:18]:
                print(f"{e.device_time_total / 1e3:9.2f} ms {100 * e.device_time_total / total:5.1f}%  x{e.count:6d}  {e.key[:100]}")
        del eng
        torch.cuda.empty_cache()
        if args.eager and B <= 8:
            n = min(args.new, 16)
            t, _ = time_region(lambda: model.generate(ids, max_new_tokens=n, num_steps=args.steps))
            rec["eager_loop_tok_s"] = round(B * n / (t / 1e3), 2)
        print(json.dumps(rec), flush=True)
    if args.reference:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                        "baseline"))
        import refload

        mod = refload.module("raven_modeling_minimal")
        mod.RavenForCausalLM._tied_weights_keys = {"lm_head.weight": "transformer.wte.weight"}
        cfgmod = refload.module("raven_config_minimal")
        with torch.device("cuda"):
            ref_model = mod.RavenForCausalLM(cfgmod.RavenConfig()).to(torch.bfloat16).eval()
        for B in [int(b) for b in args.batches.split(",") if int(b) <= 8]:
            ids = torch.randint(0, V - 100, (B, args.prompt), device="cuda")
            n = 8

            def loop():
                with torch.no_grad():
                    cache = mod.HuginnDynamicCache()
                    out = ref_model(ids, num_steps=args.steps, use_cache=True, past_key_values=cache,
                                    cache_position=torch.arange(args.prompt, device="cuda"))
                    tok = out.logits[:, -1].argmax(-1, keepdim=True)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for t in range(n):
                        out = ref_model(tok, num_steps=args.steps, use_cache=True, past_key_values=cache,
                                        cache_position=torch.tensor([args.prompt + t], device="cuda"))
                        tok = out.logits[:, -1].argmax(-1, keepdim=True)
                    e1.record()
                    torch.cuda.synchronize()
                    return e0.elapsed_time(e1)

            ms = loop()
            print(json.dumps({"impl": "reference HF hand loop", "batch": B, "decode_tok_s": round(B * n / (ms / 1e3), 2),
                              "ms_per_token": round(ms / n, 1)}), flush=True)


if __name__ == "__main__":
    main()
