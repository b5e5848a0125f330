"""Compare what the model says at different recurrence depths, for one prompt or in a small REPL.

Counterpart of evaluate_raven/quick_chat_rec_compare.py:52-219.

    python -m recurrent_pretraining_b200.evaluate.chat_compare --model /path/to/hf_folder --tokenizer /path/to/tok \
        --recurrences 4 8 16 32 64
"""
from __future__ import annotations

import argparse
import time

import torch


@torch.no_grad()
def compare(model, encode, decode, prompt: str, recurrences=(4, 8, 16, 32), max_new_tokens: int = 64,
            adaptive: bool = False, exit_threshold: float = 5e-4) -> list[dict]:
    """One greedy continuation per recurrence count (plus, optionally, a KL-adaptive one capped at the largest count);
    returns [{num_steps, text, seconds, tokens_per_second, mean_steps}]."""
    device = next(model.parameters()).device
    ids = torch.tensor([encode(prompt)], device=device)
    rows = []
    settings = [dict(num_steps=r) for r in recurrences]
    if adaptive:
        settings.append(dict(num_steps=max(recurrences), criterion="kl", exit_threshold=exit_threshold))
    for kw in settings:
        t0 = time.time()
        out = model.generate(ids, max_new_tokens=max_new_tokens, return_dict_in_generate=True, **kw)
        dt = time.time() - t0
        seq = out["sequences"][0, ids.shape[1]:].tolist()
        steps = out["scores"].get("compute_steps") if isinstance(out.get("scores"), dict) else None
        mean_steps = kw["num_steps"]
        if steps:
            flat = [float(s) for tok in steps for s in (tok if isinstance(tok, (list, tuple)) else [tok])]
            mean_steps = sum(flat) / max(len(flat), 1)
        rows.append({"num_steps": kw["num_steps"], "adaptive": "criterion" in kw, "text": decode(seq),
                     "seconds": round(dt, 3), "tokens_per_second": round(len(seq) / max(dt, 1e-9), 2),
                     "mean_steps": round(mean_steps, 2)})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--recurrences", type=int, nargs="+", default=[4, 8, 16, 32])
    ap.add_argument("--max_new_tokens", type=int, default=128)
    ap.add_argument("--adaptive", action="store_true")
    ap.add_argument("--prompt", default=None, help="one-shot mode; without it a REPL starts")
    a = ap.parse_args(argv)
    from transformers import AutoTokenizer

    from ..models.hf import RavenForCausalLM

    tok = AutoTokenizer.from_pretrained(a.tokenizer)
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    model = RavenForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16 if dev != "cpu" else torch.float32)
    model = model.to(dev).eval()

    def once(prompt):
        for row in compare(model, lambda s: tok.encode(s), tok.decode, prompt, a.recurrences, a.max_new_tokens,
                           a.adaptive):
            tag = f"r={row['num_steps']}" + (" (kl-adaptive)" if row["adaptive"] else "")
            print(f"--- {tag}: {row['tokens_per_second']} tok/s, mean steps {row['mean_steps']}\n{row['text']}\n")

    if a.prompt:
        return once(a.prompt)
    while True:
        try:
            prompt = input("prompt> ")
        except EOFError:
            break
        if prompt.strip() in ("", "quit", "exit"):
            break
        once(prompt)


if __name__ == "__main__":
    main()
