"""Per-sample benchmark scores as a function of the recurrence depth ("saturation" curves): run one task at one depth
and store the list of per-sample scores, so that curves over depth can be assembled and bootstrapped afterwards.

Counterpart of evaluate_raven/saturation_eval_dist.py:1-93 and misc_benchmark_variants/eval_alternate_loops.py.  The
harness itself (lm-eval) is an optional import; ``sample_scores`` -- which metric of which sample stream counts for a
task family -- and the sweep / file logic run without it (``evaluate_fn`` can be any callable returning an lm-eval
style result dict)."""
from __future__ import annotations

import os
from typing import Callable, Iterable, Optional

import torch

# task-name fragment -> (metric key, filter name or None, "all streams" flag)
_RULES = (("gsm8k", "exact_match", "flexible-extract", False), ("mmlu", "acc", None, True),
          ("blimp", "acc", None, True), ("bbh", "acc_norm", None, True), ("musr", "acc_norm", None, True),
          ("minerva", "math_verify", None, True), ("ifeval", "prompt_level_loose_acc", None, False),
          ("humaneval", "pass@1", None, False), ("mbpp", "pass@1", None, False),
          ("triviaqa", "exact_match,remove_whitespace", None, False),
          ("fld_default", "exact_match,remove_whitespace", None, False))
_STREAM = {"mastermind": "mastermind_46_hard", "acp_bench": "acp_app_mcq"}


def sample_scores(task: str, results: dict) -> list:
    """The per-sample scores that the saturation charts use for ``task`` out of an lm-eval result dict."""
    samples = results["samples"]
    for frag, stream in _STREAM.items():
        if frag in task:
            return [s["acc"] for s in samples[stream]]
    for frag, key, flt, all_streams in _RULES:
        if frag in task:
            rows = [s for k in samples for s in samples[k]] if all_streams else samples[task]
            return [s[key] for s in rows if flt is None or s.get("filter") == flt]
    rows = samples[task]
    return [s["acc_norm"] if "acc_norm" in s else s["acc"] for s in rows]


def lm_eval_fn(model_wrapper, num_fewshot: int = 0, limit=None, use_chat: bool = False) -> Callable:
    """An ``evaluate_fn`` backed by lm-eval (import-gated)."""
    def run(task: str) -> dict:
        from lm_eval import evaluator  # type: ignore

        return evaluator.simple_evaluate(model=model_wrapper, tasks=[task], num_fewshot=num_fewshot, limit=limit,
                                         apply_chat_template=use_chat, fewshot_as_multiturn=use_chat,
                                         system_instruction="You are a helpful assistant." if use_chat else None)

    return run


def saturation_eval(task: str, num_steps: int, set_recurrence: Callable[[int], None], evaluate_fn: Callable[[str], dict],
                    num_fewshot: int = 0, out_dir: str = ".") -> str:
    """Evaluate ``task`` at ``num_steps`` recurrences; writes ``saturation_{task}_{num_steps}_{num_fewshot}.pth`` holding
    ``{num_steps: [per-sample scores]}`` and returns the path."""
    set_recurrence(num_steps)
    scores = sample_scores(task, evaluate_fn(task))
    path = os.path.join(out_dir, f"saturation_{task}_{num_steps}_{num_fewshot}.pth")
    torch.save({num_steps: scores}, path)
    return path


def sweep(task: str, depths: Iterable[int], set_recurrence, evaluate_fn, num_fewshot: int = 0, out_dir: str = ".",
          done: Optional[Callable[[int, float], None]] = None) -> dict:
    """Mean score per depth (the alternate-loops evaluation); every depth also leaves its per-sample file."""
    curve = {}
    for d in depths:
        path = saturation_eval(task, d, set_recurrence, evaluate_fn, num_fewshot, out_dir)
        vals = torch.load(path)[d]
        curve[d] = float(sum(vals)) / max(len(vals), 1)
        if done is not None:
            done(d, curve[d])
    return curve


def main(argv=None) -> None:
    import argparse

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--pretrained", required=True, help="HF folder written by evaluate.convert_to_hf")
    ap.add_argument("--task", default="ifeval")
    ap.add_argument("--num_steps", type=int, nargs="+", default=[32])
    ap.add_argument("--num_fewshot", type=int, default=0)
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--use_chat", action="store_true")
    ap.add_argument("--out_dir", default=".")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    from transformers import AutoTokenizer

    from ..models.hf import RavenForCausalLM
    from .lm_eval_wrapper import RecurrentLM

    model = RavenForCausalLM.from_pretrained(args.pretrained).to(args.device).to(torch.bfloat16)
    lm = RecurrentLM(model, AutoTokenizer.from_pretrained(args.pretrained), device=args.device)
    curve = sweep(args.task, args.num_steps, lambda d: setattr(lm, "recurrence", d),
                  lm_eval_fn(lm, args.num_fewshot, args.limit, args.use_chat), args.num_fewshot, args.out_dir,
                  done=lambda d, v: print(f"{args.task} @ {d} recurrences: {v:.4f}", flush=True))
    print(curve)


if __name__ == "__main__":
    main()
