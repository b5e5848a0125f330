"""Command line in the shape of ``lm_eval`` for checkpoints of this framework, importing the local model code instead
of Hub remote code:

    python -m recurrent_pretraining_b200.evaluate.local_lm_eval --model_args pretrained=out/hf,mean_recurrence=32 \
        --tasks hellaswag,arc_easy --batch_size 8 --gen_kwargs criterion=entropy-diff,exit_threshold=1e-2

Counterpart of evaluate_raven/local_lm_eval.py (a copy of the harness CLI that imports the local ``recpre``).  Here the
argument handling is this module's own; the harness is imported only when tasks are actually run.  ``pretrained`` may
be an HF folder (``evaluate.convert_to_hf``) or a training checkpoint ``.pth``."""
from __future__ import annotations

import argparse
import json
from typing import Optional


def parse_kv(text: Optional[str]) -> dict:
    """``a=1,b=x,c=1e-2`` -> dict with ints / floats / bools / strings."""
    out = {}
    for part in filter(None, (text or "").split(",")):
        k, _, v = part.partition("=")
        v = v.strip()
        if v.lower() in ("true", "false"):
            out[k.strip()] = v.lower() == "true"
            continue
        for cast in (int, float):
            try:
                out[k.strip()] = cast(v)
                break
            except ValueError:
                continue
        else:
            out[k.strip()] = v
    return out


def build_lm(model_args: dict, gen_kwargs: dict, batch_size: int, device: str, tokenizer=None):
    """The scoring wrapper for ``model_args``: adaptive when ``gen_kwargs`` name an exit criterion."""
    import torch

    from .adaptive_eval import AdaptiveComputeLM
    from .lm_eval_wrapper import RecurrentLM

    path = model_args["pretrained"]
    recurrence = model_args.get("mean_recurrence")
    if str(path).endswith(".pth"):
        if tokenizer is None:
            raise ValueError("a training checkpoint needs --tokenizer")
        return RecurrentLM.from_checkpoint(path, tokenizer, device=device, batch_size=batch_size, recurrence=recurrence)
    from ..models.hf import RavenForCausalLM

    model = RavenForCausalLM.from_pretrained(path)
    dtype = model_args.get("dtype", "bfloat16")
    model = model.to(device).to(getattr(torch, dtype) if isinstance(dtype, str) else dtype)
    if tokenizer is None:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(model_args.get("tokenizer", path))
    common = dict(device=device, batch_size=batch_size, recurrence=recurrence)
    if "criterion" in gen_kwargs:
        return AdaptiveComputeLM(model, tokenizer, criterion=gen_kwargs["criterion"],
                                 exit_threshold=gen_kwargs.get("exit_threshold", "auto"),
                                 lookup_strategy=gen_kwargs.get("cache_lookup_strategy", "full"),
                                 continuous_compute=bool(gen_kwargs.get("continuous_compute", False)), **common)
    return RecurrentLM(model, tokenizer, **common)


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="hf", help="accepted for command-line compatibility; the local model is used")
    ap.add_argument("--model_args", required=True)
    ap.add_argument("--tasks", required=True)
    ap.add_argument("--num_fewshot", type=int, default=None)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--limit", type=float, default=None)
    ap.add_argument("--gen_kwargs", default=None)
    ap.add_argument("--apply_chat_template", action="store_true")
    ap.add_argument("--output_path", default=None)
    ap.add_argument("--tokenizer", default=None)
    args = ap.parse_args(argv)
    gen_kwargs = parse_kv(args.gen_kwargs)
    lm = build_lm(parse_kv(args.model_args), gen_kwargs, args.batch_size, args.device, args.tokenizer)
    try:
        from lm_eval import evaluator  # type: ignore
    except ImportError as exc:
        raise SystemExit("lm-eval is not installed; the wrapper classes of this package implement its model interface "
                         "(loglikelihood, loglikelihood_rolling, generate_until) and can be driven directly") from exc
    results = evaluator.simple_evaluate(model=lm, tasks=args.tasks.split(","), num_fewshot=args.num_fewshot,
                                        limit=args.limit, gen_kwargs=args.gen_kwargs,
                                        apply_chat_template=args.apply_chat_template)
    if hasattr(lm, "compute_summary"):
        results["adaptive_compute"] = lm.compute_summary()
    if args.output_path:
        with open(args.output_path, "w") as f:
            json.dump(results.get("results", results), f, indent=2, default=str)
    print(json.dumps(results.get("results", results), indent=2, default=str))
    return results


def prepare_results(results: dict, save_filepath, print_results: bool = True) -> None:
    """Print the result tables (when lm-eval's table formatter is importable) and store the results as JSON
    (evaluate_raven/quick_checkpoint_eval.py:314-324)."""
    from pathlib import Path

    if print_results:
        try:
            from lm_eval.utils import make_table  # type: ignore

            print(make_table(results))
            if "groups" in results:
                print(make_table(results, "groups"))
        except ImportError:
            print(json.dumps(results.get("results", results), indent=2, default=str))
    Path(save_filepath).write_text(json.dumps(results, indent=2, ensure_ascii=False, default=str), encoding="utf-8")


def quick_eval_check(checkpoint_name: str, tokenizer_path: str, device="cuda", out_dir: str = "outputs/eval",
                     tasks: Optional[str] = "arc_easy,tinyHellaswag,tinyMMLU,piqa,openbookqa", num_fewshot: int = 0,
                     batch_size: int = 16, limit=None, seed: int = 233, recurrence: int = 32,
                     simple_evaluate=None) -> Optional[dict]:
    """Benchmark a raw TRAINING checkpoint (no conversion) at a fixed recurrence and store
    ``results_<tasks>_<checkpoint>_<recurrence>.json`` under ``out_dir``
    (evaluate_raven/quick_checkpoint_eval.py:327-390).  ``simple_evaluate`` defaults to lm-eval's; tests and callers
    without that package pass their own ``f(model=..., tasks=[...], ...) -> dict``."""
    from pathlib import Path

    from .lm_eval_wrapper import RecurrentLM

    if simple_evaluate is None:
        try:
            from lm_eval import evaluator  # type: ignore

            simple_evaluate = evaluator.simple_evaluate
        except ImportError as exc:
            raise SystemExit("lm-eval is not installed; pass simple_evaluate= or drive RecurrentLM directly") from exc
    if tasks is None:
        from lm_eval.tasks import TaskManager  # type: ignore

        print("\n".join(TaskManager().task_index.keys()))
        return None
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    model_name = str(checkpoint_name).split("/")[-1].split(".")[0]
    lm = RecurrentLM.from_checkpoint(checkpoint_name, tokenizer_path, device=device, batch_size=batch_size,
                                     recurrence=recurrence)
    results = simple_evaluate(model=lm, tasks=tasks.split(","), num_fewshot=num_fewshot, batch_size=batch_size,
                              device=str(device), limit=limit, random_seed=seed, numpy_random_seed=seed,
                              torch_random_seed=seed)
    prepare_results(results, out / f"results_{tasks}_{model_name}_{recurrence}.json")
    return results


if __name__ == "__main__":
    main()
