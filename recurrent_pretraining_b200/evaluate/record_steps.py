"""Histogram of the recurrence steps that adaptive decoding actually spends, collected while some other code (a
benchmark harness) calls ``model.generate``.

Counterpart of evaluate_raven/record_steps_in_bench.py:30-78, which monkey-patches ``generate``; here the patch is a
context manager that restores the method on exit.
"""
from __future__ import annotations

from collections import Counter
from contextlib import contextmanager


class StepRecorder:
    def __init__(self):
        self.hist: Counter = Counter()
        self.calls = 0

    def add(self, compute_steps) -> None:
        for tok in compute_steps or []:
            for s in (tok if isinstance(tok, (list, tuple)) else [tok]):
                self.hist[int(s)] += 1

    @property
    def total(self) -> int:
        return sum(self.hist.values())

    @property
    def mean(self) -> float:
        return sum(k * v for k, v in self.hist.items()) / max(self.total, 1)

    def summary(self) -> dict:
        return {"calls": self.calls, "tokens": self.total, "mean_steps": round(self.mean, 3),
                "histogram": dict(sorted(self.hist.items()))}


@contextmanager
def record_steps(model, **forced_kwargs):
    """Inside the block every ``model.generate`` call runs with ``forced_kwargs`` added (e.g. ``criterion="kl",
    exit_threshold=5e-4``) and its per-token step counts are added to the recorder that the block receives."""
    rec = StepRecorder()
    original = model.generate

    def patched(*args, **kwargs):
        want_dict = kwargs.get("return_dict_in_generate", False)
        out = original(*args, **{**kwargs, **forced_kwargs, "return_dict_in_generate": True})
        rec.calls += 1
        scores = out.get("scores") if isinstance(out, dict) else None
        if isinstance(scores, dict):
            rec.add(scores.get("compute_steps"))
        return out if want_dict else out["sequences"]

    model.generate = patched
    try:
        yield rec
    finally:
        model.generate = original


def step_statistics(step_counts) -> dict:
    """The summary the reference attaches to every task's results (record_steps_in_bench.py:63-69)."""
    import statistics

    counts = [int(c) for c in step_counts if c > 0]          # 0 marks a padded token
    if not counts:
        raise ValueError("No steps recorded, is this an adaptive generation?")
    return {"adaptive_avg_steps": float(sum(counts) / len(counts)), "adaptive_min_steps": min(counts),
            "adaptive_max_steps": max(counts), "adaptive_std_steps": float(statistics.pstdev(counts)),
            "adaptive_total_tokens": len(counts)}


def evaluate_with_steps(model, tasks, model_args=None, simple_evaluate=None, **kwargs):
    """Run a benchmark harness over ``model`` (a scoring wrapper whose ``.model`` / ``._model`` is the network) and
    collect the adaptive-compute steps of every generated token in the same pass; the statistics are added to each
    task's results.  Returns ``(results, step_counts)``.  ``simple_evaluate`` defaults to lm-eval's."""
    if simple_evaluate is None:
        try:
            from lm_eval import simple_evaluate  # type: ignore
        except ImportError as exc:
            raise SystemExit("lm-eval is not installed; pass simple_evaluate=") from exc
    net = getattr(model, "_model", None) or getattr(model, "model", model)
    with record_steps(net) as rec:
        results = simple_evaluate(model, model_args=model_args, tasks=tasks, **kwargs)
    counts = [s for s, n in sorted(rec.hist.items()) for _ in range(n)]
    if results is not None:
        stats = step_statistics(counts)
        for task in results.get("results", {}):
            results["results"][task].update(stats)
    return results, counts


def save_step_histogram(step_counts, filename: str) -> str:
    """Histogram of the step counts: a PNG when matplotlib is importable, otherwise (or for a ``.json`` / ``.txt`` name)
    the bin counts as JSON."""
    import json

    hist = Counter(int(c) for c in step_counts)
    if not filename.endswith((".json", ".txt")):
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt

            mean = sum(k * v for k, v in hist.items()) / max(sum(hist.values()), 1)
            plt.figure(figsize=(10, 6))
            plt.bar(sorted(hist), [hist[k] for k in sorted(hist)], alpha=0.7, edgecolor="black")
            plt.xlabel("Number of Steps")
            plt.ylabel("Frequency")
            plt.title(f"Distribution of Adaptive Computation Steps\nMean: {mean:.2f}")
            plt.grid(True, alpha=0.3)
            plt.savefig(filename, dpi=300, bbox_inches="tight")
            plt.close()
            return filename
        except ImportError:
            filename = filename.rsplit(".", 1)[0] + ".json"
    with open(filename, "w") as f:
        json.dump({str(k): hist[k] for k in sorted(hist)}, f, indent=1)
    return filename


def parse_gen_kwargs(gen_kwargs_str) -> dict:
    """``key1=val1,key2=val2`` -> dict with booleans and numbers converted (record_steps_in_bench.py:90-110)."""
    from .local_lm_eval import parse_kv

    return parse_kv(gen_kwargs_str)
