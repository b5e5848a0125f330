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
