"""pass@k for code benchmarks: the unbiased estimator over n samples per problem, candidate assembly, and a local
runner that executes each candidate together with its test in a fresh interpreter under a time limit.

The reference delegates both to the Hugging Face ``code_eval`` metric (evaluate_raven/misc_benchmark_variants/
pass_at_k_utils.py:1-34), which needs a download; this module has no dependency.  Running model-written code is only
done when the caller asks for it (``run=True``)."""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from typing import Iterable, Optional, Sequence


def pass_at_k_estimate(n: int, c: int, k: int) -> float:
    """1 - C(n - c, k) / C(n, k): probability that at least one of k samples drawn from n (c of them correct) passes."""
    if n - c < k:
        return 1.0
    prob_all_fail = 1.0
    for i in range(n - c + 1, n + 1):
        prob_all_fail *= 1.0 - k / i
    return 1.0 - prob_all_fail


def build_predictions(resps: Sequence[Sequence[str]], docs: Sequence[dict]) -> list:
    """Prompt + completion for every sampled completion of every problem."""
    return [[doc["prompt"] + r for r in resp] for resp, doc in zip(resps, docs)]


def build_predictions_instruct(resps: Sequence[Sequence[str]], docs: Sequence[dict]) -> list:
    """As above for chat-style answers: everything from the last code fence on is cut off."""
    def cut(r: str) -> str:
        i = r.rfind("```")
        return r if i == -1 else r[:i]

    return [[doc["prompt"] + cut(r) for r in resp] for resp, doc in zip(resps, docs)]


def run_candidate(program: str, test: str, timeout_s: float = 5.0) -> bool:
    """True when ``program`` followed by ``test`` exits with status 0 in a separate interpreter."""
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "candidate.py")
        with open(path, "w") as f:
            f.write(program + "\n\n" + test + "\n")
        try:
            r = subprocess.run([sys.executable, "-I", path], cwd=tmp, capture_output=True, timeout=timeout_s)
            return r.returncode == 0
        except subprocess.TimeoutExpired:
            return False


def pass_at_k(references: Sequence[str], predictions: Sequence[Sequence[str]], k: Optional[Iterable[int]] = None,
              run: bool = True, timeout_s: float = 5.0, correct_counts: Optional[Sequence[int]] = None) -> dict:
    """``{"pass@k": mean estimate}`` for every k; ``references`` are test snippets, ``predictions[i]`` the candidate
    programs of problem i.  With ``run=False`` pass ``correct_counts`` (how many candidates of each problem passed)."""
    ks = [k] if isinstance(k, int) else list(k or [1])
    if correct_counts is None:
        if not run:
            raise ValueError("either run the candidates or pass correct_counts")
        correct_counts = [sum(run_candidate(p, ref, timeout_s) for p in preds)
                          for ref, preds in zip(references, predictions)]
    out = {}
    for kk in ks:
        vals = [pass_at_k_estimate(len(preds), c, kk) for preds, c in zip(predictions, correct_counts)
                if len(preds) >= kk]
        out[f"pass@{kk}"] = sum(vals) / len(vals) if vals else float("nan")
    return out
