"""Benchmarks with adaptive compute: the scoring wrapper whose generation runs ``generate`` with an exit criterion
(per-token early exit from the recurrence), optional cache sharing and latent reuse, and which records how many
recurrences every generated token used.

Counterpart of evaluate_raven/misc_benchmark_variants/hf_eval_adaptive_compute.py:1-327 (that script no longer imports
in the reference tree) and of evaluate_raven/record_steps_in_bench.py.  ``exit_threshold="auto"`` picks the per-criterion
default of the exit evaluators (recpre/raven_modeling_minimal.py:2106-2307)."""
from __future__ import annotations

import json
from typing import List, Optional

import torch

from .lm_eval_wrapper import RecurrentLM

AUTO_THRESHOLDS = {"entropy-diff": 1e-3, "latent-diff": 0.03, "kl": 1e-3, "minp-kl": 1e-5, "argmax-stability": 5,
                   "cosine": 1e-3, "none": None}


class AdaptiveComputeLM(RecurrentLM):
    def __init__(self, model, tokenizer, criterion: str = "entropy-diff", exit_threshold="auto",
                 lookup_strategy: str = "full", continuous_compute: bool = False, max_steps: Optional[int] = None,
                 exit_evaluator=None, **kw):
        super().__init__(model, tokenizer, **kw)
        if not self._hf:
            raise TypeError("adaptive generation needs the HF-style model (RavenForCausalLM)")
        # a ready-made evaluator object (e.g. ``NumStepsGenerator`` with a schedule of depths per token) overrides the
        # named criterion, as in evaluate_raven/misc_benchmark_variants/eval_alternate_loops.py
        self.exit_evaluator = exit_evaluator
        if exit_evaluator is not None:
            criterion = "none"
        if criterion not in AUTO_THRESHOLDS:
            raise ValueError(f"unknown exit criterion {criterion!r}; one of {sorted(AUTO_THRESHOLDS)}")
        self.criterion = criterion
        self.exit_threshold = AUTO_THRESHOLDS[criterion] if exit_threshold in ("auto", None) else float(exit_threshold)
        self.lookup_strategy, self.continuous_compute = lookup_strategy, continuous_compute
        self.max_steps = max_steps or self.recurrence
        self.step_log: List[List[int]] = []        # per request: recurrences used by each generated token

    def gen_kwargs(self) -> dict:
        kw = dict(num_steps=self.max_steps, cache_lookup_strategy=self.lookup_strategy)
        if self.exit_evaluator is not None:
            kw["exit_evaluator"] = self.exit_evaluator
        elif self.criterion != "none":
            kw.update(criterion=self.criterion, exit_threshold=self.exit_threshold)
        if self.continuous_compute:
            kw["continuous_compute"] = True
        return kw

    @torch.no_grad()
    def generate_until(self, requests, disable_tqdm: bool = True) -> List[str]:
        res = []
        for r in requests:
            ctx, gk = r.args if hasattr(r, "args") else r
            gk = gk if isinstance(gk, dict) else {}
            until = gk.get("until", [])
            until = [until] if isinstance(until, str) else list(until)
            max_new = int(gk.get("max_gen_toks", self.max_gen_toks))
            ids = torch.tensor([self.tok_encode(ctx)[-(self.max_length - max_new):]], device=self.device)
            out = self.model.generate(ids, max_new_tokens=max_new, do_sample=False, return_dict_in_generate=True,
                                      eos_token_id=self.eot_token_id, **self.gen_kwargs())
            seq = out.sequences if hasattr(out, "sequences") else out
            steps = getattr(out, "scores", None)
            if isinstance(steps, dict):      # {"compute_steps": per token [per sequence], "exit_values": ...}
                steps = steps.get("compute_steps", [])
            row = []
            for s in (steps or []):
                s = s[0] if hasattr(s, "__len__") else s
                row.append(int(s[0] if hasattr(s, "__len__") else s))
            self.step_log.append(row)
            text = self.tok_decode(seq[0, ids.shape[1]:].tolist())
            for u in until:
                if u and u in text:
                    text = text.split(u)[0]
            res.append(text)
        return res

    def compute_summary(self) -> dict:
        flat = [s for row in self.step_log for s in row]
        if not flat:
            return {"tokens": 0}
        t = torch.tensor(flat, dtype=torch.float32)
        hist = torch.bincount(t.long(), minlength=self.max_steps + 1).tolist()
        return {"tokens": len(flat), "mean_steps": float(t.mean()), "median_steps": float(t.median()),
                "max_steps": int(t.max()), "histogram": hist,
                "compute_saved_vs_fixed": 1.0 - float(t.mean()) / self.max_steps}

    def dump(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"criterion": self.criterion, "exit_threshold": self.exit_threshold,
                       "lookup_strategy": self.lookup_strategy, "summary": self.compute_summary(),
                       "steps": self.step_log}, f)
