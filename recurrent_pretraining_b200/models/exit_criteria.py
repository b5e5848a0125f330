"""Per-recurrence exit criteria for adaptive-depth decoding.

Each criterion keeps state across the recurrence steps of one token and returns ``(exit mask [B], head outputs or
None, criterion values [B])``.  Definitions and default thresholds are those of
recpre/raven_modeling_minimal.py:2106-2307: ``kl`` (1e-3) is ``sum p_prev * (log p_prev - log p_cur)`` against the
previous step's distribution (uniform before the first step), ``minp-kl`` (1e-5) the same on min-p(0.1) filtered
probabilities, ``entropy-diff`` (1e-3), ``latent-diff`` (0.03, relative L2 change averaged over positions),
``cosine`` (1e-3), ``argmax-stability`` (5 consecutive identical argmaxes) and ``none``.  Logit-based criteria run
``ln_f -> coda -> ln_f -> lm_head`` through ``model.predict_from_latents`` at every check.
"""
from __future__ import annotations

from typing import Callable, Union

import torch
import torch.nn.functional as F


class PerIterationExitEvaluator:
    def init(self, initial_latents: torch.Tensor) -> None:
        pass

    def check(self, model, latents: torch.Tensor, aux_inputs: dict):
        raise NotImplementedError


def _auto(value, default, cast=float):
    return default if value == "auto" else cast(value)


class NoOpExitEvaluator(PerIterationExitEvaluator):
    def check(self, model, latents, aux_inputs):
        B, dev = latents.shape[0], latents.device
        return torch.zeros(B, device=dev, dtype=torch.bool), None, torch.zeros(B, device=dev)


class _LogitCriterion(PerIterationExitEvaluator):
    def __init__(self, reduce: bool = True):
        self.reduce = reduce

    def _logits(self, model, latents, aux_inputs):
        out = model.predict_from_latents(latents, **aux_inputs)
        return out, (out.logits[:, -1, :] if self.reduce else out.logits)


class EntropyDiffExitEvaluator(_LogitCriterion):
    def __init__(self, exit_threshold: Union[str, float] = "auto", reduce: bool = True):
        super().__init__(reduce)
        self.exit_threshold = _auto(exit_threshold, 1e-3)

    def init(self, initial_latents):
        self.prev = torch.full((initial_latents.shape[0],), 100.0, device=initial_latents.device)

    def check(self, model, latents, aux_inputs):
        out, logits = self._logits(model, latents, aux_inputs)
        p = F.softmax(logits, dim=-1)
        ent = -(p * torch.log(p + 1e-10)).sum(-1)
        vals = (ent - self.prev).abs()
        self.prev = ent
        return vals < self.exit_threshold, out, vals


class KLExitEvaluator(_LogitCriterion):
    def __init__(self, model, exit_threshold: Union[str, float] = "auto", reduce: bool = True):
        super().__init__(reduce)
        self.exit_threshold = _auto(exit_threshold, 1e-3)
        self.V = model.config.padded_vocab_size

    def init(self, initial_latents):
        B = initial_latents.shape[0]
        self.prev = torch.full((B, self.V), 1.0 / self.V, device=initial_latents.device).log()

    def _logp(self, logits):
        return F.log_softmax(logits, dim=-1)

    def check(self, model, latents, aux_inputs):
        out, logits = self._logits(model, latents, aux_inputs)
        logp = self._logp(logits)
        vals = F.kl_div(logp, self.prev, reduction="none", log_target=True).sum(-1)
        self.prev = logp
        return vals < self.exit_threshold, out, vals


class MinKLExitEvaluator(KLExitEvaluator):
    def __init__(self, model, exit_threshold: Union[str, float] = "auto", reduce: bool = True):
        super().__init__(model, exit_threshold, reduce)
        self.exit_threshold = _auto(exit_threshold, 1e-5)

    def _logp(self, logits):
        p = F.softmax(logits, dim=-1)
        p = torch.where(p < 0.1 * p.max(dim=-1, keepdim=True)[0], torch.full_like(p, 1.0 / self.V), p)
        return (p / p.sum(-1, keepdim=True)).log()


class ArgmaxStabilityExitEvaluator(_LogitCriterion):
    def __init__(self, exit_threshold: Union[str, int] = "auto", reduce: bool = True):
        super().__init__(reduce)
        self.exit_threshold = _auto(exit_threshold, 5, int)

    def init(self, initial_latents):
        B, dev = initial_latents.shape[0], initial_latents.device
        self.prev = torch.full((B,), -1, dtype=torch.long, device=dev)
        self.stable = torch.zeros(B, dtype=torch.long, device=dev)

    def check(self, model, latents, aux_inputs):
        out, logits = self._logits(model, latents, aux_inputs)
        cur = logits.argmax(-1)
        self.stable = torch.where(cur == self.prev, self.stable + 1, torch.zeros_like(self.stable))
        self.prev = cur
        return self.stable >= self.exit_threshold, out, self.stable


class LatentDiffExitEvaluator(PerIterationExitEvaluator):
    def __init__(self, exit_threshold: Union[str, float] = "auto", reduce: bool = True):
        self.exit_threshold, self.reduce = _auto(exit_threshold, 0.03), reduce

    def init(self, initial_latents):
        self.prev = initial_latents.detach().clone()

    def check(self, model, latents, aux_inputs):
        vals = (latents - self.prev).float().norm(dim=-1) / latents.float().norm(dim=-1)
        if self.reduce:
            vals = vals.mean(-1)
        self.prev = latents.detach().clone()
        return vals < self.exit_threshold, None, vals


class CosineExitEvaluator(PerIterationExitEvaluator):
    def __init__(self, exit_threshold: Union[str, float] = "auto", reduce: bool = True):
        self.exit_threshold, self.reduce = _auto(exit_threshold, 1e-3), reduce

    def init(self, initial_latents):
        self.prev = initial_latents.detach().clone()

    def check(self, model, latents, aux_inputs):
        a, b = latents.float(), self.prev.float()
        cos = (a * b).sum(-1) / a.norm(dim=-1) / b.norm(dim=-1)
        if self.reduce:
            cos = cos.mean(1)
        self.prev = latents.detach().clone()
        vals = 1 - cos
        return vals < self.exit_threshold, None, vals


class NumStepsGenerator(PerIterationExitEvaluator):
    """Exit after ``steps_fn(token_index)`` recurrences: scripted per-token depth."""

    def __init__(self, steps_fn: Callable):
        self.steps_fn, self.counter, self.target, self.current = steps_fn, 0, 0, 0

    def init(self, initial_latents):
        self.target = self.steps_fn(self.counter)
        self.counter += 1
        self.current = 0

    def check(self, model, latents, aux_inputs):
        self.current += 1
        B, dev = latents.shape[0], latents.device
        return (torch.full((B,), self.current >= self.target, dtype=torch.bool, device=dev), None,
                torch.zeros(B, device=dev))


def get_adaptive_exit_evaluator(model, criterion: str, exit_threshold="auto", reduce: bool = True):
    if criterion == "entropy-diff":
        return EntropyDiffExitEvaluator(exit_threshold, reduce)
    if criterion == "latent-diff":
        return LatentDiffExitEvaluator(exit_threshold, reduce)
    if criterion == "cosine":
        return CosineExitEvaluator(exit_threshold, reduce)
    if criterion == "minp-kl":
        return MinKLExitEvaluator(model, exit_threshold, reduce)
    if "kl" in criterion:
        return KLExitEvaluator(model, exit_threshold, reduce)
    if criterion == "argmax-stability":
        return ArgmaxStabilityExitEvaluator(exit_threshold, reduce)
    if criterion == "none":
        return NoOpExitEvaluator()
    raise ValueError(f"Invalid adaptive compute strategy: {criterion}")
