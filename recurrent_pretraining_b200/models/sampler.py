"""Sampling of the per-step recurrence pair (n no-grad iterations, k grad iterations).

Contract (recpre/model_dynamic.py:1249-1351): the pair is a pure function of the scheme name,
(mean_recurrence, mean_backprop_depth), the micro-batch step counter and -- unless the scheme
is in lock-step -- the rank.  Two CPU generators seeded ``(514229 + step) * (rank+1)`` and
``(317811 + step) * (rank+1)`` (mod 2^31-1) drive n and k, so a run can be resumed or
re-executed (activation recompute) with identical depths.  Evaluation always uses
``(mean_recurrence, 0)``.
"""
from __future__ import annotations

import math

import torch

_MOD = 2**31 - 1

SCHEMES = (
    "bptt", "non-uniform", "gupta", "simple", "poisson-lognormal-filling", "poisson-lognormal-fill",
    "poisson-lognormal", "poisson-unbounded", "poisson-fill", "poisson-bounded", "negative-binomial", "sobol",
    "geometric", "fixed", "non-recurrent", "full",
)


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed % _MOD)
    return g


def sample_gamma(alpha, beta):
    """Gamma(alpha, rate beta) by the Marsaglia-Tsang squeeze on the global generator (alpha < 1 through the
    alpha + 1 boost), drawing the same random numbers in the same order as recpre/model_dynamic.py:1465-1482."""
    if alpha < 1:
        return sample_gamma(alpha + 1, beta) * torch.rand(1).pow(1 / alpha)
    d = alpha - 1 / 3
    c = 1 / math.sqrt(9 * d)
    while True:
        x = torch.randn(1)
        v = (1 + c * x) ** 3
        u = torch.rand(1)
        if u < 1 - 0.0331 * x ** 4:
            return d * v / beta
        if torch.log(u) < 0.5 * x * x + d * (1 - v + torch.log(v)):
            return d * v / beta


def sample_negative_binomial(t, target_mean):
    """Gamma-Poisson mixture whose mean is ``target_mean``: success probability p = mean / (t / 2 + mean), dispersion
    r = mean p / (1 - p) (recpre/model_dynamic.py:1485-1492)."""
    p = target_mean / (t / 2 + target_mean)
    r = target_mean * p / (1 - p)
    beta = (1 - p) / p
    return torch.poisson(sample_gamma(r, beta))


def _negative_binomial(t: float, mean: float) -> float:
    return float(sample_negative_binomial(t, mean))


def depth_targets(scheme: str, mean_recurrence: int, mean_backprop_depth: int, step: int) -> tuple[int, int]:
    """(t, s): target no-grad depth and grad depth, including the ``curriculum-N`` ramp."""
    t_full = max(mean_recurrence - mean_backprop_depth, 0)
    if "curriculum-" in scheme:
        ramp = int(scheme.split("curriculum-")[1])
        if step <= ramp:
            slope = step / ramp
            return max(math.ceil(slope * (mean_recurrence - mean_backprop_depth)), 0), max(
                math.ceil(slope * mean_backprop_depth), 1)
    return t_full, mean_backprop_depth


def sample_recurrence(scheme: str, mean_recurrence: int, mean_backprop_depth: int, step: int, *, training: bool = True,
                      rank: int = 0, lockstep_n: bool = False, lockstep_k: bool = False) -> tuple[int, int]:
    """Return (n, k) as Python ints."""
    if not training:
        return int(mean_recurrence), 0
    seed_n, seed_k = 514229 + step, 317811 + step
    if not lockstep_n:
        seed_n *= rank + 1
    if not lockstep_k:
        seed_k *= rank + 1
    gn, gk = _gen(seed_n), _gen(seed_k)
    t, s = depth_targets(scheme, mean_recurrence, mean_backprop_depth, step)

    def randint(lo, hi, g):
        return int(torch.randint(low=lo, high=hi, size=(1,), generator=g))

    def poisson(rate, g):
        return float(torch.poisson(torch.tensor([rate], dtype=torch.float), generator=g))

    def lognormal_rate(mean_total, g):
        sigma = 0.5
        mu = math.log(mean_total) - sigma**2 / 2
        return float(torch.zeros((1,)).log_normal_(mean=mu, std=sigma, generator=g))

    # the order of the tests matters: names are matched by substring, longest first
    if "bptt" in scheme:
        n = randint(0, t * 2, gn)
        k = randint(1, 1 + min(t * 2 - n, s * 2), gk)
    elif "non-uniform" in scheme:
        total = randint(0, 2 * t, gn)
        k = randint(1, 2 * min(t, s) + 1, gk)
        n = max(total - k, 0)
    elif "gupta" in scheme:
        n = randint(0, t * 2, gn)
        draw = torch.rand(size=(1,), generator=gk)
        skew = torch.randint(low=2 * t, high=t * 8, size=(1,), generator=gk)
        k = int((1 + (t - n) * draw**skew).to(torch.long))  # float32 arithmetic, truncated toward zero
    elif "simple" in scheme:
        n = randint(0, 2 * t, gn)
        k = randint(1, 2 * s + 1, gk)
    elif "poisson-lognormal-filling" in scheme:
        p = poisson(lognormal_rate(t + s, gn), gn) + 1
        n, k = max(p - s, 0), min(s, p)
    elif "poisson-lognormal-fill" in scheme:
        n, k = poisson(lognormal_rate(t, gn), gn), s
    elif "poisson-lognormal" in scheme:
        n = poisson(lognormal_rate(t, gn), gn)
        k = randint(1, 2 * s + 1, gk)
    elif "poisson-unbounded" in scheme:
        n = poisson(t, gn)
        k = randint(1, 2 * s + 1, gk)
    elif "poisson-fill" in scheme:
        n, k = poisson(t, gn), s
    elif "poisson-bounded" in scheme:
        n = min(poisson(t, gn), 2 * t - 1)
        k = randint(1, 2 * s + 1, gk)
    elif "negative-binomial" in scheme:
        n = _negative_binomial(2 * t, t)
        k = int(torch.randint(1, 2 * s + 1, (1,)))
    elif "sobol" in scheme:
        eng = torch.quasirandom.SobolEngine(dimension=2, scramble=True, seed=seed_n)
        a, b = eng.draw(1).flatten().tolist()
        n, k = int(a * 2 * t), int(b * 2 * s + 1)
    elif "geometric" in scheme:
        n = float(torch.as_tensor(1.0).geometric_(1 / t, generator=gn))
        k = randint(1, 2 * s + 1, gk)
    elif "fixed" in scheme:
        n, k = t, s
    elif "non-recurrent" in scheme:
        n, k = 0, 1
    elif "full" in scheme:
        n, k = 0, randint(1, 2 * s + 1, gk)
    else:
        raise ValueError(f"unknown sampling scheme {scheme!r}")
    return int(n), int(k)
