"""Learning-rate and batch-size schedules (train.py:831-862 of the reference)."""
from __future__ import annotations

import math


def get_lr(base_lr, step, warmup_steps=0, max_steps: int = 0, cooldown_steps: int = 0, schedule: str = "cosine",
           min_lr: float = 0.0) -> float:
    """Linear warm-up, then cosine | linear | constant/trapezoid, then a linear cool-down that never goes below
    ``min_lr``; past ``max_steps`` the rate is ``min_lr``.  ``step`` counts micro-batch steps, as in the reference.

    Two call forms: ``get_lr(base_lr, step, warmup_steps, max_steps, cooldown_steps, schedule, min_lr)`` and the
    reference's ``get_lr(step, max_steps, cfg)`` with a settings object (``optim_config["lr"]``, ``warmup_steps``,
    ``cooldown_steps``, ``lr_schedule``, ``min_lr``)."""
    if hasattr(warmup_steps, "optim_config"):
        cfg, step, max_steps = warmup_steps, base_lr, step
        base_lr, warmup_steps, cooldown_steps = cfg.optim_config["lr"], cfg.warmup_steps, cfg.cooldown_steps
        schedule, min_lr = cfg.lr_schedule, cfg.min_lr
    if warmup_steps and step < warmup_steps:
        return base_lr * step / warmup_steps
    if cooldown_steps and step > max_steps - cooldown_steps:
        return max(base_lr * (max_steps - step) / cooldown_steps, min_lr)
    if step > max_steps:
        return min_lr
    frac = (step - warmup_steps) / max(max_steps - warmup_steps, 1)
    if schedule == "linear":
        return base_lr - frac * (base_lr - min_lr)
    if schedule in ("constant", "trapezoid"):
        return base_lr
    if schedule == "cosine":
        return min_lr + (base_lr - min_lr) * (1 + math.cos(math.pi * min(max(frac, 0.0), 1.0))) / 2
    raise ValueError(f"Unsupported lr_schedule: {schedule}")


def get_batch_size(step: int, batch_size_ramp=0, final_accumulation: int = 1) -> int:
    """Gradient-accumulation steps during a linear batch-size ramp (train.py:856-862): ``get_batch_size(step, ramp,
    final_accumulation)`` or the reference's ``get_batch_size(step, cfg)`` (``batch_size_ramp``, ``batch_size``,
    ``micro_batch_size``).  Never below one accumulation step (the reference's formula gives zero at step 0)."""
    ratio = None
    if hasattr(batch_size_ramp, "batch_size_ramp"):
        cfg = batch_size_ramp
        batch_size_ramp, final_accumulation = cfg.batch_size_ramp, cfg.batch_size // cfg.micro_batch_size
        ratio = cfg.batch_size / cfg.micro_batch_size
    if batch_size_ramp and step <= batch_size_ramp:
        return max(math.ceil(step / batch_size_ramp * (ratio if ratio is not None else final_accumulation)), 1)
    return final_accumulation
